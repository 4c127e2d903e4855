"""Multimodal pipelines on top of the encoders and the language model.

Signal processing (mel spectrogram, Griffin-Lim), fusion layers (cross-modal attention, Perceiver,
contrastive alignment, per-modality MoEs), a unified tokenizer, and the task pipelines (image
classification, CTC speech recognition, OCR, captioning, VQA, video description, DDIM sampling).
Everything is torch code that runs on CPU or GPU tensors; the heavy encoders it drives use the
framework's CUDA kernels (see ``models/encoders.py``).

Reference counterparts: src/multimodal.cpp (``CrossModalAttention``, ``JointMultimodalModel``,
``ImageNetClassifier``, ``SpeechRecognizer`` CTC-greedy, ``OCRPipeline``, ``VideoUnderstanding``,
``ImageCaptioning``, ``VisualQA``, ``TextToImage`` :400-483 (DDIM loop around a 5-point Laplacian
"noise predictor"), ``AudioSynthesizer`` :490-555 (Griffin-Lim with an O(n^2) DFT),
``MelSpectrogram`` :566-621, ``AudioFeatureExtractor``, ``MultiModalTokenizer``, ``ModalityEncoder``,
``CrossModalAlignment`` (InfoNCE), ``Perceiver``, Vision/Audio/VisionText/AudioText/AllModality
MoE). FFTs replace the quadratic DFTs.
"""
from __future__ import annotations

import hashlib
import math

import torch
import torch.nn as nn
import torch.nn.functional as tF

from ..models.moe_variants import ExpertFFN, moe_dispatch_batched, softmax_with_topk

# --------------------------------------------------------------------------- audio DSP


def hz_to_mel(f):
    return 2595.0 * math.log10(1.0 + f / 700.0)


def mel_to_hz(m):
    return 700.0 * (10.0 ** (m / 2595.0) - 1.0)


class MelSpectrogram:
    """Hann-windowed STFT power -> triangular mel filterbank -> log. waveform [C, N] or [N]."""

    def __init__(self, sample_rate: int = 22050, n_mels: int = 80, n_fft: int = 1024, hop: int = 256):
        self.sample_rate, self.n_mels, self.n_fft, self.hop = sample_rate, n_mels, n_fft, hop
        self.filterbank = self.mel_filterbank(n_mels, n_fft)

    def mel_filterbank(self, n_filters: int, fft_size: int) -> torch.Tensor:
        bins = fft_size // 2 + 1
        pts = torch.linspace(hz_to_mel(0.0), hz_to_mel(self.sample_rate / 2), n_filters + 2)
        hz = torch.tensor([mel_to_hz(float(m)) for m in pts])
        idx = torch.floor((fft_size + 1) * hz / self.sample_rate).long().clamp_max(bins - 1)
        fb = torch.zeros(n_filters, bins)
        for m in range(1, n_filters + 1):
            lo, c, hi = int(idx[m - 1]), int(idx[m]), int(idx[m + 1])
            for k in range(lo, c):
                fb[m - 1, k] = (k - lo) / max(1, c - lo)
            for k in range(c, hi):
                fb[m - 1, k] = (hi - k) / max(1, hi - c)
        return fb

    def stft_power(self, waveform: torch.Tensor) -> torch.Tensor:
        w = waveform if waveform.dim() == 2 else waveform[None]
        win = torch.hann_window(self.n_fft, device=w.device)
        spec = torch.stft(w.float(), self.n_fft, self.hop, window=win, return_complex=True, center=True)
        return spec.abs() ** 2                                  # [C, bins, frames]

    def compute(self, waveform: torch.Tensor) -> torch.Tensor:
        p = self.stft_power(waveform)
        mel = self.filterbank.to(p.device) @ p
        return torch.log(mel.clamp_min(1e-10))                  # [C, n_mels, frames]


class AudioSynthesizer:
    """Mel (log) spectrogram -> waveform: pseudo-inverse of the filterbank, then Griffin-Lim phase
    reconstruction."""

    def __init__(self, mel: MelSpectrogram | None = None, iters: int = 32):
        self.mel = mel or MelSpectrogram()
        self.iters = iters

    def synthesize(self, mel_spectrogram: torch.Tensor) -> torch.Tensor:
        m = mel_spectrogram if mel_spectrogram.dim() == 3 else mel_spectrogram[None]
        fb = self.mel.filterbank.to(m.device)
        mag = (torch.linalg.pinv(fb) @ torch.exp(m.float())).clamp_min(0).sqrt()        # [C, bins, frames]
        win = torch.hann_window(self.mel.n_fft, device=m.device)
        g = torch.Generator(device="cpu").manual_seed(0)
        phase = torch.exp(2j * math.pi * torch.rand(mag.shape, generator=g).to(m.device))
        for _ in range(self.iters):
            wav = torch.istft(mag * phase, self.mel.n_fft, self.mel.hop, window=win, center=True)
            spec = torch.stft(wav, self.mel.n_fft, self.mel.hop, window=win, return_complex=True, center=True)
            spec = spec[..., : mag.shape[-1]]
            if spec.shape[-1] < mag.shape[-1]:
                spec = tF.pad(spec, (0, mag.shape[-1] - spec.shape[-1]))
            phase = spec / spec.abs().clamp_min(1e-8)
        return torch.istft(mag * phase, self.mel.n_fft, self.mel.hop, window=win, center=True)


class AudioFeatureExtractor:
    """waveform -> mel -> audio encoder -> frame features."""

    def __init__(self, encoder: nn.Module, mel: MelSpectrogram | None = None):
        self.encoder, self.mel = encoder, mel or MelSpectrogram(n_mels=getattr(encoder.proj, "in_features", 80))

    def extract(self, audio: torch.Tensor) -> torch.Tensor:
        m = self.mel.compute(audio)
        return self.encoder(m.to(next(self.encoder.parameters()).dtype))


# --------------------------------------------------------------------------- fusion layers


class CrossModalFusion(nn.Module):
    """Every modality stream attends over the concatenation of all streams; returns the fused
    streams concatenated along the sequence."""

    def __init__(self, hidden: int, heads: int = 4):
        super().__init__()
        self.attn = nn.MultiheadAttention(hidden, heads, batch_first=True)
        self.norm = nn.LayerNorm(hidden)

    def forward(self, modalities):
        allm = torch.cat(modalities, dim=1)
        q = self.norm(allm)
        out, _ = self.attn(q, q, q, need_weights=False)
        return allm + out


class Perceiver(nn.Module):
    """Learned (or given) queries cross-attend over an arbitrary-length input: [B, N, d] -> [B, Q, d]."""

    def __init__(self, hidden: int, num_queries: int, num_heads: int):
        super().__init__()
        self.h = num_heads
        self.latents = nn.Parameter(torch.randn(1, num_queries, hidden) * 0.02)
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (nn.Linear(hidden, hidden) for _ in range(4))

    def forward(self, inputs, queries=None):
        B, N, d = inputs.shape
        q = self.latents.expand(B, -1, -1) if queries is None else queries
        D = d // self.h
        qh = self.q_proj(q).view(B, -1, self.h, D).transpose(1, 2)
        kh = self.k_proj(inputs).view(B, N, self.h, D).transpose(1, 2)
        vh = self.v_proj(inputs).view(B, N, self.h, D).transpose(1, 2)
        att = torch.softmax(qh @ kh.transpose(-1, -2) / math.sqrt(D), dim=-1)
        return self.out_proj((att @ vh).transpose(1, 2).reshape(B, -1, d))


class CrossModalAlignment:
    """Symmetric InfoNCE between L2-normalised image and text embeddings."""

    def __init__(self, temperature: float = 0.07):
        self.temperature = temperature

    def align(self, image_emb, text_emb):
        a, b = tF.normalize(image_emb.float(), dim=-1), tF.normalize(text_emb.float(), dim=-1)
        return a @ b.t() / self.temperature

    def contrastive_loss(self, image_emb, text_emb):
        sim = self.align(image_emb, text_emb)
        tgt = torch.arange(sim.shape[0], device=sim.device)
        return 0.5 * (tF.cross_entropy(sim, tgt) + tF.cross_entropy(sim.t(), tgt))


class ModalityMoE(nn.Module):
    """Top-2 MoE over one or more token streams. With several streams a learned per-modality bias
    is added to the router logits of each stream (cross-modal routing)."""

    def __init__(self, hidden: int, num_experts: int = 4, n_modalities: int = 1, top_k: int = 2):
        super().__init__()
        self.top_k = top_k
        self.router = nn.Linear(hidden, num_experts, bias=False)
        self.modality_bias = nn.Parameter(torch.zeros(n_modalities, num_experts))
        self.experts = nn.ModuleList([ExpertFFN(hidden, 2 * hidden) for _ in range(num_experts)])

    def forward(self, *streams):
        outs = []
        for m, x in enumerate(streams):
            xf = x.reshape(-1, x.shape[-1])
            logits = self.router(xf) + self.modality_bias[min(m, self.modality_bias.shape[0] - 1)]
            idx, w = softmax_with_topk(logits, self.top_k)
            y, _ = moe_dispatch_batched(xf, self.experts, idx, w.to(xf.dtype))
            outs.append(x + y.view_as(x))
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)


def VisionMoE(hidden, num_experts=4):
    return ModalityMoE(hidden, num_experts, 1)


def AudioMoE(hidden, num_experts=4):
    return ModalityMoE(hidden, num_experts, 1)


def VisionTextMoE(hidden, num_experts=6):
    return ModalityMoE(hidden, num_experts, 2)


def AudioTextMoE(hidden, num_experts=6):
    return ModalityMoE(hidden, num_experts, 2)


def AllModalityMoE(hidden, num_experts=8, n_modalities=4):
    return ModalityMoE(hidden, num_experts, n_modalities)


# --------------------------------------------------------------------------- tokenizer


class MultiModalTokenizer:
    """Text through BPE (bytes when no BPE is given); images and audio as runs of placeholder ids
    inside reserved ranges (image patches from 30000, audio frames from 31000), bracketed by the
    range's first id."""

    IMAGE_BASE, AUDIO_BASE = 30000, 31000

    def __init__(self, bpe=None, image_codes: int = 512, audio_codes: int = 512):
        self.bpe, self.image_codes, self.audio_codes = bpe, image_codes, audio_codes

    def vocab_size(self) -> int:
        return max(self.bpe.vocab_size if self.bpe is not None and hasattr(self.bpe, "vocab_size") else 256, 32000)

    def encode(self, text: str) -> list[int]:
        return list(self.bpe.encode(text)) if self.bpe is not None else list(text.encode("utf-8"))

    def decode(self, tokens) -> str:
        toks = [t for t in tokens if t < self.IMAGE_BASE]
        if self.bpe is not None:
            return self.bpe.decode(toks)
        return bytes(t for t in toks if t < 256).decode("utf-8", errors="replace")

    def _codes(self, feats: torch.Tensor, base: int, n_codes: int) -> list[int]:
        # bucket the mean intensity of each patch / frame: a fixed, training-free code book
        v = feats.float().reshape(feats.shape[0], -1).mean(dim=1)
        lo, hi = float(v.min()), float(v.max())
        q = ((v - lo) / max(hi - lo, 1e-8) * (n_codes - 2)).long() + 1
        return [base] + [base + int(c) for c in q] + [base]

    def encode_image(self, image: torch.Tensor, patch: int = 16) -> list[int]:
        C, H, W = image.shape
        p = image[:, : H // patch * patch, : W // patch * patch].reshape(C, H // patch, patch, W // patch, patch)
        return self._codes(p.permute(1, 3, 0, 2, 4).reshape(-1, C * patch * patch), self.IMAGE_BASE, self.image_codes)

    def encode_audio(self, audio: torch.Tensor, frame: int = 400) -> list[int]:
        a = audio.reshape(-1)
        n = a.numel() // frame
        return self._codes(a[: n * frame].reshape(n, frame).abs(), self.AUDIO_BASE, self.audio_codes)


class ModalityEncoder:
    def __init__(self, model: nn.Module, modality: str):
        self.model, self.modality = model, modality

    def encode(self, x):
        with torch.no_grad():
            return self.model(x)


# --------------------------------------------------------------------------- task pipelines


class ImageNetClassifier(nn.Module):
    def __init__(self, vit: nn.Module, hidden: int, n_classes: int = 1000):
        super().__init__()
        self.vit = vit
        self.head = nn.Linear(hidden, n_classes)

    def classify(self, image):
        return self.head(self.vit(image)[:, 0])

    forward = classify

    @torch.no_grad()
    def evaluate(self, loader) -> float:
        ok = n = 0
        for img, label in loader:
            ok += int((self.classify(img).argmax(-1) == label).sum())
            n += label.numel()
        return ok / max(n, 1)


def ctc_greedy(logits: torch.Tensor, blank: int = 0) -> list[int]:
    """Collapse repeats, drop blanks. logits [T, V]."""
    ids = logits.argmax(-1).tolist()
    out, prev = [], None
    for i in ids:
        if i != prev and i != blank:
            out.append(i)
        prev = i
    return out


class _CTCPipeline(nn.Module):
    def __init__(self, encoder: nn.Module, hidden: int, alphabet: str):
        super().__init__()
        self.encoder = encoder
        self.alphabet = alphabet
        self.head = nn.Linear(hidden, len(alphabet) + 1)          # index 0 = blank

    def _text(self, feats) -> str:
        return "".join(self.alphabet[i - 1] for i in ctc_greedy(self.head(feats[0])))


class SpeechRecognizer(_CTCPipeline):
    def __init__(self, audio_encoder, hidden, alphabet="abcdefghijklmnopqrstuvwxyz '", mel: MelSpectrogram | None = None):
        super().__init__(audio_encoder, hidden, alphabet)
        self.mel = mel

    @torch.no_grad()
    def transcribe(self, audio) -> str:
        feats = self.encoder(self.mel.compute(audio) if self.mel is not None else audio)
        return self._text(feats)


class OCRPipeline(_CTCPipeline):
    def __init__(self, ocr_encoder, hidden, alphabet="abcdefghijklmnopqrstuvwxyz0123456789 .,"):
        super().__init__(ocr_encoder, hidden, alphabet)

    @torch.no_grad()
    def recognize(self, image) -> str:
        return self._text(self.encoder(image))


class _PrefixGenerator(nn.Module):
    """Encoder features are projected into the decoder's embedding space and prepended to the
    text prompt; the decoder (any module mapping embeddings [B, S, d] -> logits [B, S, V] through
    ``forward_embeddings``, or token ids through ``__call__`` when there is no prefix) decodes
    greedily."""

    def __init__(self, encoder, decoder, enc_hidden: int, dec_hidden: int, tokenizer: MultiModalTokenizer | None = None):
        super().__init__()
        self.encoder, self.decoder = encoder, decoder
        self.bridge = nn.Linear(enc_hidden, dec_hidden)
        self.tok = tokenizer or MultiModalTokenizer()

    @torch.no_grad()
    def _generate(self, features, prompt_ids, max_tokens: int, eos: int | None = None) -> list[int]:
        prefix = self.bridge(features)
        emb = self.decoder.embed_tokens
        ids = list(prompt_ids)
        out = []
        for _ in range(max_tokens):
            x = prefix if not ids else torch.cat(
                [prefix, emb(torch.tensor([ids], device=prefix.device))], dim=1)
            nxt = int(self.decoder.forward_embeddings(x)[0, -1].argmax())
            if eos is not None and nxt == eos:
                break
            ids.append(nxt)
            out.append(nxt)
        return out


class ImageCaptioning(_PrefixGenerator):
    def caption(self, image, max_tokens: int = 32) -> str:
        return self.tok.decode(self._generate(self.encoder(image), [], max_tokens))


class VisualQA(_PrefixGenerator):
    def answer(self, image, question: str, max_tokens: int = 32) -> str:
        return self.tok.decode(self._generate(self.encoder(image), self.tok.encode(question), max_tokens))


class VideoUnderstanding(_PrefixGenerator):
    def describe(self, video_frames, max_tokens: int = 32) -> str:
        return self.tok.decode(self._generate(self.encoder(video_frames), [], max_tokens))


class JointMultimodalModel(nn.Module):
    """Text, image and audio features (already encoded, same width) fused by cross-modal attention
    and mean-pooled into one joint embedding."""

    def __init__(self, hidden: int, heads: int = 4):
        super().__init__()
        self.fusion = CrossModalFusion(hidden, heads)

    def forward(self, text, image=None, audio=None):
        streams = [s for s in (text, image, audio) if s is not None]
        return self.fusion(streams).mean(dim=1)


# --------------------------------------------------------------------------- diffusion sampling


def laplacian_eps(x: torch.Tensor, t: float, cond: torch.Tensor) -> torch.Tensor:
    """Training-free stand-in for a noise predictor: the 5-point Laplacian of the sample plus a
    prompt-dependent bias (the reference's predictor)."""
    k = x.new_tensor([[0.0, 1.0, 0.0], [1.0, -4.0, 1.0], [0.0, 1.0, 0.0]])[None, None]
    C = x.shape[1]
    lap = tF.conv2d(tF.pad(x, (1, 1, 1, 1), mode="replicate"), k.expand(C, 1, 3, 3), groups=C)
    return -lap + (1.0 - t) * cond


class TextToImage:
    """Deterministic DDIM sampler (eta = 0) with a linear beta schedule. ``eps_model(x, t, cond)``
    predicts the noise; the default is :func:`laplacian_eps`."""

    def __init__(self, latent_dim: int = 64, image_size: int = 256, channels: int = 3, eps_model=None,
                 train_steps: int = 1000):
        self.latent_dim, self.image_size, self.channels = latent_dim, image_size, channels
        self.eps_model = eps_model or laplacian_eps
        betas = torch.linspace(1e-4, 0.02, train_steps)
        self.alpha_bar = torch.cumprod(1.0 - betas, dim=0)

    def _condition(self, prompt: str) -> torch.Tensor:
        h = hashlib.sha256(prompt.encode("utf-8")).digest()
        v = torch.tensor([b / 255.0 - 0.5 for b in h[: self.channels]])
        return v.view(1, self.channels, 1, 1)

    @torch.no_grad()
    def generate(self, prompt: str, steps: int = 50, device="cpu") -> torch.Tensor:
        seed = int.from_bytes(hashlib.sha256(prompt.encode("utf-8")).digest()[:4], "little")
        g = torch.Generator().manual_seed(seed)
        s = self.latent_dim
        x = torch.randn(1, self.channels, s, s, generator=g).to(device)
        cond = self._condition(prompt).to(device)
        ts = torch.linspace(len(self.alpha_bar) - 1, 0, steps).long()
        for i, t in enumerate(ts):
            ab = self.alpha_bar[t].to(device)
            ab_prev = self.alpha_bar[ts[i + 1]].to(device) if i + 1 < steps else torch.tensor(1.0, device=device)
            eps = self.eps_model(x, float(t) / len(self.alpha_bar), cond)
            x0 = ((x - (1 - ab).sqrt() * eps) / ab.sqrt()).clamp(-3, 3)
            x = ab_prev.sqrt() * x0 + (1 - ab_prev).sqrt() * eps
        img = tF.interpolate(x, size=(self.image_size, self.image_size), mode="bilinear", align_corners=False)
        return ((img.clamp(-1, 1) + 1) * 0.5)[0]
