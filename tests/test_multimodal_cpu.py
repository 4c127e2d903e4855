"""Multimodal pipelines: DSP round trips, fusion layers, tokenizer, CTC decoding, DDIM sampling."""
import math

import torch
import torch.nn as nn

from mythos_b200.apps import multimodal as mm
from mythos_b200.models import encoders as enc


def test_mel_spectrogram_peaks_at_the_tone_and_griffin_lim_keeps_it():
    sr = 8000
    t = torch.arange(sr) / sr
    wave = torch.sin(2 * math.pi * 1000.0 * t)
    mel = mm.MelSpectrogram(sample_rate=sr, n_mels=40, n_fft=512, hop=128)
    m = mel.compute(wave)
    assert m.shape[0] == 1 and m.shape[1] == 40
    peak = int(m[0].mean(dim=1).argmax())
    centre = mm.mel_to_hz(mm.hz_to_mel(0) + (peak + 1) * (mm.hz_to_mel(sr / 2) - mm.hz_to_mel(0)) / 41)
    assert abs(centre - 1000.0) < 150.0
    assert torch.allclose(mel.filterbank.sum(dim=1) > 0, torch.ones(40, dtype=torch.bool))
    back = mm.AudioSynthesizer(mel, iters=8).synthesize(m)
    m2 = mel.compute(back[0])
    assert int(m2[0].mean(dim=1).argmax()) == peak


def test_fusion_perceiver_alignment_and_modality_moe():
    torch.manual_seed(0)
    a, b = torch.randn(2, 5, 16), torch.randn(2, 3, 16)
    assert mm.CrossModalFusion(16, 2)([a, b]).shape == (2, 8, 16)
    assert mm.Perceiver(16, 4, 2)(a).shape == (2, 4, 16)
    assert mm.JointMultimodalModel(16, 2)(a, b).shape == (2, 16)
    al = mm.CrossModalAlignment(0.07)
    e = torch.randn(6, 8)
    assert float(al.contrastive_loss(e, e)) < float(al.contrastive_loss(e, torch.randn(6, 8)))
    assert mm.VisionMoE(16)(a).shape == a.shape
    assert mm.VisionTextMoE(16)(a, b).shape == (2, 8, 16)
    out = mm.AllModalityMoE(16)(a, b, a)
    out.sum().backward()
    assert out.shape == (2, 13, 16)


def test_tokenizer_and_ctc():
    tok = mm.MultiModalTokenizer()
    ids = tok.encode("héllo")
    assert tok.decode(ids) == "héllo"
    img = tok.encode_image(torch.rand(3, 32, 32))
    assert img[0] == 30000 and img[-1] == 30000 and len(img) == 6 and all(30000 <= t < 31000 for t in img)
    aud = tok.encode_audio(torch.randn(1, 1600))
    assert len(aud) == 6 and all(31000 <= t < 32000 for t in aud)
    assert tok.decode(ids + img) == "héllo"
    logits = torch.full((6, 4), -5.0)
    for t, c in enumerate([1, 1, 0, 1, 2, 2]):
        logits[t, c] = 5.0
    assert mm.ctc_greedy(logits) == [1, 1, 2]


def test_pipelines_run_end_to_end():
    torch.manual_seed(1)
    vit = enc.ViTEncoder(img_size=16, patch_size=8, hidden=16, layers=1, heads=2)
    clf = mm.ImageNetClassifier(vit, 16, n_classes=5)
    img = torch.randn(2, 3, 16, 16)
    assert clf.classify(img).shape == (2, 5)
    assert 0.0 <= clf.evaluate([(img, torch.tensor([0, 1]))]) <= 1.0
    ocr = mm.OCRPipeline(enc.OCREncoder(hidden=16, layers=1, heads=2), 16)
    assert isinstance(ocr.recognize(torch.randn(1, 3, 16, 64)), str)
    mel = mm.MelSpectrogram(sample_rate=8000, n_mels=16, n_fft=256, hop=64)
    asr = mm.SpeechRecognizer(enc.AudioEncoder(n_mels=16, hidden=16, layers=1, heads=2), 16, mel=mel)
    assert isinstance(asr.transcribe(torch.randn(4000)), str)

    class TinyDecoder(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed_tokens = nn.Embedding(300, 16)
            self.out = nn.Linear(16, 300)

        def forward_embeddings(self, x):
            return self.out(x.cumsum(dim=1))

    cap = mm.ImageCaptioning(vit, TinyDecoder(), 16, 16)
    assert isinstance(cap.caption(img[:1], max_tokens=4), str)
    vqa = mm.VisualQA(vit, TinyDecoder(), 16, 16)
    assert isinstance(vqa.answer(img[:1], "what?", max_tokens=3), str)


def test_ddim_sampler_is_deterministic_and_prompt_dependent():
    t2i = mm.TextToImage(latent_dim=8, image_size=16)
    a = t2i.generate("a red square", steps=5)
    b = t2i.generate("a red square", steps=5)
    c = t2i.generate("a blue circle", steps=5)
    assert a.shape == (3, 16, 16) and torch.equal(a, b) and not torch.equal(a, c)
    assert float(a.min()) >= 0.0 and float(a.max()) <= 1.0
