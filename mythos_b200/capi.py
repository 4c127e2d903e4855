"""Python side of the C API (``csrc/capi/oil_c_api.cpp``): sessions that own a loaded model, its
tokenizer and (on CUDA) a persistent inference engine, so repeated ``oil_generate`` calls reuse
packed weights and the KV cache instead of rebuilding them."""
from __future__ import annotations

import os

import torch


class Session:
    def __init__(self, path: str, device: str = "auto"):
        from .oil.model_io import load_model
        from .tools.common import pick_device
        from .train.bpe import BPETokenizer

        self.device = pick_device(device)
        self.model, _ = load_model(path, device=self.device)
        self.model.eval()
        vocab = (path[:-4] if path.endswith(".oil") else path) + ".vocab"
        self.tokenizer = BPETokenizer.load(vocab) if os.path.exists(vocab) else None
        self.engine = None

    def _engine(self, need_len: int):
        from .infer.engine import InferenceEngine

        if self.engine is None or self.engine.max_seq_len < need_len:
            cap = min(self.model.cfg.max_seq_len, max(need_len, 512)) + 16
            self.engine = InferenceEngine.from_model(self.model, device=self.device, max_batch=1, max_seq_len=cap)
        return self.engine

    def generate(self, prompt: str, max_tokens: int = 64, temperature: float = 0.0, top_k: int = 0,
                 top_p: float = 1.0, seed: int = 0) -> str:
        from .infer.sampler import SamplerConfig
        from .tools.infer import generate_text

        sampler = SamplerConfig(temperature=max(0.0, temperature), top_k=max(0, top_k), top_p=top_p, seed=seed)
        if self.device.type != "cuda":
            text, _ = generate_text(self.model, self.tokenizer, prompt, max_tokens, sampler, self.device)
            return text
        tok = self.tokenizer
        ids = tok.encode(prompt) if tok is not None else list(prompt.encode("utf-8"))
        ids = [min(i, self.model.cfg.vocab_size - 1) for i in ids] or [0]
        eng = self._engine(len(ids) + max_tokens)
        room = eng.max_seq_len - len(ids)
        res = eng.generate([ids], max_new_tokens=max(1, min(max_tokens, room)), sampler=sampler,
                           use_graph=sampler.greedy)
        new = res.tokens[0]
        return tok.decode(new) if tok is not None else bytes(t & 0xFF for t in new).decode("utf-8", "replace")

    def close(self) -> None:
        self.engine = None
        self.model = None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


def load(path: str, device: str = "auto") -> Session:
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    return Session(path, device)
