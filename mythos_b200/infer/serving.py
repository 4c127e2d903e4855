"""Serving-side machinery on top of :class:`InferenceEngine`'s step-wise API.

One module for the reference's inference extras (src/inference_opt.cpp, D2-D20):

* ``ContinuousBatcher`` (D3): FIFO admission up to ``max_batch`` running sequences, one decode step
  for all of them per ``step()``, finished sequences retire and free their pages at once. Unlike the
  reference each request keeps its own paged KV state.
* ``RequestScheduler`` (D12): priority + deadline heap in front of the batcher; ``DynamicBatcher``
  (D11): groups waiting requests by a token budget.
* ``SpeculativeDecoder`` (D2): draft gamma tokens with a small model, score them with the target in
  one pass, accept with min(1, p_t/p_d), resample the first rejection from max(0, p_t - p_d),
  adapt gamma from an EMA of the acceptance rate.
* ``beam_search`` (D6 ``TreeDecoder``), ``compute_logprobs`` (D17), ``EmbeddingEndpoint`` (D18,
  mean-pooled final hidden states), ``Reranker`` (D19, query-document log-likelihood),
  ``GrammarDecoder`` (D20, token allow-mask from a user callback), ``ModelShard`` (D10, run a layer
  range — the pipeline-parallel stage).
"""
from __future__ import annotations

import heapq
import itertools
import math
import time
from dataclasses import dataclass, field

import torch

from .sampler import SamplerConfig, sample


@dataclass
class Request:
    prompt: list
    max_new_tokens: int = 64
    sampler: SamplerConfig = field(default_factory=lambda: SamplerConfig(temperature=0.0))
    priority: int = 0
    deadline: float = math.inf
    eos_id: int | None = None
    request_id: int = 0
    # filled while running
    seq: int = -1
    output: list = field(default_factory=list)
    submitted: float = 0.0
    first_token_at: float = 0.0
    finished_at: float = 0.0


class RequestScheduler:
    """Highest priority first, then earliest deadline, then arrival order."""

    def __init__(self):
        self._heap = []
        self._count = itertools.count()

    def push(self, req: Request) -> None:
        heapq.heappush(self._heap, (-req.priority, req.deadline, next(self._count), req))

    def pop(self) -> Request | None:
        now = time.time()
        while self._heap:
            _, deadline, _, req = heapq.heappop(self._heap)
            if deadline >= now:
                return req
            req.finished_at = now  # expired before it could start
        return None

    def __len__(self):
        return len(self._heap)


class DynamicBatcher:
    """Collect requests until the token budget or the batch limit is reached."""

    def __init__(self, max_batch: int = 64, max_tokens: int = 65536):
        self.max_batch, self.max_tokens = max_batch, max_tokens

    def take(self, scheduler: RequestScheduler) -> list[Request]:
        batch, tokens = [], 0
        while len(batch) < self.max_batch and len(scheduler):
            req = scheduler.pop()
            if req is None:
                break
            need = len(req.prompt) + req.max_new_tokens
            if batch and tokens + need > self.max_tokens:
                scheduler.push(req)
                break
            batch.append(req)
            tokens += need
        return batch


class ContinuousBatcher:
    def __init__(self, engine, max_batch: int | None = None):
        self.engine = engine
        self.max_batch = max_batch or engine.max_batch
        self.scheduler = RequestScheduler()
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self._ids = itertools.count(1)
        self._next_token: dict[int, int] = {}

    def submit(self, prompt, **kw) -> Request:
        req = Request(prompt=list(prompt), request_id=next(self._ids), submitted=time.time(), **kw)
        self.scheduler.push(req)
        return req

    def _admit(self) -> None:
        while len(self.running) < self.max_batch and len(self.scheduler):
            req = self.scheduler.pop()
            if req is None:
                break
            req.seq, logits = self.engine.start_sequence(req.prompt)
            tok = int(sample(logits, req.sampler, step=0)[0])
            req.output.append(tok)
            req.first_token_at = time.time()
            self._next_token[req.request_id] = tok
            self.running.append(req)

    def step(self) -> int:
        """Admit waiting requests, decode one token for every running one. Returns the number of
        tokens produced."""
        self._admit()
        live = [r for r in self.running if not self._done(r)]
        produced = 0
        if live:
            logits = self.engine.decode([r.seq for r in live], [self._next_token[r.request_id] for r in live])
            for i, r in enumerate(live):
                tok = int(sample(logits[i:i + 1], r.sampler, step=len(r.output))[0])
                r.output.append(tok)
                self._next_token[r.request_id] = tok
                produced += 1
        for r in list(self.running):
            if self._done(r):
                self.engine.release(r.seq)
                r.finished_at = time.time()
                self.running.remove(r)
                self.finished.append(r)
                self._next_token.pop(r.request_id, None)
        return produced

    @staticmethod
    def _done(r: Request) -> bool:
        return len(r.output) >= r.max_new_tokens or (r.eos_id is not None and r.output and r.output[-1] == r.eos_id)

    def run_until_idle(self, max_steps: int = 1 << 20) -> list[Request]:
        for _ in range(max_steps):
            if not self.running and not len(self.scheduler):
                break
            self.step()
        return self.finished


# --------------------------------------------------------------------------------------- model-level helpers
@torch.no_grad()
def _logits_full(model, ids: torch.Tensor) -> torch.Tensor:
    dev = next(model.parameters()).device
    return model(ids.to(dev, torch.int32)).float()


@torch.no_grad()
def compute_logprobs(model, ids) -> torch.Tensor:
    """log p(token_t | tokens_<t) for t >= 1 of one sequence."""
    ids = torch.as_tensor(ids, dtype=torch.int32)[None]
    lp = torch.log_softmax(_logits_full(model, ids[:, :-1]), dim=-1)[0]
    return lp.gather(1, ids[0, 1:].long()[:, None].to(lp.device)).squeeze(1).cpu()


class SpeculativeDecoder:
    def __init__(self, target, draft, gamma: int = 4, adaptive: bool = True):
        self.target, self.draft, self.gamma, self.adaptive = target, draft, gamma, adaptive
        self.accept_ema = 0.7
        self.stats = {"proposed": 0, "accepted": 0}

    @torch.no_grad()
    def generate(self, prompt, max_new_tokens: int, temperature: float = 1.0, seed: int = 0) -> list[int]:
        g = torch.Generator().manual_seed(seed)
        seq = list(prompt)
        out = []
        while len(out) < max_new_tokens:
            gamma = max(1, min(self.gamma, max_new_tokens - len(out)))
            drafted, dprobs = [], []
            cur = list(seq)
            for _ in range(gamma):
                pd = torch.softmax(_logits_full(self.draft, torch.tensor([cur]))[0, -1].cpu() / max(temperature, 1e-5), -1)
                tok = int(torch.multinomial(pd, 1, generator=g)) if temperature > 1e-5 else int(pd.argmax())
                drafted.append(tok)
                dprobs.append(pd)
                cur.append(tok)
            lt = _logits_full(self.target, torch.tensor([cur]))[0].cpu() / max(temperature, 1e-5)
            pt_all = torch.softmax(lt[len(seq) - 1:], -1)  # gamma + 1 distributions
            n_ok = 0
            for i, tok in enumerate(drafted):
                pt, pd = pt_all[i], dprobs[i]
                self.stats["proposed"] += 1
                if temperature <= 1e-5:
                    ok = int(pt.argmax()) == tok
                else:
                    ok = float(torch.rand((), generator=g)) < min(1.0, float(pt[tok] / pd[tok].clamp(min=1e-20)))
                if ok:
                    n_ok += 1
                    self.stats["accepted"] += 1
                    continue
                resid = (pt - pd).clamp(min=0)
                nxt = int(pt.argmax()) if temperature <= 1e-5 or float(resid.sum()) <= 0 else int(
                    torch.multinomial(resid / resid.sum(), 1, generator=g))
                seq += drafted[:n_ok] + [nxt]
                out += drafted[:n_ok] + [nxt]
                break
            else:
                bonus = int(pt_all[gamma].argmax()) if temperature <= 1e-5 else int(
                    torch.multinomial(pt_all[gamma], 1, generator=g))
                seq += drafted + [bonus]
                out += drafted + [bonus]
            if self.adaptive:
                self.accept_ema = 0.9 * self.accept_ema + 0.1 * (n_ok / gamma)
                self.gamma = max(1, min(8, self.gamma + (1 if self.accept_ema > 0.8 else -1 if self.accept_ema < 0.4 else 0)))
        return out[:max_new_tokens]


@torch.no_grad()
def beam_search(model, prompt, max_new_tokens: int, beams: int = 4, eos_id: int | None = None,
                length_penalty: float = 1.0) -> list[tuple[list[int], float]]:
    """Returns the final beams as (tokens, score) sorted best first."""
    live = [(list(prompt), 0.0)]
    done = []
    for _ in range(max_new_tokens):
        cand = []
        for toks, score in live:
            lp = torch.log_softmax(_logits_full(model, torch.tensor([toks]))[0, -1], -1).cpu()
            top = torch.topk(lp, beams)
            for v, i in zip(top.values.tolist(), top.indices.tolist()):
                cand.append((toks + [i], score + v))
        cand.sort(key=lambda c: c[1] / (len(c[0]) ** length_penalty), reverse=True)
        live = []
        for toks, score in cand[: beams * 2]:
            if eos_id is not None and toks[-1] == eos_id:
                done.append((toks, score))
            elif len(live) < beams:
                live.append((toks, score))
        if not live:
            break
    allb = done + live
    allb.sort(key=lambda c: c[1] / (len(c[0]) ** length_penalty), reverse=True)
    n = len(prompt)
    return [(t[n:], s) for t, s in allb[:beams]]


class EmbeddingEndpoint:
    """Mean-pooled, L2-normalised final hidden states."""

    def __init__(self, model):
        self.model = model

    @torch.no_grad()
    def embed(self, ids) -> torch.Tensor:
        dev = next(self.model.parameters()).device
        h = self.model.hidden_states(torch.as_tensor(ids, dtype=torch.int32)[None].to(dev)).float()[0]
        v = h.mean(0)
        return (v / v.norm().clamp(min=1e-12)).cpu()


class Reranker:
    """Scores documents by the mean log-likelihood of the document given the query."""

    def __init__(self, model):
        self.model = model

    def score(self, query_ids, doc_ids) -> float:
        lp = compute_logprobs(self.model, list(query_ids) + list(doc_ids))
        return float(lp[len(query_ids) - 1:].mean())

    def rank(self, query_ids, docs) -> list[int]:
        scores = [self.score(query_ids, d) for d in docs]
        return sorted(range(len(docs)), key=lambda i: scores[i], reverse=True)


class GrammarDecoder:
    """Constrained greedy/sampled decoding: ``allowed(tokens_so_far) -> iterable of token ids``."""

    def __init__(self, model, allowed, vocab_size: int | None = None):
        self.model, self.allowed = model, allowed
        self.vocab = vocab_size or model.cfg.vocab_size

    @torch.no_grad()
    def generate(self, prompt, max_new_tokens: int, sampler: SamplerConfig | None = None) -> list[int]:
        sampler = sampler or SamplerConfig(temperature=0.0)
        seq, out = list(prompt), []
        dev = next(self.model.parameters()).device
        for step in range(max_new_tokens):
            logits = _logits_full(self.model, torch.tensor([seq]))[:, -1]
            mask = torch.zeros(1, self.vocab, dtype=torch.uint8, device=logits.device)
            ids = list(self.allowed(out))
            if not ids:
                break
            mask[0, torch.tensor(ids, device=logits.device)] = 1
            lg = logits.to(torch.bfloat16) if logits.is_cuda else logits
            tok = int(sample(lg.contiguous(), sampler, allow_mask=mask, step=step)[0])
            seq.append(tok)
            out.append(tok)
        return out


class ModelShard:
    """Layers [start, end) of a dense model as a callable stage (embedding on the first stage, final
    norm + head on the last): the unit of pipeline parallelism."""

    def __init__(self, model, start: int, end: int):
        self.model, self.start, self.end = model, start, end
        self.first, self.last = start == 0, end == len(model.layers)

    def __call__(self, x, stream=None, pos=None):
        m = self.model
        if self.first:
            ids = x
            B, S = ids.shape
            if pos is None:
                pos = torch.arange(S, device=ids.device, dtype=torch.int32).repeat(B)
            x, stream = m.tok_embeddings(ids), None
        for blk in m.layers[self.start:self.end]:
            x, stream = blk(x, stream, pos)
        if self.last:
            h, _ = m.norm(x, stream)
            return m.logits(h), None
        return x, stream
