"""Agentic layer around a language model: self-monitoring, reflection, verification, safety, search
and planning utilities, and the self-improvement flywheel (propose -> sandbox compile/run ->
measure -> apply or roll back -> JSONL log).

These are heuristics, as in the reference (src/asi.cpp, include/oil/asi.h: ``SelfMonitor``
entropy-based confidence, ``SelfReflector``, ``RecursiveSelfImprover``, ``CodeGenSelfImprover``
(templated kernel text + ``g++ -c``), ``SelfVerifier``, ``CapabilityAmplifier``, ``SafetyGuardrails``
(pattern block-list + kill switch), ``HITL``, ``AlignmentSystem``, ``WorldModel``,
``CuriosityDrivenExplorer``, ``MultiAgentSystem``, ``NeuralArchitectureSearch`` (evolutionary over
{layers, hidden} with an analytic score), ``HPOptimizer`` (population-based training),
``ContinuousLearner``, ``KnowledgeDistillation``, ``PromptOptimizer``, ``ChainOfThought``, ``ToolUse``,
``MemorySystem`` (cosine top-k), ``PlanningEngine``, ``EvaluationHarness``, ``Flywheel``).
Differences: knowledge distillation really updates the student (the reference computes the KL
and discards it, src/asi.cpp:1048-1101), and generated kernels are sm_100a CUDA text compiled
with ``nvcc -c`` when nvcc is present (``g++ -c`` for the C++ variant).

A "model" here is anything with ``generate_text(prompt, max_tokens) -> str`` and
``next_token_logits(text) -> Tensor[V]``; :class:`EngineTextModel` adapts the inference engine.
"""
from __future__ import annotations

import json
import math
import os
import random
import re
import shutil
import subprocess
import tempfile
import time
from dataclasses import asdict, dataclass, field

import torch


class EngineTextModel:
    """Adapter: inference engine + tokenizer -> the text interface used below."""

    def __init__(self, engine, tokenizer):
        self.engine, self.tok = engine, tokenizer

    def generate_text(self, prompt: str, max_tokens: int = 64) -> str:
        ids = self.tok.encode(prompt) or [0]
        res = self.engine.generate([ids], max_new_tokens=max_tokens, use_graph=False)
        return self.tok.decode(res.tokens[0])

    def next_token_logits(self, text: str) -> torch.Tensor:
        ids = self.tok.encode(text) or [0]
        seq, logits = self.engine.start_sequence(ids, reuse_prefix=False)
        self.engine.release(seq)
        return logits[0].float().cpu()


# --------------------------------------------------------------------------- monitoring / reflection


@dataclass
class MetaCognitionState:
    confidence: float = 0.0
    uncertainty: float = 0.0
    reasoning_depth: int = 0
    needs_reanalysis: bool = False
    recommendation: str = ""
    reasoning_chain: list = field(default_factory=list)
    token_confidences: list = field(default_factory=list)


class SelfMonitor:
    def __init__(self, model):
        self.model = model

    @staticmethod
    def estimate_confidence(logits: torch.Tensor) -> float:
        """1 - normalised entropy of the next-token distribution."""
        p = torch.softmax(logits.float().reshape(-1), dim=-1)
        h = -(p * torch.log(p.clamp_min(1e-12))).sum()
        return float(1.0 - h / math.log(max(2, p.numel())))

    def analyze(self, inp: str, out: str) -> MetaCognitionState:
        st = MetaCognitionState()
        words = out.split()
        prefix = inp
        for w in words[:16]:
            st.token_confidences.append(self.estimate_confidence(self.model.next_token_logits(prefix)))
            prefix += " " + w
        st.confidence = sum(st.token_confidences) / max(1, len(st.token_confidences))
        st.uncertainty = 1.0 - st.confidence
        st.reasoning_depth = sum(out.count(k) for k in ("because", "therefore", "so ", "step"))
        st.needs_reanalysis = st.confidence < 0.3 or not out.strip()
        st.recommendation = "re-run with a reflection pass" if st.needs_reanalysis else "accept"
        st.reasoning_chain = [s.strip() for s in re.split(r"[.\n]", out) if s.strip()][:8]
        return st


class SelfReflector:
    def __init__(self, model):
        self.model = model

    def reflect(self, inp: str, out: str) -> str:
        return self.model.generate_text(f"Question: {inp}\nAnswer: {out}\nList mistakes in the answer:", 64)

    def refine(self, original: str, reflection: str) -> str:
        return self.model.generate_text(f"Answer: {original}\nCritique: {reflection}\nImproved answer:", 64)


class RecursiveSelfImprover:
    """Evaluate -> propose a configuration change -> keep it only if the evaluation improves."""

    def __init__(self, evaluate, config: dict):
        self.evaluate, self.config = evaluate, dict(config)
        self.history = []

    def self_modify(self, analysis: str) -> dict:
        cand = dict(self.config)
        if "capacity" in analysis or "underfit" in analysis:
            cand["hidden_size"] = int(cand.get("hidden_size", 256) * 1.25) // 64 * 64 or 64
        elif "overfit" in analysis:
            cand["hidden_size"] = max(64, int(cand.get("hidden_size", 256) * 0.8) // 64 * 64)
        else:
            cand["lr"] = cand.get("lr", 3e-4) * random.Random(len(self.history)).choice([0.5, 2.0])
        return cand

    def improvement_cycle(self, iterations: int = 10) -> dict:
        best = self.evaluate(self.config)
        for i in range(iterations):
            cand = self.self_modify("underfit" if i % 2 == 0 else "lr")
            score = self.evaluate(cand)
            self.history.append((cand, score))
            if score > best:
                best, self.config = score, cand
        return self.config


# --------------------------------------------------------------------------- code generation + sandbox

_CUDA_GEMM_TEMPLATE = """// generated: C[M,N] = A[M,K] * B[N,K]^T, {M}x{N}x{K}, one 16x16 tile per block
#include <cuda_runtime.h>
extern "C" __global__ void gen_{op}(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C) {{
  __shared__ float sa[16][17], sb[16][17];
  const int row = blockIdx.y * 16 + threadIdx.y, col = blockIdx.x * 16 + threadIdx.x;
  float acc = 0.f;
  for (int k0 = 0; k0 < {K}; k0 += 16) {{
    sa[threadIdx.y][threadIdx.x] = (row < {M} && k0 + threadIdx.x < {K}) ? A[row * {K} + k0 + threadIdx.x] : 0.f;
    sb[threadIdx.y][threadIdx.x] = (blockIdx.x * 16 + threadIdx.y < {N} && k0 + threadIdx.x < {K})
        ? B[(blockIdx.x * 16 + threadIdx.y) * {K} + k0 + threadIdx.x] : 0.f;
    __syncthreads();
    for (int k = 0; k < 16; ++k) acc += sa[threadIdx.y][k] * sb[threadIdx.x][k];
    __syncthreads();
  }}
  if (row < {M} && col < {N}) C[row * {N} + col] = acc;
}}
"""

_CPP_GEMM_TEMPLATE = """// generated: C[M,N] = A[M,K] * B[N,K]^T, {M}x{N}x{K}
extern "C" void gen_{op}(const float* A, const float* B, float* C) {{
  for (int m = 0; m < {M}; ++m)
    for (int n = 0; n < {N}; ++n) {{
      float acc = 0.f;
      for (int k = 0; k < {K}; ++k) acc += A[m * {K} + k] * B[n * {K} + k];
      C[m * {N} + n] = acc;
    }}
}}
"""


class CodeGenSelfImprover:
    def __init__(self, model=None, language: str = "auto"):
        self.model = model
        self.language = ("cuda" if shutil.which("nvcc") else "cpp") if language == "auto" else language
        self.kernels: dict[str, str] = {}

    def generate_kernel(self, op: str, M: int, N: int, K: int) -> str:
        tpl = _CUDA_GEMM_TEMPLATE if self.language == "cuda" else _CPP_GEMM_TEMPLATE
        return tpl.format(op=re.sub(r"\W", "_", op), M=M, N=N, K=K)

    def compile_and_test(self, code: str, timeout: float = 120.0) -> bool:
        with tempfile.TemporaryDirectory(prefix="mythos_codegen_") as d:
            cuda = "__global__" in code
            src = os.path.join(d, "k.cu" if cuda else "k.cpp")
            with open(src, "w") as f:
                f.write(code)
            cmd = (["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-c", src, "-o", os.path.join(d, "k.o")]
                   if cuda else ["g++", "-O2", "-c", src, "-o", os.path.join(d, "k.o")])
            if shutil.which(cmd[0]) is None:
                return False
            try:
                return subprocess.run(cmd, capture_output=True, timeout=timeout).returncode == 0
            except subprocess.TimeoutExpired:
                return False

    def replace_kernel(self, op: str, new_code: str) -> bool:
        if not self.compile_and_test(new_code):
            return False
        self.kernels[op] = new_code
        return True


class SelfVerifier:
    def __init__(self, model=None):
        self.model = model

    def verify(self, problem: str, solution: str) -> bool:
        """Structural checks (balanced brackets, non-empty, no TODO markers); with a model, also asks it."""
        if not solution.strip() or "TODO" in solution:
            return False
        pairs = {"(": ")", "[": "]", "{": "}"}
        stack = []
        for ch in solution:
            if ch in pairs:
                stack.append(pairs[ch])
            elif ch in pairs.values():
                if not stack or stack.pop() != ch:
                    return False
        if stack:
            return False
        if self.model is not None:
            verdict = self.model.generate_text(f"Problem: {problem}\nSolution: {solution}\nIs it correct? yes/no:", 4)
            if verdict.strip().lower().startswith("no"):
                return False
        return True

    @staticmethod
    def find_edge_cases(solution: str) -> list[str]:
        cases = ["empty input", "single element"]
        if re.search(r"/|%", solution):
            cases.append("division by zero")
        if re.search(r"\[[^\]]+\]", solution):
            cases.append("index out of range")
        if re.search(r"\bint\b|\blong\b", solution):
            cases.append("integer overflow")
        if "float" in solution or "double" in solution:
            cases.append("NaN / infinity")
        return cases


class CapabilityAmplifier:
    """Measures a capability as the mean confidence on its probe prompts; ``improve`` runs the
    supplied training callback and reports whether the measure rose."""

    PROBES = {"arithmetic": ["2 + 2 =", "7 * 6 ="], "recall": ["The capital of France is"], "code": ["def add(a, b):"]}

    def __init__(self, model, train_fn=None):
        self.model, self.train_fn = model, train_fn

    def measure(self, capability: str) -> float:
        probes = self.PROBES.get(capability, [capability])
        return sum(SelfMonitor.estimate_confidence(self.model.next_token_logits(p)) for p in probes) / len(probes)

    def improve(self, capability: str, steps: int = 100) -> bool:
        before = self.measure(capability)
        if self.train_fn is not None:
            self.train_fn(capability, steps)
        return self.measure(capability) > before


# --------------------------------------------------------------------------- safety / alignment


class SafetyGuardrails:
    DEFAULT_PATTERNS = ("rm -rf /", "format c:", "drop table", ":(){ :|:& };:", "mkfs", "dd if=/dev/zero of=/dev/")

    def __init__(self, blocked_patterns=None):
        self.blocked_patterns = [p.lower() for p in (blocked_patterns or self.DEFAULT_PATTERNS)]
        self.kill_switch = False

    def set_kill_switch(self, kill: bool) -> None:
        self.kill_switch = kill

    def is_killed(self) -> bool:
        return self.kill_switch

    def _ok(self, text: str) -> bool:
        t = text.lower()
        return not self.kill_switch and not any(p in t for p in self.blocked_patterns)

    check_output = _ok
    check_input = _ok


class HITL:
    """Human-in-the-loop gate. Without an approver callback every request is denied while paused
    and approved otherwise."""

    def __init__(self, approver=None):
        self.paused, self.approver, self.log = False, approver, []

    def pause(self):
        self.paused = True

    def resume(self):
        self.paused = False

    def is_paused(self) -> bool:
        return self.paused

    def request_approval(self, action: str) -> bool:
        ok = (not self.paused) if self.approver is None else bool(self.approver(action))
        self.log.append((action, ok))
        return ok


class AlignmentSystem:
    max_loop_iterations = 100
    POSITIVE = ("help", "safe", "please", "thank", "explain", "careful")
    NEGATIVE = ("harm", "attack", "steal", "destroy", "deceive", "exploit")

    def value_alignment_score(self, output: str) -> float:
        t = output.lower()
        pos = sum(t.count(w) for w in self.POSITIVE)
        neg = sum(t.count(w) for w in self.NEGATIVE)
        return 0.5 if pos + neg == 0 else pos / (pos + neg)


# --------------------------------------------------------------------------- world model / exploration / agents


class WorldModel:
    """Linear-Gaussian latent dynamics ``s' = tanh(A s + B a)`` fitted by least squares from
    observed transitions; ``plan`` rolls a random-shooting search forward."""

    def __init__(self, state_dim: int, action_dim: int, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.A = torch.randn(state_dim, state_dim, generator=g) * 0.1
        self.B = torch.randn(state_dim, action_dim, generator=g) * 0.1
        self.action_dim = action_dim

    def simulate_step(self, state, action):
        return torch.tanh(self.A @ state + self.B @ action)

    def fit(self, states, actions, next_states):
        X = torch.cat([states, actions], dim=1)
        Y = torch.atanh(next_states.clamp(-0.999, 0.999))
        W = torch.linalg.lstsq(X, Y).solution.t()
        self.A, self.B = W[:, : states.shape[1]].contiguous(), W[:, states.shape[1]:].contiguous()

    def plan(self, state, goal, horizon: int = 8, candidates: int = 64, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        best, best_cost = None, float("inf")
        for _ in range(candidates):
            acts = torch.randn(horizon, self.action_dim, generator=g)
            s = state
            for a in acts:
                s = self.simulate_step(s, a)
            cost = float((s - goal).pow(2).sum())
            if cost < best_cost:
                best, best_cost = acts, cost
        return list(best)


class CuriosityDrivenExplorer:
    """Intrinsic reward = distance to the nearest visited state (novelty)."""

    def __init__(self, step_fn, n_actions: int):
        self.step_fn, self.n_actions = step_fn, n_actions
        self.visited: list[torch.Tensor] = []

    def intrinsic_reward(self, state) -> float:
        if not self.visited:
            return 1.0
        return float(torch.stack([(state - v).norm() for v in self.visited]).min())

    def explore(self, state, n_steps: int) -> list[int]:
        actions = []
        for _ in range(n_steps):
            scores = [self.intrinsic_reward(self.step_fn(state, a)) for a in range(self.n_actions)]
            a = int(max(range(self.n_actions), key=lambda i: scores[i]))
            state = self.step_fn(state, a)
            self.visited.append(state)
            actions.append(a)
        return actions


class MultiAgentSystem:
    def __init__(self, n_agents: int, policy=None):
        self.agents = [{"history": [], "state": f"agent{i}"} for i in range(n_agents)]
        self.policy = policy or (lambda agent, inbox: f"{agent['state']} ack {len(inbox)}")

    def communicate(self, src: int, dst: int) -> None:
        msg = self.agents[src]["history"][-1] if self.agents[src]["history"] else self.agents[src]["state"]
        self.agents[dst]["history"].append(f"from {src}: {msg}")

    def run_episode(self, steps: int) -> None:
        n = len(self.agents)
        for t in range(steps):
            for i, ag in enumerate(self.agents):
                ag["history"].append(self.policy(ag, ag["history"][-n:]))
                self.communicate(i, (i + 1 + t) % n)

    def get_histories(self):
        return [list(a["history"]) for a in self.agents]


# --------------------------------------------------------------------------- search / tuning


@dataclass
class Architecture:
    layers: int
    hidden: int
    score: float = 0.0


class NeuralArchitectureSearch:
    """Evolutionary search over (layers, hidden). The default score is analytic: a saturating
    quality term in the parameter count minus a cost term, peaking at a mid-size model."""

    def __init__(self, evaluate=None, seed: int = 0):
        self.rng = random.Random(seed)
        self._eval = evaluate

    def evaluate(self, a: Architecture) -> float:
        if self._eval is not None:
            return self._eval(a)
        params = 12 * a.layers * a.hidden * a.hidden
        return math.log10(params) - 2.0e-9 * params

    def mutate(self, a: Architecture) -> Architecture:
        layers = max(1, a.layers + self.rng.choice([-2, -1, 0, 1, 2]))
        hidden = max(64, (a.hidden + self.rng.choice([-128, -64, 0, 64, 128])) // 64 * 64)
        return Architecture(layers, hidden)

    def search(self, population: int = 50, generations: int = 20) -> Architecture:
        pop = [Architecture(self.rng.randint(2, 48), self.rng.randint(2, 64) * 64) for _ in range(population)]
        for _ in range(generations):
            for a in pop:
                a.score = self.evaluate(a)
            pop.sort(key=lambda a: a.score, reverse=True)
            elite = pop[: max(2, population // 4)]
            pop = elite + [self.mutate(self.rng.choice(elite)) for _ in range(population - len(elite))]
        for a in pop:
            a.score = self.evaluate(a)
        return max(pop, key=lambda a: a.score)


class HPOptimizer:
    """Population-based training over a dict of hyper-parameters: exploit (copy the best), explore
    (perturb by 0.8x / 1.25x)."""

    def __init__(self, evaluate, space: dict, seed: int = 0):
        self.evaluate, self.space, self.rng = evaluate, space, random.Random(seed)

    def population_based_training(self, n_population: int = 8, n_generations: int = 10) -> dict:
        pop = [{k: self.rng.uniform(lo, hi) for k, (lo, hi) in self.space.items()} for _ in range(n_population)]
        for _ in range(n_generations):
            scored = sorted(pop, key=self.evaluate, reverse=True)
            top = scored[: max(1, n_population // 4)]
            pop = list(top)
            while len(pop) < n_population:
                base = dict(self.rng.choice(top))
                for k, (lo, hi) in self.space.items():
                    base[k] = min(hi, max(lo, base[k] * self.rng.choice([0.8, 1.25])))
                pop.append(base)
        return max(pop, key=self.evaluate)


class ContinuousLearner:
    """Exemplar replay buffer (reservoir sampling) and a forgetting check against a reference score."""

    def __init__(self, evaluate=None, capacity: int = 1024, seed: int = 0):
        self.evaluate, self.capacity, self.rng = evaluate, capacity, random.Random(seed)
        self.exemplars: list = []
        self.seen = 0
        self.baseline = None

    def update(self, new_data) -> None:
        for x in new_data:
            self.seen += 1
            if len(self.exemplars) < self.capacity:
                self.exemplars.append(x)
            else:
                j = self.rng.randrange(self.seen)
                if j < self.capacity:
                    self.exemplars[j] = x

    def prevent_forgetting(self, threshold: float = 0.95) -> bool:
        """True when performance on the exemplars stays above ``threshold`` x the first measurement."""
        if self.evaluate is None or not self.exemplars:
            return True
        score = self.evaluate(self.exemplars)
        if self.baseline is None:
            self.baseline = score
        return score >= threshold * self.baseline


class KnowledgeDistillation:
    """Student matches the teacher's softened distribution: ``T^2 * KL(p_T || p_S)`` (+ optional
    hard-label CE), with real optimizer steps on the student."""

    def __init__(self, teacher, student, temperature: float = 2.0, alpha: float = 1.0, lr: float = 1e-3):
        self.teacher, self.student, self.T, self.alpha = teacher, student, temperature, alpha
        self.opt = torch.optim.AdamW(student.parameters(), lr=lr)

    def loss(self, x, labels=None):
        with torch.no_grad():
            t = self.teacher(x)
        s = self.student(x)
        kl = torch.nn.functional.kl_div(torch.log_softmax(s.float() / self.T, -1), torch.softmax(t.float() / self.T, -1),
                                        reduction="batchmean") * self.T ** 2
        if labels is None or self.alpha >= 1.0:
            return kl
        ce = torch.nn.functional.cross_entropy(s.float().reshape(-1, s.shape[-1]), labels.reshape(-1))
        return self.alpha * kl + (1 - self.alpha) * ce

    def distill(self, data, steps: int) -> list[float]:
        losses = []
        it = iter(data)
        for _ in range(steps):
            try:
                batch = next(it)
            except StopIteration:
                it = iter(data)
                batch = next(it)
            x, y = batch if isinstance(batch, (tuple, list)) else (batch, None)
            loss = self.loss(x, y)
            self.opt.zero_grad()
            loss.backward()
            self.opt.step()
            losses.append(float(loss.detach()))
        return losses


# --------------------------------------------------------------------------- prompting / tools / memory / planning


class PromptOptimizer:
    MUTATIONS = ("Let's think step by step. ", "Answer concisely. ", "You are an expert. ", "Check your work. ")

    def __init__(self, model, scorer=None, seed: int = 0):
        self.model, self.rng = model, random.Random(seed)
        self.scorer = scorer

    def evaluate(self, prompt: str, task: str) -> float:
        if self.scorer is not None:
            return self.scorer(prompt, task)
        return SelfMonitor.estimate_confidence(self.model.next_token_logits(prompt + task))

    def optimize(self, task: str, n_iterations: int = 20) -> str:
        best, best_s = "", self.evaluate("", task)
        for _ in range(n_iterations):
            cand = self.rng.choice(self.MUTATIONS) + best if self.rng.random() < 0.7 else self.rng.choice(self.MUTATIONS)
            s = self.evaluate(cand, task)
            if s > best_s:
                best, best_s = cand, s
        return best


class ChainOfThought:
    def __init__(self, model):
        self.model, self.chain = model, []

    def reason(self, problem: str, max_steps: int = 10) -> str:
        self.chain = []
        ctx = f"Problem: {problem}\n"
        for i in range(max_steps):
            step = self.model.generate_text(ctx + f"Step {i + 1}:", 32).strip()
            if not step:
                break
            self.chain.append(step)
            ctx += f"Step {i + 1}: {step}\n"
            if "answer" in step.lower() or "therefore" in step.lower():
                break
        return self.chain[-1] if self.chain else ""

    def get_chain(self):
        return list(self.chain)


class ToolUse:
    def __init__(self, model=None):
        self.model = model
        self.tools = {"calculator": ("evaluate an arithmetic expression", self._calc),
                      "length": ("number of characters", lambda a: str(len(a))),
                      "upper": ("upper-case the text", lambda a: a.upper())}

    @staticmethod
    def _calc(expr: str) -> str:
        """+ - * / % and parentheses over numbers, evaluated by walking the syntax tree (no eval):
        no names, calls or powers, at most 256 characters and 64 operations, results bounded."""
        import ast
        import operator

        if len(expr) > 256 or not re.fullmatch(r"[0-9+\-*/(). %]+", expr) or "**" in expr:
            return "error: unsupported expression"
        ops = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv,
               ast.Mod: operator.mod, ast.FloorDiv: operator.floordiv}
        budget = [64]

        def ev(node):
            budget[0] -= 1
            if budget[0] < 0:
                raise ValueError("expression too long")
            if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)):
                return node.value
            if isinstance(node, ast.UnaryOp) and isinstance(node.op, (ast.UAdd, ast.USub)):
                v = ev(node.operand)
                return -v if isinstance(node.op, ast.USub) else v
            if isinstance(node, ast.BinOp) and type(node.op) in ops:
                v = ops[type(node.op)](ev(node.left), ev(node.right))
                if abs(v) > 1e300:
                    raise ValueError("result out of range")
                return v
            raise ValueError("unsupported expression")

        try:
            return str(ev(ast.parse(expr.strip(), mode="eval").body))
        except Exception as e:                                  # noqa: BLE001
            return f"error: {e}"

    def register(self, name: str, description: str, fn) -> None:
        self.tools[name] = (description, fn)

    def call_tool(self, tool_name: str, args: str) -> str:
        if tool_name not in self.tools:
            return f"error: unknown tool {tool_name}"
        return self.tools[tool_name][1](args)

    def get_available_tools(self):
        return sorted(self.tools)


class MemorySystem:
    def __init__(self, capacity: int = 10000):
        self.capacity = capacity
        self.keys: list[torch.Tensor] = []
        self.values: list[torch.Tensor] = []

    def store(self, key, value) -> None:
        if len(self.keys) >= self.capacity:
            self.keys.pop(0)
            self.values.pop(0)
        self.keys.append(key.float().reshape(-1))
        self.values.append(value)

    def retrieve(self, query, k: int = 5):
        if not self.keys:
            return []
        K = torch.stack(self.keys)
        sim = torch.nn.functional.cosine_similarity(K, query.float().reshape(1, -1), dim=1)
        top = torch.topk(sim, min(k, len(self.keys))).indices.tolist()
        return [self.values[i] for i in top]

    def consolidate(self, threshold: float = 0.98) -> int:
        """Drop near-duplicate keys (cosine above threshold); returns how many were removed."""
        keep_k, keep_v = [], []
        for k, v in zip(self.keys, self.values):
            if all(float(torch.nn.functional.cosine_similarity(k, q, dim=0)) < threshold for q in keep_k):
                keep_k.append(k)
                keep_v.append(v)
        removed = len(self.keys) - len(keep_k)
        self.keys, self.values = keep_k, keep_v
        return removed


@dataclass
class PlanStep:
    action: str
    dependencies: list = field(default_factory=list)


class PlanningEngine:
    def __init__(self, model=None, executor=None):
        self.model, self.executor = model, executor

    def plan(self, goal: str, max_steps: int = 20) -> list[PlanStep]:
        if self.model is not None:
            raw = self.model.generate_text(f"Goal: {goal}\nNumbered steps:", 128)
            lines = [re.sub(r"^\s*\d+[.)]\s*", "", ln).strip() for ln in raw.splitlines() if ln.strip()]
        else:
            lines = [f"analyse: {goal}", f"decompose: {goal}", f"execute: {goal}", f"verify: {goal}"]
        steps = [PlanStep(a, [lines[i - 1]] if i else []) for i, a in enumerate(lines[:max_steps])]
        return steps

    def execute(self, plan) -> bool:
        done = set()
        for st in plan:
            if any(d not in done for d in st.dependencies):
                return False
            if self.executor is not None and not self.executor(st.action):
                return False
            done.add(st.action)
        return True


@dataclass
class EvalResult:
    accuracy: float
    loss: float
    samples: int


class EvaluationHarness:
    """Named benchmarks are lists of (prompt, expected continuation)."""

    def __init__(self, model, benchmarks: dict | None = None):
        self.model = model
        self.benchmarks = benchmarks or {"arithmetic": [("1 + 1 =", "2"), ("3 + 4 =", "7")],
                                         "copy": [("repeat: cat ->", "cat")]}

    def evaluate(self, benchmark_name: str, n_samples: int = 100) -> EvalResult:
        items = self.benchmarks[benchmark_name][:n_samples]
        hits, loss = 0, 0.0
        for prompt, want in items:
            out = self.model.generate_text(prompt, 8)
            hits += int(want.strip() in out)
            loss += 1.0 - SelfMonitor.estimate_confidence(self.model.next_token_logits(prompt))
        n = max(1, len(items))
        return EvalResult(hits / n, loss / n, len(items))

    def evaluate_all(self):
        return [self.evaluate(b) for b in self.benchmarks]


# --------------------------------------------------------------------------- flywheel


@dataclass
class SandboxResult:
    compiled: bool = False
    passed: bool = False
    score: float = 0.0
    stdout_capture: str = ""
    stderr_capture: str = ""
    runtime_ms: float = 0.0
    exit_code: int = -1


@dataclass
class FlywheelIteration:
    iter: int = 0
    task: str = ""
    solution: str = ""
    compiled: bool = False
    verified: bool = False
    delta: float = 0.0
    applied: bool = False
    rolled_back: bool = False
    file: str = ""
    line: int = 0
    proof: str = ""
    runtime_ms: float = 0.0


class Flywheel:
    """Self-improvement loop over C++ snippets: self-play proposes a task and a solution, the
    sandbox compiles and runs it with a timeout in a private temp directory, the improvement is
    measured (tests passed, runtime, static quality), applied to the target file with a backup,
    rolled back if the target no longer compiles, and every iteration is appended to a JSONL log."""

    TASKS = (("sum_array", "int solve(const int* a, int n) { int s = 0; for (int i = 0; i < n; ++i) s += a[i]; return s; }",
              "int a[4] = {1, 2, 3, 4}; CHECK(solve(a, 4) == 10); CHECK(solve(a, 0) == 0);"),
             ("max_array", "int solve(const int* a, int n) { int m = a[0]; for (int i = 1; i < n; ++i) if (a[i] > m) m = a[i]; return m; }",
              "int a[4] = {3, 9, 2, 5}; CHECK(solve(a, 4) == 9); CHECK(solve(a, 1) == 3);"))

    def __init__(self, model=None, codegen: CodeGenSelfImprover | None = None, verifier: SelfVerifier | None = None,
                 safety: SafetyGuardrails | None = None, workdir: str | None = None, patience: int = 5):
        self.model, self.codegen = model, codegen or CodeGenSelfImprover(model, "cpp")
        self.verifier, self.safety = verifier or SelfVerifier(), safety or SafetyGuardrails()
        self.workdir = workdir or tempfile.mkdtemp(prefix="mythos_flywheel_")
        self.history: list[FlywheelIteration] = []
        self.no_improvement_count, self.patience = 0, patience
        self._best: dict[str, float] = {}

    # -- helpers
    def sandbox_path(self) -> str:
        p = os.path.join(self.workdir, "sandbox")
        os.makedirs(p, exist_ok=True)
        return p

    def get_log_path(self) -> str:
        return os.path.join(self.workdir, "flywheel.jsonl")

    def get_history(self):
        return self.history

    def self_play(self, i: int = 0):
        name, solution, tests = self.TASKS[i % len(self.TASKS)]
        if self.model is not None:
            proposal = self.model.generate_text(f"// C++ function for task {name}\n", 128)
            if "solve" in proposal and self.verifier.verify(name, proposal):
                solution = proposal
        return name, solution, tests

    @staticmethod
    def generate_test_program(code: str, tests: str) -> str:
        return ("#include <cstdio>\nstatic int passed = 0, failed = 0;\n"
                "#define CHECK(c) do { if (c) ++passed; else ++failed; } while (0)\n"
                f"{code}\nint main() {{ {tests} std::printf(\"PASSED %d FAILED %d\\n\", passed, failed); "
                "return failed ? 1 : 0; }\n")

    @staticmethod
    def count_tests_passed(stdout: str) -> int:
        m = re.search(r"PASSED (\d+)", stdout)
        return int(m.group(1)) if m else 0

    @staticmethod
    def run_with_timeout(binary: str, timeout_sec: float):
        try:
            r = subprocess.run([binary], capture_output=True, text=True, timeout=timeout_sec)
            return True, r.stdout, r.stderr, r.returncode
        except subprocess.TimeoutExpired as e:
            return False, e.stdout or "", "timeout", -9

    def sandbox_compile_and_test(self, code: str, tests: str, timeout_sec: float = 5.0) -> SandboxResult:
        res = SandboxResult()
        if not self.safety.check_output(code) or shutil.which("g++") is None:
            res.stderr_capture = "blocked by guardrails" if shutil.which("g++") else "no compiler"
            return res
        d = self.sandbox_path()
        src, exe = os.path.join(d, "t.cpp"), os.path.join(d, "t.bin")
        with open(src, "w") as f:
            f.write(self.generate_test_program(code, tests))
        c = subprocess.run(["g++", "-O1", "-o", exe, src], capture_output=True, text=True, timeout=60)
        res.compiled = c.returncode == 0
        if not res.compiled:
            res.stderr_capture = c.stderr[-2000:]
            return res
        t0 = time.perf_counter()
        ok, out, err, rc = self.run_with_timeout(exe, timeout_sec)
        res.runtime_ms = (time.perf_counter() - t0) * 1e3
        res.stdout_capture, res.stderr_capture, res.exit_code = out, err, rc
        res.passed = ok and rc == 0
        res.score = self.count_tests_passed(out) + self.estimate_code_quality(code)
        return res

    @staticmethod
    def calculate_cyclomatic_complexity(code: str) -> int:
        return 1 + len(re.findall(r"\b(if|for|while|case|catch)\b|&&|\|\||\?", code))

    @staticmethod
    def measure_nesting_depth(code: str) -> int:
        depth = best = 0
        for ch in code:
            if ch == "{":
                depth += 1
                best = max(best, depth)
            elif ch == "}":
                depth -= 1
        return best

    def estimate_code_quality(self, code: str) -> float:
        """0..1: shorter, flatter, less branchy code scores higher."""
        cc, nd, n = self.calculate_cyclomatic_complexity(code), self.measure_nesting_depth(code), len(code)
        return max(0.0, 1.0 - 0.03 * cc - 0.05 * nd - n / 20000.0)

    def measure_improvement(self, task: str, result: SandboxResult) -> float:
        prev = self._best.get(task)
        delta = result.score if prev is None else result.score - prev
        if prev is None or result.score > prev:
            self._best[task] = result.score
        return delta

    @staticmethod
    def make_diff(original: str, improved: str) -> str:
        import difflib

        return "".join(difflib.unified_diff(original.splitlines(True), improved.splitlines(True), "a", "b"))

    def apply_improvement(self, improved: str, target_file: str) -> bool:
        backup = target_file + ".bak"
        if os.path.exists(target_file):
            shutil.copyfile(target_file, backup)
        with open(target_file, "w") as f:
            f.write(improved)
        ok = self.codegen.compile_and_test(improved)
        if not ok:
            self.rollback(target_file, backup)
        return ok

    @staticmethod
    def rollback(file_path: str, backup_path: str) -> bool:
        if os.path.exists(backup_path):
            shutil.copyfile(backup_path, file_path)
            return True
        if os.path.exists(file_path):
            os.remove(file_path)
        return False

    @staticmethod
    def extract_proof(solution: str) -> str:
        m = re.search(r"//\s*proof:(.*)", solution)
        return m.group(1).strip() if m else ""

    def log_iteration(self, it: FlywheelIteration) -> None:
        with open(self.get_log_path(), "a") as f:
            f.write(json.dumps(asdict(it)) + "\n")

    def check_convergence(self) -> bool:
        return self.no_improvement_count >= self.patience

    def run(self, max_iters: int = 100) -> list[FlywheelIteration]:
        for i in range(max_iters):
            if self.safety.is_killed() or self.check_convergence():
                break
            task, solution, tests = self.self_play(i)
            it = FlywheelIteration(iter=i, task=task, solution=solution, proof=self.extract_proof(solution))
            res = self.sandbox_compile_and_test(solution, tests)
            it.compiled, it.verified, it.runtime_ms = res.compiled, res.passed, res.runtime_ms
            if res.passed:
                it.delta = self.measure_improvement(task, res)
                if it.delta > 0:
                    it.file = os.path.join(self.workdir, f"{task}.cpp")
                    it.applied = self.apply_improvement(solution, it.file)
                    it.rolled_back = not it.applied
            self.no_improvement_count = 0 if it.applied else self.no_improvement_count + 1
            self.history.append(it)
            self.log_iteration(it)
        return self.history
