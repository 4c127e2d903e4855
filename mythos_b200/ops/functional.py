"""Differentiable operators of the framework.

Every function here has two execution paths with the same semantics:

* CUDA tensors run the hand-written sm_100a kernels (``mythos_b200._C``) wrapped in
  ``torch.autograd.Function`` objects. Activations are bf16; weight gradients are accumulated in
  fp32 directly into a caller-provided ``grad_target`` buffer (the flat gradient buffer that the
  sharded optimizer and the fused reduce-scatter work on), so no per-parameter ``.grad`` tensors
  exist on this path.
* CPU tensors run the PyTorch reference formulas of :mod:`mythos_b200.ops.reference` under
  ordinary autograd. That path is the oracle of the kernel tests.

There is no fallback from the first path to the second: a CUDA tensor without the compiled
extension raises.
"""
from __future__ import annotations

import math
import os

import torch

from . import native, reference as ref

EPI_BF16, EPI_F32, EPI_F32_ACC, EPI_F32_ATOMIC = 0, 1, 2, 3
# MYTHOS_FUSED_EPILOGUES=0 runs SwiGLU / RoPE as separate kernels (for A/B timing of the fusion)
FUSED_EPILOGUES = os.environ.get("MYTHOS_FUSED_EPILOGUES", "1") != "0"
# Weight gradients are added into the flat fp32 gradient buffer with a read-add-store epilogue (one
# tile per output block, bit-reproducible). MYTHOS_WGRAD_SPLITK=1 lets the wgrad GEMM split K over SM
# pairs and add with fp32 atomics instead: +5-15 % on some layer shapes of the 1.3B model in isolation,
# no measurable change of the whole training step, and the order of the additions varies run to run.
# MYTHOS_FUSED_ROPE_BWD=0: the attention backward leaves dq / dk rotated and two RoPE passes undo it
# (for A/B timing of the in-kernel rotation)
FUSED_ROPE_BWD = os.environ.get("MYTHOS_FUSED_ROPE_BWD", "1") != "0"
WGRAD_EPI = EPI_F32_ATOMIC if os.environ.get("MYTHOS_WGRAD_SPLITK", "0") == "1" else EPI_F32_ACC


def _C():
    return native.require()


# --------------------------------------------------------------------------------------- recompute
class _CheckpointFn(torch.autograd.Function):
    """Keeps only the inputs of ``fn``; the backward pass runs ``fn`` again to rebuild what its
    operators need (the reference's ``CheckpointFn``, include/oil/autograd.h:23-44, and the
    checkpoint flag of its engine, src/autograd.cpp:1226-1244, 1288-1290)."""

    @staticmethod
    def forward(ctx, fn, *args):
        ctx.fn = fn
        ctx.is_tensor = [torch.is_tensor(a) for a in args]
        ctx.others = [None if torch.is_tensor(a) else a for a in args]
        ctx.save_for_backward(*[a for a in args if torch.is_tensor(a)])
        with torch.no_grad():
            out = fn(*args)
        ctx.single = torch.is_tensor(out)
        return out if ctx.single else tuple(out)

    @staticmethod
    def backward(ctx, *grads):
        saved = list(ctx.saved_tensors)
        args, leaves = [], []
        for is_t, other in zip(ctx.is_tensor, ctx.others):
            if is_t:
                t = saved.pop(0).detach()
                if t.is_floating_point():
                    t.requires_grad_()
                leaves.append(t)
                args.append(t)
            else:
                leaves.append(None)
                args.append(other)
        with torch.enable_grad():
            out = ctx.fn(*args)
        outs = [out] if torch.is_tensor(out) else list(out)
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None,) + tuple(None if t is None else t.grad for t in leaves)


def checkpoint(fn, *args):
    """``fn(*args)`` with activation recomputation: intermediate activations are dropped after the
    forward pass and rebuilt in the backward pass (one extra forward of ``fn``). Parameters reached
    through ``fn`` receive their gradients as usual. Without autograd it is a plain call."""
    if not torch.is_grad_enabled() or not any(torch.is_tensor(a) and a.requires_grad for a in args):
        return fn(*args)
    return _CheckpointFn.apply(fn, *args)


# --------------------------------------------------------------------------------------- GEMM
def gemm(a, b, *, a_mn: bool = False, b_mn: bool = False, out=None, epi: int = EPI_BF16, alpha: float = 1.0):
    """``out[M,N] (+)= alpha * A @ B^T`` on tcgen05. ``a_mn``/``b_mn``: the operand is stored
    transposed (``[K,M]`` / ``[K,N]``). ``epi`` selects bf16 store, fp32 store, fp32 read-add-store
    or fp32 atomic accumulate (split-K)."""
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=torch.bfloat16 if epi == EPI_BF16 else torch.float32)
    _C().gemm(a, b, out, a_mn, b_mn, epi, alpha, native.status_word(a.device))
    return out


class _LinearFn(torch.autograd.Function):
    """y = x W^T with W [N,K] bf16. Backward: dx = dy W (MN-major B), dW = dy^T x (both MN-major)
    accumulated in fp32 into ``grad_target`` when given, else returned."""

    @staticmethod
    def forward(ctx, x, w, grad_target):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        y = gemm(x2, w)
        ctx.save_for_backward(x2, w)
        ctx.grad_target = grad_target
        ctx.x_shape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(ctx.x_shape)
        dw = None
        if ctx.grad_target is not None:
            gemm(dy2, x2, a_mn=True, b_mn=True, out=ctx.grad_target, epi=WGRAD_EPI)
        elif ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True, epi=EPI_F32).to(w.dtype)
        return dx, dw, None


_ROPE_TABLES: dict = {}


def rope_table(theta: float, max_pos: int, device, head_dim: int = 128):
    """[max_pos, head_dim/2, 2] fp32 (cos, sin) of angle ``pos * theta^(-2j/head_dim)``; cached."""
    key = (float(theta), int(max_pos), str(device), head_dim)
    t = _ROPE_TABLES.get(key)
    if t is None:
        j = torch.arange(head_dim // 2, device=device, dtype=torch.float32)
        inv = torch.exp2(-2.0 * j / head_dim * math.log2(theta))
        ang = torch.arange(max_pos, device=device, dtype=torch.float32)[:, None] * inv[None, :]
        t = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
        _ROPE_TABLES[key] = t
    return t


class _LinearRopeFn(torch.autograd.Function):
    """y = x W^T with the rotary embedding of the q and k heads applied in the GEMM epilogue. The
    gradient handed back by the attention function is already rotated back (it is the gradient of
    the un-rotated projection), so the backward pass is the one of a plain linear layer."""

    @staticmethod
    def forward(ctx, x, w, grad_target, pos, table, rope_cols):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        y = torch.empty(x2.shape[0], w.shape[0], device=x.device, dtype=torch.bfloat16)
        _C().gemm_rope(x2, w, y, pos, table, rope_cols, native.status_word(x.device))
        ctx.save_for_backward(x2, w)
        ctx.grad_target = grad_target
        ctx.x_shape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        dx, dw, _ = _LinearFn.backward(ctx, dy)
        return dx, dw, None, None, None, None


def fused_rope_ok(x, w, head_dim: int, theta: float) -> bool:
    """The epilogue rotation covers heads of 128 on the paired-SM GEMM (>= 256 rows and columns)."""
    rows = x.numel() // x.shape[-1]
    return (FUSED_EPILOGUES and x.is_cuda and head_dim == 128 and theta > 0 and rows >= 256 and w.shape[0] >= 256
            and w.shape[0] % 128 == 0 and x.shape[-1] % 8 == 0)


def linear_rope(x, w, grad_target, pos, theta: float, rope_cols: int, max_pos: int):
    """``x @ w.T`` followed by RoPE on columns [0, rope_cols) (heads of 128), in one kernel. ``pos``
    values must be below ``max_pos``. Pair with ``attention_qkv(..., rope_applied=True)``."""
    table = rope_table(theta, max_pos, x.device)
    return _LinearRopeFn.apply(x, w, grad_target, pos, table, rope_cols)


class _FusedFFNFn(torch.autograd.Function):
    """SwiGLU FFN ``down(silu(gate(x)) * up(x))`` in two GEMM launches forward and four backward:
    the activation runs in the epilogue of the gate/up GEMM, its derivative in the epilogue of the
    down-projection dgrad GEMM (dL/dh is never written)."""

    @staticmethod
    def forward(ctx, x, w_gu, w_down, gt_gu, gt_down):
        C = _C()
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        M, F2 = x2.shape[0], w_gu.shape[0]
        st = native.status_word(x.device)
        gu = torch.empty(M, F2, device=x.device, dtype=torch.bfloat16)
        h = torch.empty(M, F2 // 2, device=x.device, dtype=torch.bfloat16)
        C.gemm_swiglu_fwd(x2, w_gu, gu, h, st)
        y = gemm(h, w_down)
        ctx.save_for_backward(x2, w_gu, w_down, gu, h)
        ctx.gts = (gt_gu, gt_down)
        ctx.x_shape = x.shape
        return y.reshape(*x.shape[:-1], w_down.shape[0])

    @staticmethod
    def backward(ctx, dy):
        C = _C()
        x2, w_gu, w_down, gu, h = ctx.saved_tensors
        gt_gu, gt_down = ctx.gts
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dgu = torch.empty_like(gu)
        C.gemm_swiglu_bwd(dy2, w_down, gu, dgu, native.status_word(dy.device))
        dw_down = dw_gu = None
        if gt_down is not None:
            gemm(dy2, h, a_mn=True, b_mn=True, out=gt_down, epi=WGRAD_EPI)
        elif ctx.needs_input_grad[2]:
            dw_down = gemm(dy2, h, a_mn=True, b_mn=True, epi=EPI_F32).to(w_down.dtype)
        dx = gemm(dgu, w_gu, b_mn=True).reshape(ctx.x_shape) if ctx.needs_input_grad[0] else None
        if gt_gu is not None:
            gemm(dgu, x2, a_mn=True, b_mn=True, out=gt_gu, epi=WGRAD_EPI)
        elif ctx.needs_input_grad[1]:
            dw_gu = gemm(dgu, x2, a_mn=True, b_mn=True, epi=EPI_F32).to(w_gu.dtype)
        return dx, dw_gu, dw_down, None, None


def fused_ffn_ok(x, w_gu, w_down) -> bool:
    rows = x.numel() // x.shape[-1]
    f = w_gu.shape[0] // 2
    return (FUSED_EPILOGUES and x.is_cuda and rows >= 256 and f % 128 == 0 and f >= 256 and x.shape[-1] % 8 == 0
            and w_down.shape[0] >= 256 and w_down.shape[1] == f)


def swiglu_ffn(x, w_gu, w_down, gt_gu=None, gt_down=None):
    """``(silu(x Wg^T) * (x Wu^T)) Wd^T`` with ``w_gu`` = [Wg; Wu] ([2F, d]) and ``w_down`` [d, F].
    CUDA with F a multiple of 128: the fused-epilogue GEMMs; otherwise linear -> swiglu -> linear."""
    if fused_ffn_ok(x, w_gu, w_down):
        return _FusedFFNFn.apply(x, w_gu, w_down, gt_gu, gt_down)
    return linear(swiglu(linear(x, w_gu, gt_gu)), w_down, gt_down)


def linear(x, w, grad_target=None):
    """``x @ w.T``. CUDA: tcgen05 GEMMs (bf16). CPU: torch matmul in the weight's dtype."""
    if x.is_cuda:
        return _LinearFn.apply(x, w, grad_target)
    return torch.nn.functional.linear(x, w.to(x.dtype))


# --------------------------------------------------------------------------------------- RMSNorm
def _n_partial(rows: int, device) -> int:
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    return max(1, min(rows, sms * 3))


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, gamma, eps, grad_target):
        C = _C()
        xc = x.contiguous()
        y = torch.empty_like(xc)
        rows = xc.numel() // xc.shape[-1]
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        if residual is not None:
            h = torch.empty_like(xc)
            C.rmsnorm_fwd(xc, residual.contiguous(), gamma, y, h, rstd, eps)
            h_out = h
        else:
            h = xc
            C.rmsnorm_fwd(xc, None, gamma, y, None, rstd, eps)
            h_out = torch.empty(0, device=x.device, dtype=x.dtype)  # placeholder: h is x itself
            ctx.mark_non_differentiable(h_out)
        ctx.save_for_backward(h, gamma, rstd)
        ctx.grad_target = grad_target
        ctx.has_residual = residual is not None
        return y, h_out

    @staticmethod
    def backward(ctx, dy, dh):
        C = _C()
        h, gamma, rstd = ctx.saved_tensors
        dim = h.shape[-1]
        rows = h.numel() // dim
        dx = torch.empty_like(h)
        npart = _n_partial(rows, h.device)
        partial = torch.empty(npart, dim, device=h.device, dtype=torch.float32)
        # the gradient that arrives through the residual stream is added inside the kernel
        dres = dh.contiguous() if (ctx.has_residual and dh is not None) else None
        if ctx.grad_target is not None:
            C.rmsnorm_bwd(dy.contiguous(), h, gamma, rstd, dx, partial, ctx.grad_target, True, dres)
            dgamma = None
        else:
            dg = torch.empty(dim, device=h.device, dtype=torch.float32)
            C.rmsnorm_bwd(dy.contiguous(), h, gamma, rstd, dx, partial, dg, False, dres)
            dgamma = dg.to(gamma.dtype)
        return dx, (dx if ctx.has_residual else None), dgamma, None, None


def rmsnorm(x, gamma, eps: float = 1e-5, residual=None, grad_target=None):
    """Returns ``(y, h)``: ``h = x + residual`` (``x`` itself without residual) and
    ``y = h * rsqrt(mean(h^2)+eps) * gamma``."""
    if x.is_cuda:
        y, h = _RMSNormFn.apply(x, residual, gamma, eps, grad_target)
        return y, (h if residual is not None else x)
    h = x if residual is None else x + residual
    rstd = torch.rsqrt(h.float().pow(2).mean(-1, keepdim=True) + eps)
    return (h.float() * rstd * gamma.float()).to(x.dtype), h


class _LayerNormFn(torch.autograd.Function):
    """LayerNorm with native forward and backward kernels (the backward recomputes mean and rstd from
    x; formula of the reference's layer-norm gradient, src/autograd.cpp)."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _C().layernorm_fwd(xc, gamma, beta, y, eps)
        ctx.save_for_backward(xc, gamma)
        ctx.eps, ctx.has_beta = eps, beta is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma = ctx.saved_tensors
        dim = x.shape[-1]
        dx = torch.empty_like(x)
        n_partial = _n_partial(x.numel() // dim, x.device)
        partial = torch.empty(n_partial, 2 * dim, device=x.device, dtype=torch.float32)
        dgb = torch.empty(2 * dim, device=x.device, dtype=torch.float32)
        _C().layernorm_bwd(dy.contiguous(), x, gamma, dx, partial, dgb, ctx.eps)
        return dx, dgb[:dim].to(gamma.dtype), (dgb[dim:].to(gamma.dtype) if ctx.has_beta else None), None


def layernorm(x, gamma, beta=None, eps: float = 1e-5):
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        if torch.is_grad_enabled() and (x.requires_grad or gamma.requires_grad):
            return _LayerNormFn.apply(x, gamma, beta, eps)
        y = torch.empty_like(x.contiguous())
        _C().layernorm_fwd(x.contiguous(), gamma, beta, y, eps)
        return y
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), gamma.float(),
                                          None if beta is None else beta.float(), eps).to(x.dtype)


# --------------------------------------------------------------------------------------- attention
_SUPPORTED_BWD_HEAD_DIMS = (64, 128)     # 64 runs the 128-wide kernel on zero-padded heads


def _pad_heads(t, width: int):
    """[B, S, H, D] (any strides) -> contiguous [B, S, H, width] with zeros beyond D."""
    out = t.new_zeros(*t.shape[:-1], width)
    out[..., : t.shape[-1]].copy_(t)
    return out


class _AttentionFn(torch.autograd.Function):
    """RoPE (in place on the q and k slices of the fused projection) + causal flash attention.

    qkv: [B, S, (H + 2*Hkv) * D] bf16, laid out q | k | v along the last dimension."""

    @staticmethod
    def forward(ctx, qkv, pos, H, Hkv, D, theta, causal, scale, rope_applied=False, rope_max_pos=0):
        C = _C()
        B, S, W = qkv.shape
        assert W == (H + 2 * Hkv) * D and qkv.is_contiguous()
        flat = qkv.view(B * S, W)
        q = flat[:, : H * D].unflatten(-1, (H, D))
        k = flat[:, H * D: (H + Hkv) * D].unflatten(-1, (Hkv, D))
        if theta > 0 and not rope_applied:
            C.rope(q, pos, theta, False)
            C.rope(k, pos, theta, False)
        q4 = qkv[..., : H * D].unflatten(-1, (H, D))
        k4 = qkv[..., H * D: (H + Hkv) * D].unflatten(-1, (Hkv, D))
        v4 = qkv[..., (H + Hkv) * D:].unflatten(-1, (Hkv, D))
        o = torch.empty(B, S, H, D, device=qkv.device, dtype=qkv.dtype)
        lse = torch.empty(B, H, S, device=qkv.device, dtype=torch.float32)
        C.flash_attn_fwd(q4, k4, v4, o, lse, causal, scale, native.status_word(qkv.device))
        ctx.save_for_backward(qkv, pos, o, lse)
        ctx.cfg = (H, Hkv, D, theta, causal, scale, rope_max_pos)
        return o.view(B, S, H * D)

    @staticmethod
    def backward(ctx, do):
        C = _C()
        qkv, pos, o, lse = ctx.saved_tensors
        H, Hkv, D, theta, causal, scale, rope_max_pos = ctx.cfg
        if D not in _SUPPORTED_BWD_HEAD_DIMS:
            raise NotImplementedError(f"flash attention backward supports head_dim {_SUPPORTED_BWD_HEAD_DIMS}, got {D}")
        B, S, W = qkv.shape
        q4 = qkv[..., : H * D].unflatten(-1, (H, D))
        k4 = qkv[..., H * D: (H + Hkv) * D].unflatten(-1, (Hkv, D))
        v4 = qkv[..., (H + Hkv) * D:].unflatten(-1, (Hkv, D))
        dqkv = torch.empty_like(qkv)
        dq4 = dqkv[..., : H * D].unflatten(-1, (H, D))
        dk4 = dqkv[..., H * D: (H + Hkv) * D].unflatten(-1, (Hkv, D))
        dv4 = dqkv[..., (H + Hkv) * D:].unflatten(-1, (Hkv, D))
        dq_accum = torch.empty(B * S * H * D, device=qkv.device, dtype=torch.float32)
        delta = torch.empty(B * H * S, device=qkv.device, dtype=torch.float32)
        do4 = do.reshape(B, S, H, D).contiguous()
        # With a position bound the kernel undoes the rotation itself (dq while converting the fp32
        # accumulator, dk in its epilogue) from the same cos/sin table the fused projection used.
        fused_rope = FUSED_ROPE_BWD and D == 128 and theta > 0 and rope_max_pos > 0
        if D == 128:
            C.flash_attn_bwd(q4, k4, v4, o, do4, lse, dq4, dk4, dv4, dq_accum, delta, causal, scale,
                             native.status_word(qkv.device), pos if fused_rope else None,
                             rope_table(theta, rope_max_pos, qkv.device) if fused_rope else None)
        else:
            # Zero columns change neither the scores nor o . do, so the padded problem has the same
            # lse and delta; the gradients of the padding columns come out zero and are dropped.
            P = 128
            qp, kp, vp, op, dop = (_pad_heads(t, P) for t in (q4, k4, v4, o.view(B, S, H, D), do4))
            dqp, dkp, dvp = torch.empty_like(qp), torch.empty_like(kp), torch.empty_like(vp)
            dq_accum = torch.empty(B * S * H * P, device=qkv.device, dtype=torch.float32)
            C.flash_attn_bwd(qp, kp, vp, op, dop, lse, dqp, dkp, dvp, dq_accum, delta, causal, scale,
                             native.status_word(qkv.device))
            dq4.copy_(dqp[..., :D])
            dk4.copy_(dkp[..., :D])
            dv4.copy_(dvp[..., :D])
        if theta > 0 and not fused_rope:
            flat = dqkv.view(B * S, W)
            C.rope(flat[:, : H * D].unflatten(-1, (H, D)), pos, theta, True)
            C.rope(flat[:, H * D: (H + Hkv) * D].unflatten(-1, (Hkv, D)), pos, theta, True)
        return dqkv, None, None, None, None, None, None, None, None, None


def attention_qkv(qkv, pos, n_heads: int, n_kv_heads: int, head_dim: int, theta: float = 10000.0,
                  causal: bool = True, scale: float | None = None, rope_applied: bool = False,
                  rope_max_pos: int = 0):
    """Self-attention over a fused projection ``qkv`` = [B, S, (H+2Hkv)*D] (q | k | v). RoPE with
    half-split pairs is applied to q and k at positions ``pos`` ([B*S] int32); ``theta <= 0``
    disables it. Returns [B, S, H*D]. On CUDA the projection buffer is rotated in place.
    ``rope_applied``: q and k arrive rotated (``linear_rope``); the forward pass then skips the
    rotation, the backward pass still rotates the gradient back (CUDA only). ``rope_max_pos`` > 0
    promises positions below that bound: the backward kernel then rotates dq and dk back itself
    (head_dim 128) instead of two extra passes over the gradient."""
    scale = (1.0 / math.sqrt(head_dim)) if scale is None else scale
    if qkv.is_cuda:
        return _AttentionFn.apply(qkv, pos, n_heads, n_kv_heads, head_dim, theta, causal, scale, rope_applied,
                                  rope_max_pos)
    assert not rope_applied
    B, S, _ = qkv.shape
    H, Hkv, D = n_heads, n_kv_heads, head_dim
    q = qkv[..., : H * D].reshape(B * S, H, D)
    k = qkv[..., H * D: (H + Hkv) * D].reshape(B * S, Hkv, D)
    v = qkv[..., (H + Hkv) * D:].reshape(B, S, Hkv, D)
    if theta > 0:
        q = ref.rope(q, pos, theta)
        k = ref.rope(k, pos, theta)
    o, _ = ref.attention(q.reshape(B, S, H, D), k.reshape(B, S, Hkv, D), v, causal, scale)
    return o.reshape(B, S, H * D)


def flash_attention(q, k, v, causal: bool = True, scale: float | None = None):
    """Forward-only attention on [B,S,H,D] tensors (no RoPE). Returns (o, lse)."""
    D = q.shape[-1]
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    if q.is_cuda:
        B, S, H, _ = q.shape
        o = torch.empty(B, S, H, D, device=q.device, dtype=q.dtype)
        lse = torch.empty(B, H, S, device=q.device, dtype=torch.float32)
        _C().flash_attn_fwd(q, k, v, o, lse, causal, scale, native.status_word(q.device))
        return o, lse
    return ref.attention(q, k, v, causal, scale)


# --------------------------------------------------------------------------------------- gates
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        gu = gate_up.contiguous()
        out = torch.empty(*gu.shape[:-1], gu.shape[-1] // 2, device=gu.device, dtype=gu.dtype)
        _C().swiglu_fused_fwd(gu, out)
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        dgu = torch.empty_like(gu)
        _C().swiglu_fused_bwd(gu, dout.contiguous(), dgu)
        return dgu


def swiglu(gate_up):
    """``silu(gate) * up`` for a fused [.., 2*ffn] projection (gate first)."""
    if gate_up.is_cuda:
        return _SwiGLUFn.apply(gate_up)
    f = gate_up.shape[-1] // 2
    g, u = gate_up[..., :f], gate_up[..., f:]
    return g * torch.sigmoid(g) * u


class _ReLU2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        out = torch.empty_like(xc)
        _C().relu2_fwd(xc, out)
        ctx.save_for_backward(xc)
        return out

    @staticmethod
    def backward(ctx, dout):
        (x,) = ctx.saved_tensors
        dx = torch.empty_like(x)
        _C().relu2_bwd(x, dout.contiguous(), dx)
        return dx


def relu2(x):
    """Squared ReLU (BitNet-style FFN activation)."""
    if x.is_cuda:
        return _ReLU2Fn.apply(x)
    return torch.relu(x).pow(2)


_ACT_IDS = {"relu": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3, "sigmoid": 4, "tanh": 5}


class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kind_id):
        xc = x.contiguous()
        out = torch.empty_like(xc)
        _C().act_fwd(xc, out, kind_id)
        ctx.save_for_backward(xc)
        ctx.kind_id = kind_id
        return out

    @staticmethod
    def backward(ctx, dout):
        (x,) = ctx.saved_tensors
        dx = torch.empty_like(x)
        _C().act_bwd(x, dout.contiguous(), dx, ctx.kind_id)
        return dx, None


class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _C().softmax_rows(xc, y)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        dx = torch.empty_like(y)
        _C().softmax_rows_bwd(y, dy.contiguous(), dx)
        return dx


def softmax(x):
    """Softmax over the last dimension (native forward and backward on CUDA bf16)."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _SoftmaxFn.apply(x)
    return torch.softmax(x.float(), dim=-1).to(x.dtype)


def activation(x, kind: str):
    """Pointwise activation: relu, gelu (erf), gelu_tanh, silu, sigmoid, tanh. On CUDA bf16 tensors
    whose element count is a multiple of 8 both directions run native kernels."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
        if torch.is_grad_enabled() and x.requires_grad:
            return _ActFn.apply(x, _ACT_IDS[kind])
        xc = x.contiguous()
        out = torch.empty_like(xc)
        _C().act_fwd(xc, out, _ACT_IDS[kind])
        return out
    xf = x
    if kind == "relu":
        return torch.relu(xf)
    if kind == "gelu":
        return ref.gelu_erf(xf)
    if kind == "gelu_tanh":
        return ref.gelu_tanh(xf)
    if kind == "silu":
        return xf * torch.sigmoid(xf)
    if kind == "sigmoid":
        return torch.sigmoid(xf)
    return torch.tanh(xf)


# --------------------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, grad_target):
        out = torch.empty(*ids.shape, table.shape[1], device=table.device, dtype=table.dtype)
        _C().embedding_fwd(ids.contiguous(), table, out)
        ctx.save_for_backward(ids)
        ctx.grad_target = grad_target
        ctx.tshape = table.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        if ctx.grad_target is not None:
            _C().embedding_bwd(ids.contiguous(), dout.contiguous(), ctx.grad_target)
            return None, None, None
        dt = torch.zeros(ctx.tshape, device=dout.device, dtype=torch.float32)
        _C().embedding_bwd(ids.contiguous(), dout.contiguous(), dt)
        return None, dt.to(dout.dtype), None


def embedding(ids, table, grad_target=None):
    """Row gather; ids int32. Backward scatter-adds in fp32 (into ``grad_target`` when given)."""
    if table.is_cuda:
        return _EmbeddingFn.apply(ids, table, grad_target)
    return torch.nn.functional.embedding(ids.long().clamp(0, table.shape[0] - 1), table)


# --------------------------------------------------------------------------------------- loss
class _CrossEntropyFn(torch.autograd.Function):
    """Sum of per-row losses; the gradient (softmax - onehot) * grad_scale overwrites ``logits``
    during the forward pass, so backward is free. The upstream gradient must be 1."""

    @staticmethod
    def forward(ctx, logits, targets, grad_scale):
        losses = torch.empty(logits.shape[0], device=logits.device, dtype=torch.float32)
        _C().cross_entropy_fwd_bwd(logits, targets, losses, grad_scale)
        ctx.save_for_backward(logits)
        return losses.sum() * grad_scale

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits, None, None


def cross_entropy(logits, targets, grad_scale: float | None = None):
    """Scaled sum of next-token losses: ``grad_scale * sum_rows(logsumexp - logit[target])``
    (``grad_scale`` defaults to 1/rows, i.e. the mean). logits: [rows, V]; targets int32 [rows].
    On CUDA the logits buffer is consumed (overwritten with its gradient)."""
    rows = logits.shape[0]
    gs = (1.0 / rows) if grad_scale is None else grad_scale
    if logits.is_cuda:
        if torch.is_grad_enabled() and logits.requires_grad:
            return _CrossEntropyFn.apply(logits, targets, gs)
        losses = torch.empty(rows, device=logits.device, dtype=torch.float32)
        _C().cross_entropy_fwd(logits, targets, losses)
        return losses.sum() * gs
    return ref.cross_entropy(logits, targets).sum() * gs


# --------------------------------------------------------------------------------------- quantisation / optimizer
def oil_fake_quant(w, codebooks, cb_map, bs: int, want_idx: bool = False, out=None):
    """Nearest-centroid fake quantisation of a flat fp32 tensor through sorted codebooks.
    Returns (w_q bf16 on CUDA / fp32 on CPU, indices or None)."""
    if w.is_cuda:
        flat = w.reshape(-1)
        wq = out if out is not None else torch.empty(flat.numel(), device=w.device, dtype=torch.bfloat16)
        idx = torch.empty(flat.numel(), device=w.device, dtype=torch.uint8) if want_idx else None
        _C().oil_fake_quant(flat, codebooks.contiguous(), cb_map, bs, wq, idx)
        return wq.view(w.shape) if out is None else wq, idx
    idx, deq = ref.nearest_centroid(w.reshape(-1), codebooks, cb_map, bs)
    return deq.view(w.shape), (idx if want_idx else None)


def i2s_fake_quant(w, bs: int, want_codes: bool = False, out=None):
    if w.is_cuda:
        flat = w.reshape(-1)
        nb = (flat.numel() + bs - 1) // bs
        wq = out if out is not None else torch.empty(flat.numel(), device=w.device, dtype=torch.bfloat16)
        codes = torch.empty(flat.numel(), device=w.device, dtype=torch.uint8) if want_codes else None
        scales = torch.empty(nb, device=w.device, dtype=torch.float32)
        _C().i2s_fake_quant(flat, bs, wq, codes, scales)
        return (wq.view(w.shape) if out is None else wq), codes, scales
    codes, scales, deq = ref.i2s_quant(w.reshape(-1), bs)
    return deq.view(w.shape), (codes if want_codes else None), scales


def adamw_step(p, m, v, g, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=1, grad_scale=1.0,
               clip_coef=None, p_bf16=None):
    """One fused AdamW step on flat fp32 tensors (in place). ``clip_coef``: optional 1-element
    device tensor multiplied into the gradient (global-norm clipping without a host sync)."""
    if p.is_cuda:
        _C().adamw_step(p, m, v, g, p_bf16, lr, beta1, beta2, eps, weight_decay, step, grad_scale, clip_coef)
        return
    gs = grad_scale * (float(clip_coef) if clip_coef is not None else 1.0)
    ref.adamw_step(p, m, v, g, lr, beta1, beta2, eps, weight_decay, step, gs)
    if p_bf16 is not None:
        p_bf16.copy_(p)


def sumsq(x, out=None):
    """Sum of squares of a flat fp32 tensor, accumulated into ``out`` (1-element fp32)."""
    if out is None:
        out = torch.zeros(1, device=x.device, dtype=torch.float32)
    if x.is_cuda:
        _C().sumsq(x.reshape(-1), out)
    else:
        out += x.float().pow(2).sum()
    return out
