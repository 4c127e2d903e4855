// Python binding of the sm_100a kernel library. Thin on purpose: tensors are checked
// (device, dtype, contiguity of the innermost dimension), outputs are allocated by the Python
// side, and every launch goes to torch's current CUDA stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "kernels/api.h"

namespace {

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void chk(const Tensor& t, c10::ScalarType dt, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == dt, name, " has dtype ", t.scalar_type(), ", expected ", dt);
}
void chk_c(const Tensor& t, c10::ScalarType dt, const char* name) {
  chk(t, dt, name);
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
const void* cptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }
void* mptr(OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }
int* status_ptr(const OptTensor& s) {
  if (!s.has_value()) return nullptr;
  chk_c(*s, torch::kInt32, "status");
  return s->data_ptr<int>();
}

constexpr auto BF16 = torch::kBFloat16;
constexpr auto F32 = torch::kFloat32;
constexpr auto I32 = torch::kInt32;
constexpr auto U8 = torch::kUInt8;

// out[M,N] (+)= alpha * op(a) * op(b)^T. a: [M,K] or, with a_mn, [K,M]; b: [N,K] or, with b_mn, [K,N].
void gemm(const Tensor& a, const Tensor& b, Tensor& out, bool a_mn, bool b_mn, int64_t epi, double alpha,
          const OptTensor& status) {
  chk(a, BF16, "a");
  chk(b, BF16, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm: operands must be 2-D");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "gemm: innermost stride must be 1");
  const int64_t M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: contraction sizes differ: ", K, " vs ", Kb);
  TORCH_CHECK(out.size(0) == M && out.size(1) == N, "gemm: output shape mismatch");
  chk(out, epi == mb::EPI_BF16 ? BF16 : F32, "out");
  c10::cuda::CUDAGuard guard(a.device());
  mb::gemm_bf16(a.data_ptr(), a.stride(0), a_mn, b.data_ptr(), b.stride(0), b_mn, out.data_ptr(), out.stride(0),
                (int)M, (int)N, (int)K, (int)epi, (float)alpha, status_ptr(status), cur_stream());
}

// h[M,F] = silu(gate) * up and (optionally) the pre-activations gu[M,2F] from x[M,K] and w[2F,K].
void gemm_swiglu_fwd(const Tensor& x, const Tensor& w, OptTensor gu, Tensor& h, const OptTensor& status) {
  chk(x, BF16, "x");
  chk(w, BF16, "w");
  chk(h, BF16, "h");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && h.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && h.stride(1) == 1,
              "gemm_swiglu_fwd: 2-D operands with unit inner stride");
  const int64_t M = x.size(0), K = x.size(1), F = w.size(0) / 2;
  TORCH_CHECK(w.size(1) == K && w.size(0) == 2 * F && h.size(0) == M && h.size(1) == F, "gemm_swiglu_fwd: shapes");
  if (gu.has_value()) {
    chk(*gu, BF16, "gu");
    TORCH_CHECK(gu->dim() == 2 && gu->size(0) == M && gu->size(1) == 2 * F && gu->stride(1) == 1, "gemm_swiglu_fwd: gu");
  }
  c10::cuda::CUDAGuard guard(x.device());
  mb::gemm_swiglu_fwd(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), mptr(gu), gu.has_value() ? gu->stride(0) : 0,
                      h.data_ptr(), h.stride(0), (int)M, (int)F, (int)K, status_ptr(status), cur_stream());
}

// dgu[M,2F] = SwiGLU backward of (dy[M,K] @ w_down[K,F]) at the saved pre-activations gu[M,2F].
void gemm_swiglu_bwd(const Tensor& dy, const Tensor& w_down, const Tensor& gu, Tensor& dgu, const OptTensor& status) {
  chk(dy, BF16, "dy");
  chk(w_down, BF16, "w_down");
  chk(gu, BF16, "gu");
  chk(dgu, BF16, "dgu");
  TORCH_CHECK(dy.dim() == 2 && w_down.dim() == 2 && gu.dim() == 2 && dgu.dim() == 2, "gemm_swiglu_bwd: 2-D operands");
  TORCH_CHECK(dy.stride(1) == 1 && w_down.stride(1) == 1 && gu.stride(1) == 1 && dgu.stride(1) == 1,
              "gemm_swiglu_bwd: unit inner stride");
  const int64_t M = dy.size(0), K = dy.size(1), F = w_down.size(1);
  TORCH_CHECK(w_down.size(0) == K && gu.size(0) == M && gu.size(1) == 2 * F && dgu.size(0) == M && dgu.size(1) == 2 * F,
              "gemm_swiglu_bwd: shapes");
  c10::cuda::CUDAGuard guard(dy.device());
  mb::gemm_swiglu_bwd(dy.data_ptr(), dy.stride(0), w_down.data_ptr(), w_down.stride(0), gu.data_ptr(), gu.stride(0),
                      dgu.data_ptr(), dgu.stride(0), (int)M, (int)F, (int)K, status_ptr(status), cur_stream());
}

// out[M,N] = x[M,K] w[N,K]^T with rotary embedding on the 128-wide heads in columns [0, rope_cols).
void gemm_rope(const Tensor& x, const Tensor& w, Tensor& out, const Tensor& pos, const Tensor& cos_sin, int64_t rope_cols,
               const OptTensor& status) {
  chk(x, BF16, "x");
  chk(w, BF16, "w");
  chk(out, BF16, "out");
  chk_c(pos, I32, "pos");
  chk_c(cos_sin, F32, "cos_sin");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1,
              "gemm_rope: 2-D operands with unit inner stride");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && out.size(0) == M && out.size(1) == N && pos.numel() == M, "gemm_rope: shapes");
  TORCH_CHECK(cos_sin.dim() == 3 && cos_sin.size(1) == 64 && cos_sin.size(2) == 2, "gemm_rope: table must be [P, 64, 2]");
  c10::cuda::CUDAGuard guard(x.device());
  mb::gemm_rope(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), (int)M, (int)N,
                (int)K, pos.data_ptr<int>(), cos_sin.data_ptr<float>(), (int)cos_sin.size(0), (int)rope_cols,
                status_ptr(status), cur_stream());
}

void rmsnorm_fwd(const Tensor& x, const OptTensor& residual, const Tensor& gamma, Tensor& y, OptTensor resid_out,
                 OptTensor rstd, double eps) {
  chk_c(x, BF16, "x");
  chk_c(gamma, BF16, "gamma");
  chk_c(y, BF16, "y");
  const int64_t dim = x.size(-1), rows = x.numel() / dim;
  c10::cuda::CUDAGuard guard(x.device());
  mb::rmsnorm_fwd(x.data_ptr(), cptr(residual), gamma.data_ptr(), y.data_ptr(), mptr(resid_out),
                  rstd.has_value() ? rstd->data_ptr<float>() : nullptr, (int)rows, (int)dim, (float)eps, cur_stream());
}

void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& gamma, const Tensor& rstd, Tensor& dx,
                 Tensor& dgamma_partial, Tensor& dgamma, bool accumulate, const OptTensor& dres) {
  if (dres.has_value()) {
    chk_c(*dres, BF16, "dres");
    TORCH_CHECK(dres->numel() == x.numel(), "rmsnorm_bwd: dres must have the shape of x");
  }
  chk_c(dy, BF16, "dy");
  chk_c(x, BF16, "x");
  chk_c(gamma, BF16, "gamma");
  chk_c(rstd, F32, "rstd");
  chk_c(dx, BF16, "dx");
  chk_c(dgamma_partial, F32, "dgamma_partial");
  chk_c(dgamma, F32, "dgamma");
  const int64_t dim = x.size(-1), rows = x.numel() / dim;
  const int64_t n_partial = dgamma_partial.size(0);
  TORCH_CHECK(dgamma_partial.size(1) == dim, "rmsnorm_bwd: partial buffer must be [n_partial, dim]");
  c10::cuda::CUDAGuard guard(x.device());
  mb::rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                  dgamma_partial.data_ptr<float>(), (int)rows, (int)dim, (int)n_partial, cur_stream(), cptr(dres));
  mb::rmsnorm_bwd_reduce(dgamma_partial.data_ptr<float>(), dgamma.data_ptr<float>(), (int)n_partial, (int)dim,
                         accumulate, cur_stream());
}

void layernorm_fwd(const Tensor& x, const Tensor& gamma, const OptTensor& beta, Tensor& y, double eps) {
  chk_c(x, BF16, "x");
  chk_c(gamma, BF16, "gamma");
  chk_c(y, BF16, "y");
  const int64_t dim = x.size(-1), rows = x.numel() / dim;
  c10::cuda::CUDAGuard guard(x.device());
  mb::layernorm_fwd(x.data_ptr(), gamma.data_ptr(), cptr(beta), y.data_ptr(), (int)rows, (int)dim, (float)eps,
                    cur_stream());
}

// x: [tokens, heads, head_dim] view (heads/head_dim contiguous, arbitrary token stride), rotated in place.
void rope(Tensor& x, const Tensor& pos, double theta, bool inverse) {
  chk(x, BF16, "x");
  chk_c(pos, I32, "pos");
  TORCH_CHECK(x.dim() == 3 && x.stride(2) == 1 && x.stride(1) == x.size(2), "rope: x must be [tokens, heads, head_dim]");
  TORCH_CHECK(pos.numel() == x.size(0), "rope: one position per token");
  c10::cuda::CUDAGuard guard(x.device());
  mb::rope_apply(x.data_ptr(), pos.data_ptr<int>(), (int)x.size(0), (int)x.size(1), (int)x.size(2), x.stride(0),
                 (float)theta, inverse, cur_stream());
}

void swiglu_fused_fwd(const Tensor& gate_up, Tensor& out) {
  chk_c(gate_up, BF16, "gate_up");
  chk_c(out, BF16, "out");
  const int64_t ffn = gate_up.size(-1) / 2, rows = gate_up.numel() / (2 * ffn);
  c10::cuda::CUDAGuard guard(out.device());
  mb::swiglu_fused_fwd(gate_up.data_ptr(), out.data_ptr(), rows, (int)ffn, cur_stream());
}
void swiglu_fused_bwd(const Tensor& gate_up, const Tensor& dout, Tensor& dgate_up) {
  chk_c(gate_up, BF16, "gate_up");
  chk_c(dout, BF16, "dout");
  chk_c(dgate_up, BF16, "dgate_up");
  const int64_t ffn = gate_up.size(-1) / 2, rows = gate_up.numel() / (2 * ffn);
  c10::cuda::CUDAGuard guard(dout.device());
  mb::swiglu_fused_bwd(gate_up.data_ptr(), dout.data_ptr(), dgate_up.data_ptr(), rows, (int)ffn, cur_stream());
}
void swiglu_fwd(const Tensor& gate, const Tensor& up, Tensor& out) {
  chk_c(gate, BF16, "gate");
  chk_c(up, BF16, "up");
  chk_c(out, BF16, "out");
  c10::cuda::CUDAGuard guard(out.device());
  mb::swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), cur_stream());
}
void swiglu_bwd(const Tensor& gate, const Tensor& up, const Tensor& dout, Tensor& dgate, Tensor& dup) {
  chk_c(gate, BF16, "gate");
  chk_c(up, BF16, "up");
  chk_c(dout, BF16, "dout");
  chk_c(dgate, BF16, "dgate");
  chk_c(dup, BF16, "dup");
  c10::cuda::CUDAGuard guard(dout.device());
  mb::swiglu_bwd(gate.data_ptr(), up.data_ptr(), dout.data_ptr(), dgate.data_ptr(), dup.data_ptr(), gate.numel(),
                 cur_stream());
}
void relu2_fwd(const Tensor& x, Tensor& out) {
  chk_c(x, BF16, "x");
  chk_c(out, BF16, "out");
  c10::cuda::CUDAGuard guard(x.device());
  mb::relu2_fwd(x.data_ptr(), out.data_ptr(), x.numel(), cur_stream());
}
void relu2_bwd(const Tensor& x, const Tensor& dout, Tensor& dx) {
  chk_c(x, BF16, "x");
  chk_c(dout, BF16, "dout");
  chk_c(dx, BF16, "dx");
  c10::cuda::CUDAGuard guard(x.device());
  mb::relu2_bwd(x.data_ptr(), dout.data_ptr(), dx.data_ptr(), x.numel(), cur_stream());
}
void act_fwd(const Tensor& x, Tensor& out, int64_t kind) {
  chk_c(x, BF16, "x");
  chk_c(out, BF16, "out");
  c10::cuda::CUDAGuard guard(x.device());
  mb::act_fwd(x.data_ptr(), out.data_ptr(), x.numel(), (int)kind, cur_stream());
}
void act_bwd(const Tensor& x, const Tensor& dout, Tensor& dx, int64_t kind) {
  chk_c(x, BF16, "x");
  chk_c(dout, BF16, "dout");
  chk_c(dx, BF16, "dx");
  TORCH_CHECK(dout.numel() == x.numel() && dx.numel() == x.numel(), "act_bwd: shape mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  mb::act_bwd(x.data_ptr(), dout.data_ptr(), dx.data_ptr(), x.numel(), (int)kind, cur_stream());
}
void softmax_rows_bwd(const Tensor& y, const Tensor& dy, Tensor& dx) {
  chk_c(y, BF16, "y");
  chk_c(dy, BF16, "dy");
  chk_c(dx, BF16, "dx");
  TORCH_CHECK(dy.numel() == y.numel() && dx.numel() == y.numel(), "softmax_rows_bwd: shape mismatch");
  const int64_t cols = y.size(-1);
  c10::cuda::CUDAGuard guard(y.device());
  mb::softmax_rows_bwd(y.data_ptr(), dy.data_ptr(), dx.data_ptr(), (int)(y.numel() / cols), (int)cols, cur_stream());
}
void layernorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& gamma, Tensor& dx, Tensor& partial, Tensor& dgb,
                   double eps) {
  chk_c(dy, BF16, "dy");
  chk_c(x, BF16, "x");
  chk_c(gamma, BF16, "gamma");
  chk_c(dx, BF16, "dx");
  chk_c(partial, F32, "partial");
  chk_c(dgb, F32, "dgb");
  const int64_t dim = x.size(-1), rows = x.numel() / dim;
  TORCH_CHECK(dy.numel() == x.numel() && dx.numel() == x.numel() && gamma.numel() == dim, "layernorm_bwd: shape mismatch");
  TORCH_CHECK(partial.dim() == 2 && partial.size(1) == 2 * dim && dgb.numel() == 2 * dim,
              "layernorm_bwd: partial must be [n, 2 * dim] and dgb [2 * dim]");
  c10::cuda::CUDAGuard guard(x.device());
  mb::layernorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), dx.data_ptr(), partial.data_ptr<float>(),
                    (int)partial.size(0), (int)rows, (int)dim, (float)eps, cur_stream());
  mb::rmsnorm_bwd_reduce(partial.data_ptr<float>(), dgb.data_ptr<float>(), (int)partial.size(0), (int)(2 * dim), false,
                         cur_stream());
}
void add(const Tensor& a, const Tensor& b, Tensor& out) {
  chk_c(a, BF16, "a");
  chk_c(b, BF16, "b");
  chk_c(out, BF16, "out");
  c10::cuda::CUDAGuard guard(a.device());
  mb::add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), cur_stream());
}
void softmax_rows(const Tensor& x, Tensor& y) {
  chk_c(x, BF16, "x");
  chk_c(y, BF16, "y");
  const int64_t cols = x.size(-1);
  c10::cuda::CUDAGuard guard(x.device());
  mb::softmax_rows(x.data_ptr(), y.data_ptr(), (int)(x.numel() / cols), (int)cols, cur_stream());
}

void embedding_fwd(const Tensor& ids, const Tensor& table, Tensor& out) {
  chk_c(ids, I32, "ids");
  chk_c(table, BF16, "table");
  chk_c(out, BF16, "out");
  c10::cuda::CUDAGuard guard(table.device());
  mb::embedding_fwd(ids.data_ptr<int>(), table.data_ptr(), out.data_ptr(), (int)ids.numel(), (int)table.size(1),
                    (int)table.size(0), cur_stream());
}
void embedding_bwd(const Tensor& ids, const Tensor& dout, Tensor& dtable) {
  chk_c(ids, I32, "ids");
  chk_c(dout, BF16, "dout");
  chk_c(dtable, F32, "dtable");
  c10::cuda::CUDAGuard guard(dout.device());
  mb::embedding_bwd(ids.data_ptr<int>(), dout.data_ptr(), dtable.data_ptr<float>(), (int)ids.numel(),
                    (int)dtable.size(1), (int)dtable.size(0), cur_stream());
}

void cross_entropy_fwd_bwd(Tensor& logits, const Tensor& targets, Tensor& losses, double grad_scale) {
  chk(logits, BF16, "logits");
  chk_c(targets, I32, "targets");
  chk_c(losses, F32, "losses");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "cross_entropy: logits must be [rows, vocab]");
  c10::cuda::CUDAGuard guard(logits.device());
  mb::cross_entropy_fwd_bwd(logits.data_ptr(), targets.data_ptr<int>(), losses.data_ptr<float>(), (int)logits.size(0),
                            (int)logits.size(1), logits.stride(0), (float)grad_scale, cur_stream());
}
void cross_entropy_fwd(const Tensor& logits, const Tensor& targets, Tensor& losses) {
  chk(logits, BF16, "logits");
  chk_c(targets, I32, "targets");
  chk_c(losses, F32, "losses");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "cross_entropy: logits must be [rows, vocab]");
  c10::cuda::CUDAGuard guard(logits.device());
  mb::cross_entropy_fwd(logits.data_ptr(), targets.data_ptr<int>(), losses.data_ptr<float>(), (int)logits.size(0),
                        (int)logits.size(1), logits.stride(0), cur_stream());
}

void cross_entropy_shard_stats(const Tensor& logits, const Tensor& targets, Tensor& stats, int64_t vocab_offset,
                               int64_t vocab_total) {
  chk(logits, BF16, "logits");
  chk_c(targets, I32, "targets");
  chk_c(stats, F32, "stats");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "cross_entropy_shard_stats: logits must be [rows, vocab]");
  TORCH_CHECK(stats.numel() == logits.size(0) * 3 && targets.numel() == logits.size(0),
              "cross_entropy_shard_stats: stats must be [rows, 3] and targets [rows]");
  c10::cuda::CUDAGuard guard(logits.device());
  mb::cross_entropy_shard_stats(logits.data_ptr(), targets.data_ptr<int>(), stats.data_ptr<float>(), (int)logits.size(0),
                                (int)logits.size(1), logits.stride(0), (int)vocab_offset, (int)vocab_total, cur_stream());
}
void cross_entropy_shard_grad(Tensor& logits, const Tensor& targets, const Tensor& lse, int64_t vocab_offset,
                              int64_t vocab_total, double grad_scale) {
  chk(logits, BF16, "logits");
  chk_c(targets, I32, "targets");
  chk_c(lse, F32, "lse");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "cross_entropy_shard_grad: logits must be [rows, vocab]");
  TORCH_CHECK(lse.numel() == logits.size(0) && targets.numel() == logits.size(0),
              "cross_entropy_shard_grad: lse and targets must be [rows]");
  c10::cuda::CUDAGuard guard(logits.device());
  mb::cross_entropy_shard_grad(logits.data_ptr(), targets.data_ptr<int>(), lse.data_ptr<float>(), (int)logits.size(0),
                               (int)logits.size(1), logits.stride(0), (int)vocab_offset, (int)vocab_total,
                               (float)grad_scale, cur_stream());
}

void adamw_step(Tensor& p, Tensor& m, Tensor& v, const Tensor& g, OptTensor p_bf16, double lr, double beta1,
                double beta2, double eps, double weight_decay, int64_t step, double grad_scale,
                const OptTensor& clip_coef) {
  chk_c(p, F32, "p");
  chk_c(m, F32, "m");
  chk_c(v, F32, "v");
  chk_c(g, F32, "g");
  mb::AdamWArgs a;
  a.lr = (float)lr;
  a.beta1 = (float)beta1;
  a.beta2 = (float)beta2;
  a.eps = (float)eps;
  a.weight_decay = (float)weight_decay;
  a.bc1 = (float)(1.0 - std::pow(beta1, (double)step));
  a.bc2 = (float)(1.0 - std::pow(beta2, (double)step));
  a.grad_scale = (float)grad_scale;
  c10::cuda::CUDAGuard guard(p.device());
  mb::adamw_step(p.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(), mptr(p_bf16),
                 p.numel(), a, clip_coef.has_value() ? clip_coef->data_ptr<float>() : nullptr, cur_stream());
}
void sumsq(const Tensor& x, Tensor& out) {
  chk_c(x, F32, "x");
  chk_c(out, F32, "out");
  c10::cuda::CUDAGuard guard(x.device());
  mb::sumsq_f32(x.data_ptr<float>(), x.numel(), out.data_ptr<float>(), cur_stream());
}
void oil_fake_quant(const Tensor& w, const Tensor& codebooks, const OptTensor& cb_map, int64_t bs, OptTensor w_bf16,
                    OptTensor idx) {
  chk_c(w, F32, "w");
  chk_c(codebooks, F32, "codebooks");
  c10::cuda::CUDAGuard guard(w.device());
  mb::oil_fake_quant(w.data_ptr<float>(), codebooks.data_ptr<float>(),
                     cb_map.has_value() ? cb_map->data_ptr<int>() : nullptr, (int)codebooks.size(-1), (int)bs,
                     w.numel(), mptr(w_bf16), idx.has_value() ? idx->data_ptr<uint8_t>() : nullptr, cur_stream());
}
void i2s_fake_quant(const Tensor& w, int64_t bs, OptTensor w_bf16, OptTensor trits, OptTensor scales) {
  chk_c(w, F32, "w");
  c10::cuda::CUDAGuard guard(w.device());
  mb::i2s_fake_quant(w.data_ptr<float>(), (int)bs, w.numel(), mptr(w_bf16),
                     trits.has_value() ? trits->data_ptr<uint8_t>() : nullptr,
                     scales.has_value() ? scales->data_ptr<float>() : nullptr, cur_stream());
}
void cast_f32_to_bf16(const Tensor& x, Tensor& y) {
  chk_c(x, F32, "x");
  chk_c(y, BF16, "y");
  c10::cuda::CUDAGuard guard(x.device());
  mb::cast_f32_to_bf16(x.data_ptr<float>(), y.data_ptr(), x.numel(), cur_stream());
}
void cast_bf16_to_f32(const Tensor& x, Tensor& y, bool accumulate) {
  chk_c(x, BF16, "x");
  chk_c(y, F32, "y");
  c10::cuda::CUDAGuard guard(x.device());
  mb::cast_bf16_to_f32(x.data_ptr(), y.data_ptr<float>(), x.numel(), accumulate, cur_stream());
}
void oil_codebook_stats(const Tensor& w, const Tensor& idx, const OptTensor& cb_map, int64_t cb_size, int64_t bs,
                        Tensor& counts, Tensor& sums) {
  chk_c(w, F32, "w");
  chk_c(idx, U8, "idx");
  chk_c(counts, F32, "counts");
  chk_c(sums, F32, "sums");
  c10::cuda::CUDAGuard guard(w.device());
  mb::oil_codebook_stats(w.data_ptr<float>(), idx.data_ptr<uint8_t>(),
                         cb_map.has_value() ? cb_map->data_ptr<int>() : nullptr, (int)cb_size, (int)bs, w.numel(),
                         counts.data_ptr<float>(), sums.data_ptr<float>(), cur_stream());
}

// q: [B,S,H,D] view, k/v: [B,S,Hkv,D] views (last two dims contiguous, batch stride = S * token stride).
void flash_attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& o, Tensor& lse, bool causal,
                    double scale, const OptTensor& status) {
  chk(q, BF16, "q");
  chk(k, BF16, "k");
  chk(v, BF16, "v");
  chk(o, BF16, "o");
  chk_c(lse, F32, "lse");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4 && o.dim() == 4, "flash_attn: tensors must be [B,S,H,D]");
  const int64_t B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3), Hkv = k.size(2);
  auto ok_view = [&](const Tensor& t) {
    return t.stride(3) == 1 && t.stride(2) == D && t.stride(0) == t.stride(1) * S;
  };
  TORCH_CHECK(ok_view(q) && ok_view(k) && ok_view(v) && ok_view(o), "flash_attn: unsupported strides");
  TORCH_CHECK(k.stride(1) == v.stride(1), "flash_attn: k and v must share a token stride");
  c10::cuda::CUDAGuard guard(q.device());
  mb::flash_attn_fwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), (int)B,
                             (int)S, (int)H, (int)Hkv, (int)D, q.stride(1), k.stride(1), o.stride(1), causal,
                             (float)scale, status_ptr(status), cur_stream());
}

void flash_attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& dout,
                    const Tensor& lse, Tensor& dq, Tensor& dk, Tensor& dv, Tensor& dq_accum, Tensor& delta,
                    bool causal, double scale, const OptTensor& status, const OptTensor& rope_pos,
                    const OptTensor& rope_table) {
  chk(q, BF16, "q");
  chk(k, BF16, "k");
  chk(v, BF16, "v");
  chk_c(o, BF16, "o");
  chk_c(dout, BF16, "dout");
  chk_c(lse, F32, "lse");
  chk(dq, BF16, "dq");
  chk(dk, BF16, "dk");
  chk(dv, BF16, "dv");
  chk_c(dq_accum, F32, "dq_accum");
  chk_c(delta, F32, "delta");
  const int64_t B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3), Hkv = k.size(2);
  auto ok_view = [&](const Tensor& t) {
    return t.stride(3) == 1 && t.stride(2) == D && t.stride(0) == t.stride(1) * S;
  };
  TORCH_CHECK(ok_view(q) && ok_view(k) && ok_view(v) && ok_view(dq) && ok_view(dk) && ok_view(dv),
              "flash_attn_bwd: unsupported strides");
  TORCH_CHECK(k.stride(1) == v.stride(1) && dk.stride(1) == dv.stride(1),
              "flash_attn_bwd: k/v and dk/dv must share a token stride");
  TORCH_CHECK(dq_accum.numel() >= B * S * H * D && delta.numel() >= B * H * S, "flash_attn_bwd: scratch too small");
  const int* pos_ptr = nullptr;
  const float* cs_ptr = nullptr;
  int max_pos = 0;
  if (rope_table.has_value()) {
    TORCH_CHECK(rope_pos.has_value(), "flash_attn_bwd: rope_table needs rope_pos");
    chk_c(*rope_table, F32, "rope_table");
    chk_c(*rope_pos, torch::kInt32, "rope_pos");
    TORCH_CHECK(D == 128 && rope_table->dim() == 3 && rope_table->size(1) == 64 && rope_table->size(2) == 2,
                "flash_attn_bwd: rope_table must be [max_pos, 64, 2] (head_dim 128)");
    TORCH_CHECK(rope_pos->numel() == B * S, "flash_attn_bwd: rope_pos must have batch * seq entries");
    pos_ptr = rope_pos->data_ptr<int>();
    cs_ptr = rope_table->data_ptr<float>();
    max_pos = (int)rope_table->size(0);
  }
  c10::cuda::CUDAGuard guard(q.device());
  mb::flash_attn_bwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(),
                             lse.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                             dq_accum.data_ptr<float>(), delta.data_ptr<float>(), (int)B, (int)S, (int)H, (int)Hkv,
                             (int)D, q.stride(1), k.stride(1), dq.stride(1), dk.stride(1), causal, (float)scale,
                             status_ptr(status), cur_stream(), pos_ptr, cs_ptr, max_pos);
}

mb::PeerPtrs to_peers(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() <= (size_t)mb::MAX_PEERS, "too many peers");
  mb::PeerPtrs pp{};
  for (size_t i = 0; i < ptrs.size(); ++i) pp.p[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(ptrs[i]));
  return pp;
}

// flag_ptrs / slot_ptrs: per-rank addresses (as mapped in this process) of the int32 flag array and
// the fp32 slot array. send_val: optional 1-element fp32 tensor delivered to every rank.
void symm_barrier(const std::vector<int64_t>& flag_ptrs, const std::vector<int64_t>& slot_ptrs,
                  const OptTensor& send_val, int64_t rank, int64_t epoch, int64_t limit_cycles,
                  const OptTensor& status, const OptTensor& epoch_dev) {
  mb::symm_barrier(to_peers(flag_ptrs), to_peers(slot_ptrs),
                   send_val.has_value() ? send_val->data_ptr<float>() : nullptr, (int)rank, (int)flag_ptrs.size(),
                   (int)epoch, epoch_dev.has_value() ? epoch_dev->data_ptr<int>() : nullptr, limit_cycles,
                   status_ptr(status), cur_stream());
}

// a_ptrs: every rank's [M, K] bf16 buffer as mapped here; w: [N, K]; out: [M, N]; tile_count: int32 [M / 256].
void gemm_allgather_a(const std::vector<int64_t>& a_ptrs, int64_t M, int64_t K, const Tensor& w, Tensor& out,
                      int64_t rank, Tensor& tile_count, int64_t call, int64_t copier_clusters, const OptTensor& status) {
  chk(w, BF16, "w");
  chk(out, BF16, "out");
  chk_c(tile_count, torch::kInt32, "tile_count");
  TORCH_CHECK(w.dim() == 2 && w.size(1) == K && w.stride(1) == 1, "gemm_allgather_a: w must be [N, K] with unit inner stride");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == M && out.size(1) == w.size(0) && out.stride(1) == 1,
              "gemm_allgather_a: out must be [M, N]");
  TORCH_CHECK(tile_count.numel() >= M / 256, "gemm_allgather_a: tile_count too small");
  c10::cuda::CUDAGuard guard(w.device());
  mb::gemm_allgather_a(to_peers(a_ptrs), K, w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), (int)M,
                       (int)w.size(0), (int)K, (int)rank, (int)a_ptrs.size(), tile_count.data_ptr<int>(), (int)call,
                       (int)copier_clusters, status_ptr(status), cur_stream());
}

// x: [M, K]; w_ptrs: every rank's [N, K] bf16 weight buffer as mapped here; out: [M, N]; tile_count: int32 [N / 256].
void gemm_allgather_b(const Tensor& x, const std::vector<int64_t>& w_ptrs, int64_t N, Tensor& out, int64_t rank,
                      Tensor& tile_count, int64_t call, int64_t copier_clusters, const OptTensor& status) {
  chk(x, BF16, "x");
  chk(out, BF16, "out");
  chk_c(tile_count, torch::kInt32, "tile_count");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "gemm_allgather_b: x must be [M, K] with unit inner stride");
  const int64_t M = x.size(0), K = x.size(1);
  TORCH_CHECK(out.dim() == 2 && out.size(0) == M && out.size(1) == N && out.stride(1) == 1, "gemm_allgather_b: out must be [M, N]");
  TORCH_CHECK(tile_count.numel() >= N / 256, "gemm_allgather_b: tile_count too small");
  c10::cuda::CUDAGuard guard(x.device());
  mb::gemm_allgather_b(x.data_ptr(), x.stride(0), to_peers(w_ptrs), K, out.data_ptr(), out.stride(0), (int)M, (int)N, (int)K,
                       (int)rank, (int)w_ptrs.size(), tile_count.data_ptr<int>(), (int)call, (int)copier_clusters,
                       status_ptr(status), cur_stream());
}

std::vector<int64_t> comm_barrier_wait_stats(bool reset) {
  unsigned long long v[3];
  mb::comm_barrier_wait_stats(v, reset);
  return {(int64_t)v[0], (int64_t)v[1], (int64_t)v[2]};
}

void zero_reduce_scatter(const std::vector<int64_t>& grad_ptrs, Tensor& out, int64_t shard_off, Tensor& sumsq,
                         int64_t multicast_ptr, int64_t max_blocks, OptTensor scratch) {
  chk_c(out, F32, "out");
  chk_c(sumsq, F32, "sumsq");
  if (scratch.has_value()) chk_c(*scratch, F32, "scratch");
  c10::cuda::CUDAGuard guard(out.device());
  mb::zero_reduce_scatter(to_peers(grad_ptrs), out.data_ptr<float>(), shard_off, out.numel(), (int)grad_ptrs.size(),
                          sumsq.data_ptr<float>(), cur_stream(), reinterpret_cast<const float*>(multicast_ptr),
                          (int)max_blocks, scratch.has_value() ? scratch->data_ptr<float>() : nullptr,
                          scratch.has_value() ? scratch->numel() : 0);
}
void tp_allreduce_multimem(int64_t part_mc, int64_t out_mc, int64_t n_peers, int64_t rank, int64_t n) {
  mb::tp_allreduce_multimem(reinterpret_cast<const void*>(part_mc), reinterpret_cast<void*>(out_mc), (int)n_peers, (int)rank,
                            n, cur_stream());
}

void zero_adamw_ste_allgather(Tensor& p, Tensor& m, Tensor& v, const Tensor& g,
                              const std::vector<int64_t>& compute_ptrs, int64_t shard_off, const OptTensor& seg_fmt,
                              const OptTensor& seg_cb, const OptTensor& codebooks8, const OptTensor& codebooks4,
                              const Tensor& norm_partials, OptTensor grad_norm_out, double max_norm, double lr,
                              double beta1, double beta2, double eps, double weight_decay, int64_t step,
                              double grad_scale, int64_t rank, int64_t compute_multicast_ptr) {
  chk_c(p, F32, "p");
  chk_c(m, F32, "m");
  chk_c(v, F32, "v");
  chk_c(g, F32, "g");
  chk_c(norm_partials, F32, "norm_partials");
  mb::ZeroFusedArgs a{};
  a.p = p.data_ptr<float>();
  a.m = m.data_ptr<float>();
  a.v = v.data_ptr<float>();
  a.g = g.data_ptr<float>();
  a.compute = to_peers(compute_ptrs);
  a.compute_mc = reinterpret_cast<void*>(compute_multicast_ptr);
  a.shard_off = shard_off;
  a.n = p.numel();
  a.seg_fmt = seg_fmt.has_value() ? seg_fmt->data_ptr<uint8_t>() : nullptr;
  a.seg_cb = seg_cb.has_value() ? seg_cb->data_ptr<int>() : nullptr;
  a.codebooks8 = codebooks8.has_value() ? codebooks8->data_ptr<float>() : nullptr;
  a.codebooks4 = codebooks4.has_value() ? codebooks4->data_ptr<float>() : nullptr;
  a.norm_partials = norm_partials.data_ptr<float>();
  a.grad_norm_out = grad_norm_out.has_value() ? grad_norm_out->data_ptr<float>() : nullptr;
  a.max_norm = (float)max_norm;
  a.opt.lr = (float)lr;
  a.opt.beta1 = (float)beta1;
  a.opt.beta2 = (float)beta2;
  a.opt.eps = (float)eps;
  a.opt.weight_decay = (float)weight_decay;
  a.opt.bc1 = (float)(1.0 - std::pow(beta1, (double)step));
  a.opt.bc2 = (float)(1.0 - std::pow(beta2, (double)step));
  a.opt.grad_scale = (float)grad_scale;
  a.rank = (int)rank;
  a.world = (int)compute_ptrs.size();
  TORCH_CHECK((int64_t)norm_partials.numel() >= a.world, "norm_partials needs one slot per rank");
  c10::cuda::CUDAGuard guard(p.device());
  mb::zero_adamw_ste_allgather(a, cur_stream());
}

mb::DequantWeights to_weights(const Tensor& packed, const OptTensor& codebooks, const OptTensor& cb_map,
                              const OptTensor& scales, int64_t fmt, int64_t N, int64_t K, int64_t block_size) {
  chk_c(packed, U8, "packed");
  mb::DequantWeights w{};
  w.packed = packed.data_ptr<uint8_t>();
  if (codebooks.has_value()) {
    chk_c(*codebooks, BF16, "codebooks");
    w.codebooks = codebooks->data_ptr();
    w.n_codebooks = (int)codebooks->size(0);
  }
  if (cb_map.has_value()) {
    chk_c(*cb_map, I32, "cb_map");
    w.cb_map = cb_map->data_ptr<int>();
  }
  if (scales.has_value()) {
    chk_c(*scales, F32, "scales");
    w.scales = scales->data_ptr<float>();
  }
  w.fmt = (int)fmt;
  w.N = (int)N;
  w.K = (int)K;
  w.block_size = (int)block_size;
  const int64_t need = fmt == mb::QFMT_OIL8 ? N * K : (fmt == mb::QFMT_OIL4 ? N * K / 2 : N * K / 4);
  TORCH_CHECK(packed.numel() >= need, "packed weight buffer too small: ", packed.numel(), " < ", need);
  TORCH_CHECK(fmt == mb::QFMT_I2S ? scales.has_value() : codebooks.has_value(), "missing codebooks / scales");
  return w;
}

// y = x @ dequant(W)^T. out: bf16 [M,N] (direct) or fp32 [M,N] accumulator; peer_ptrs: fp32
// accumulators of all ranks (fused all-reduce), in which case `out` is ignored.
void dequant_gemm(const Tensor& x, const Tensor& packed, const OptTensor& codebooks, const OptTensor& cb_map,
                  const OptTensor& scales, int64_t fmt, int64_t N, int64_t K, int64_t block_size, OptTensor out,
                  const std::vector<int64_t>& peer_ptrs, int64_t k_splits, const OptTensor& status,
                  int64_t peer_bf16_offset) {
  chk(x, BF16, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.size(1) == K, "dequant_gemm: x must be [M, K]");
  const auto w = to_weights(packed, codebooks, cb_map, scales, fmt, N, K, block_size);
  void* o16 = nullptr;
  float* o32 = nullptr;
  int64_t ld = N;
  if (peer_ptrs.empty()) {
    TORCH_CHECK(out.has_value(), "dequant_gemm: need an output tensor");
    TORCH_CHECK(out->dim() == 2 && out->size(0) == x.size(0) && out->size(1) == N && out->stride(1) == 1,
                "dequant_gemm: output must be [M, N]");
    ld = out->stride(0);
    if (out->scalar_type() == BF16) o16 = out->data_ptr();
    else {
      chk(*out, F32, "out");
      o32 = out->data_ptr<float>();
    }
  }
  const mb::PeerPtrs pp = to_peers(peer_ptrs);
  c10::cuda::CUDAGuard guard(x.device());
  mb::dequant_gemm(x.data_ptr(), x.stride(0), (int)x.size(0), w, o16, o32, peer_ptrs.empty() ? nullptr : &pp,
                   (int)peer_ptrs.size(), ld, (int)k_splits, status_ptr(status), cur_stream(), peer_bf16_offset);
}

void tp_push(Tensor& acc, const std::vector<int64_t>& ptrs, int64_t rank, int64_t slot_off) {
  chk_c(acc, F32, "acc");
  c10::cuda::CUDAGuard guard(acc.device());
  mb::tp_push(acc.data_ptr<float>(), to_peers(ptrs), (int)ptrs.size(), (int)rank, slot_off, acc.numel(), cur_stream());
}
void tp_reduce_slots(const Tensor& staging, int64_t slots, int64_t slot_stride, const OptTensor& residual, Tensor& out) {
  chk_c(staging, BF16, "staging");
  chk_c(out, BF16, "out");
  TORCH_CHECK(staging.numel() >= (slots - 1) * slot_stride + out.numel(), "tp_reduce_slots: staging too small");
  c10::cuda::CUDAGuard guard(out.device());
  mb::tp_reduce_slots(staging.data_ptr(), (int)slots, slot_stride, cptr(residual), out.data_ptr(), out.numel(),
                      cur_stream());
}
// part_ptrs / out_ptrs: every rank's partial and output buffer; n elements of each take part.
void tp_allreduce_pull(const std::vector<int64_t>& part_ptrs, const std::vector<int64_t>& out_ptrs, int64_t rank,
                       int64_t n) {
  TORCH_CHECK(part_ptrs.size() == out_ptrs.size(), "tp_allreduce_pull: peer lists differ in length");
  mb::tp_allreduce_pull(to_peers(part_ptrs), to_peers(out_ptrs), (int)part_ptrs.size(), (int)rank, n, cur_stream());
}

void tp_reduce_scatter_pull(const std::vector<int64_t>& part_ptrs, int64_t rank, int64_t n, Tensor& out) {
  chk_c(out, BF16, "out");
  TORCH_CHECK(out.numel() * (int64_t)part_ptrs.size() == n, "tp_reduce_scatter_pull: out must hold n / ranks elements");
  c10::cuda::CUDAGuard guard(out.device());
  mb::tp_reduce_scatter_pull(to_peers(part_ptrs), (int)part_ptrs.size(), (int)rank, n, out.data_ptr(), cur_stream());
}

// x [M, K] @ w [N, K]^T with the output rows scattered to their owner ranks (fused reduce-scatter).
void gemm_reduce_scatter(const Tensor& x, const Tensor& w, const std::vector<int64_t>& slot_ptrs, int64_t rank,
                         int64_t rows_per_rank, int64_t slot_stride, const OptTensor& status) {
  chk(x, BF16, "x");
  chk(w, BF16, "w");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.size(1) == w.size(1) && x.stride(1) == 1 && w.stride(1) == 1,
              "gemm_reduce_scatter: x [M, K], w [N, K]");
  const mb::PeerPtrs pp = to_peers(slot_ptrs);
  c10::cuda::CUDAGuard guard(x.device());
  mb::gemm_bf16_2cta_scatter(x.data_ptr(), x.stride(0), false, w.data_ptr(), w.stride(0), false, nullptr, w.size(0),
                             (int)x.size(0), (int)w.size(0), (int)x.size(1), mb::EPI_BF16, 1.0f, status_ptr(status),
                             cur_stream(), &pp, (int)slot_ptrs.size(), rows_per_rank, rank * slot_stride);
}
void tp_reduce_slots_bcast(const Tensor& staging, int64_t slots, int64_t slot_stride,
                           const std::vector<int64_t>& out_ptrs, int64_t rank, int64_t out_off, int64_t n) {
  chk_c(staging, BF16, "staging");
  c10::cuda::CUDAGuard guard(staging.device());
  mb::tp_reduce_slots_bcast(staging.data_ptr(), (int)slots, slot_stride, to_peers(out_ptrs), (int)out_ptrs.size(),
                            (int)rank, out_off, n, cur_stream());
}

void sum_residual_rmsnorm(OptTensor acc, const OptTensor& slots, int64_t n_slots, int64_t slot_stride,
                          const OptTensor& residual, const Tensor& gamma, Tensor& stream_out, Tensor& normed,
                          double eps) {
  chk_c(gamma, BF16, "gamma");
  chk_c(stream_out, BF16, "stream_out");
  chk_c(normed, BF16, "normed");
  if (acc.has_value()) chk_c(*acc, F32, "acc");
  if (slots.has_value()) chk_c(*slots, BF16, "slots");
  if (residual.has_value()) chk_c(*residual, BF16, "residual");
  const int64_t dim = normed.size(-1), rows = normed.numel() / dim;
  TORCH_CHECK(stream_out.numel() == normed.numel() && gamma.numel() == dim, "sum_residual_rmsnorm: shape mismatch");
  c10::cuda::CUDAGuard guard(normed.device());
  mb::sum_residual_rmsnorm(acc.has_value() ? acc->data_ptr<float>() : nullptr, cptr(slots), (int)n_slots, slot_stride,
                           cptr(residual), gamma.data_ptr(), stream_out.data_ptr(), normed.data_ptr(), (int)rows,
                           (int)dim, (float)eps, cur_stream());
}
void tp_sum_residual_rmsnorm(OptTensor acc, const std::vector<int64_t>& staging_ptrs,
                             const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t slot_stride, int64_t parity,
                             int64_t max_rows, const OptTensor& residual, const Tensor& gamma, Tensor& stream_out,
                             Tensor& normed, double eps, Tensor& epoch_dev, Tensor& arrive, int64_t limit_cycles,
                             const OptTensor& status) {
  chk_c(gamma, BF16, "gamma");
  chk_c(stream_out, BF16, "stream_out");
  chk_c(normed, BF16, "normed");
  chk_c(epoch_dev, I32, "epoch_dev");
  chk_c(arrive, I32, "arrive");
  if (acc.has_value()) chk_c(*acc, F32, "acc");
  if (residual.has_value()) chk_c(*residual, BF16, "residual");
  const int64_t dim = normed.size(-1), rows = normed.numel() / dim;
  TORCH_CHECK(stream_out.numel() == normed.numel() && gamma.numel() == dim, "tp_sum_residual_rmsnorm: shape mismatch");
  TORCH_CHECK(!acc.has_value() || acc->numel() >= rows * dim, "tp_sum_residual_rmsnorm: accumulator too small");
  TORCH_CHECK(staging_ptrs.size() == flag_ptrs.size() && !staging_ptrs.empty(),
              "tp_sum_residual_rmsnorm: one staging and one flag pointer per rank");
  c10::cuda::CUDAGuard guard(normed.device());
  mb::tp_sum_residual_rmsnorm(acc.has_value() ? acc->data_ptr<float>() : nullptr, to_peers(staging_ptrs),
                              to_peers(flag_ptrs), (int)rank, (int)staging_ptrs.size(), slot_stride, (int)parity,
                              (int)max_rows, cptr(residual), gamma.data_ptr(), stream_out.data_ptr(), normed.data_ptr(),
                              (int)rows, (int)dim, (float)eps, epoch_dev.data_ptr<int>(), arrive.data_ptr<int>(),
                              limit_cycles, status_ptr(status), cur_stream());
}
void qkv_rope_append(Tensor& acc, const Tensor& pos, const Tensor& seq_ids, const Tensor& block_table, Tensor& q_out,
                     Tensor& k_cache, Tensor& v_cache, double theta, OptTensor k_scale, OptTensor v_scale) {
  chk_c(acc, F32, "acc");
  chk_c(pos, I32, "pos");
  chk_c(seq_ids, I32, "seq_ids");
  chk_c(block_table, I32, "block_table");
  chk_c(q_out, BF16, "q_out");
  const bool int8 = k_scale.has_value();
  TORCH_CHECK(int8 == v_scale.has_value(), "qkv_rope_append: give both scale tensors or neither");
  chk_c(k_cache, int8 ? torch::kInt8 : BF16, "k_cache");
  chk_c(v_cache, int8 ? torch::kInt8 : BF16, "v_cache");
  const int64_t T = q_out.size(0), H = q_out.size(1), D = q_out.size(2), Hkv = k_cache.size(2);
  TORCH_CHECK(acc.numel() == T * (H + 2 * Hkv) * D, "qkv_rope_append: accumulator shape mismatch");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.size(3) == D, "qkv_rope_append: cache must be [pages, page, kv_heads, D]");
  if (int8) {
    chk_c(*k_scale, F32, "k_scale");
    chk_c(*v_scale, F32, "v_scale");
    const int64_t rows = k_cache.size(0) * k_cache.size(1) * Hkv;
    TORCH_CHECK(k_scale->numel() == rows && v_scale->numel() == rows, "qkv_rope_append: one scale per (token, kv head)");
  }
  c10::cuda::CUDAGuard guard(acc.device());
  mb::qkv_rope_append(acc.data_ptr<float>(), pos.data_ptr<int>(), seq_ids.data_ptr<int>(), block_table.data_ptr<int>(),
                      q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), (int)T, (int)H, (int)Hkv, (int)D,
                      (int)k_cache.size(1), (int)block_table.size(1), (float)theta, cur_stream(),
                      int8 ? k_scale->data_ptr<float>() : nullptr, int8 ? v_scale->data_ptr<float>() : nullptr);
}
void finalize_gate(Tensor& acc, Tensor& out, int64_t kind) {
  chk_c(acc, F32, "acc");
  chk_c(out, BF16, "out");
  const int64_t ffn = out.size(-1), rows = out.numel() / ffn;
  TORCH_CHECK(acc.numel() == 2 * out.numel(), "finalize_gate: accumulator must be [rows, 2 * ffn]");
  c10::cuda::CUDAGuard guard(acc.device());
  mb::finalize_gate(acc.data_ptr<float>(), out.data_ptr(), rows, (int)ffn, (int)kind, cur_stream());
}

void finalize_acc(Tensor& acc, const OptTensor& residual, Tensor& out) {
  chk_c(acc, F32, "acc");
  chk_c(out, BF16, "out");
  c10::cuda::CUDAGuard guard(acc.device());
  mb::finalize_acc(acc.data_ptr<float>(), cptr(residual), out.data_ptr(), out.numel(), cur_stream());
}

void dequant_to_bf16(const Tensor& packed, const OptTensor& codebooks, const OptTensor& cb_map, const OptTensor& scales,
                     int64_t fmt, int64_t N, int64_t K, int64_t block_size, Tensor& out) {
  chk_c(out, BF16, "out");
  TORCH_CHECK(out.numel() >= N * K, "dequant_to_bf16: output too small");
  const auto w = to_weights(packed, codebooks, cb_map, scales, fmt, N, K, block_size);
  c10::cuda::CUDAGuard guard(out.device());
  mb::dequant_to_bf16(w, out.data_ptr(), cur_stream());
}

void dequant_gather_rows(const Tensor& ids, const Tensor& packed, const OptTensor& codebooks, const OptTensor& cb_map,
                         const OptTensor& scales, int64_t fmt, int64_t N, int64_t K, int64_t block_size, Tensor& out) {
  chk_c(ids, I32, "ids");
  chk(out, BF16, "out");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == ids.numel() && out.size(1) == K && out.stride(1) == 1,
              "dequant_gather_rows: out must be [tokens, K] with unit inner stride");
  const auto w = to_weights(packed, codebooks, cb_map, scales, fmt, N, K, block_size);
  c10::cuda::CUDAGuard guard(out.device());
  mb::dequant_gather_rows(w, ids.data_ptr<int>(), (int)ids.numel(), out.data_ptr(), out.stride(0), cur_stream());
}

void i2s_gemv(const Tensor& x, const Tensor& packed, const Tensor& scales, int64_t N, int64_t K, int64_t block_size,
              Tensor& y) {
  chk_c(x, BF16, "x");
  chk_c(y, BF16, "y");
  const auto w = to_weights(packed, c10::nullopt, c10::nullopt, scales, mb::QFMT_I2S, N, K, block_size);
  c10::cuda::CUDAGuard guard(x.device());
  mb::i2s_gemv(x.data_ptr(), w, y.data_ptr(), cur_stream());
}

// k, v: [tokens, kv_heads, head_dim] views (token stride arbitrary); caches [pages, page, kv_heads, head_dim].
void kv_append(const Tensor& k, const Tensor& v, Tensor& k_cache, Tensor& v_cache, const Tensor& block_table,
               const Tensor& positions, const Tensor& seq_ids) {
  chk(k, BF16, "k");
  chk(v, BF16, "v");
  chk_c(k_cache, BF16, "k_cache");
  chk_c(v_cache, BF16, "v_cache");
  chk_c(block_table, I32, "block_table");
  chk_c(positions, I32, "positions");
  chk_c(seq_ids, I32, "seq_ids");
  TORCH_CHECK(k.dim() == 3 && k.stride(2) == 1 && k.stride(1) == k.size(2) && k.stride(0) == v.stride(0),
              "kv_append: k/v must be [tokens, kv_heads, head_dim] with a shared token stride");
  c10::cuda::CUDAGuard guard(k.device());
  mb::kv_append(k.data_ptr(), v.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr<int>(),
                positions.data_ptr<int>(), seq_ids.data_ptr<int>(), (int)k.size(0), (int)k.size(1), (int)k.size(2),
                (int)k_cache.size(1), (int)block_table.size(1), k.stride(0), cur_stream());
}

void paged_attn_decode(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_table,
                       const Tensor& context_lens, Tensor& out, Tensor& scratch, Tensor& counters, int64_t splits,
                       double scale, const OptTensor& status) {
  chk(q, BF16, "q");
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && q.stride(1) == q.size(2),
              "paged_attn_decode: q must be [batch, heads, head_dim] with contiguous heads");
  chk_c(k_cache, BF16, "k_cache");
  chk_c(v_cache, BF16, "v_cache");
  chk_c(block_table, I32, "block_table");
  chk_c(context_lens, I32, "context_lens");
  chk_c(out, BF16, "out");
  chk_c(scratch, F32, "scratch");
  chk_c(counters, I32, "counters");
  const int64_t B = q.size(0), H = q.size(1), D = q.size(2), Hkv = k_cache.size(2);
  TORCH_CHECK(scratch.numel() >= B * H * splits * (D + 2), "paged_attn_decode: scratch too small");
  TORCH_CHECK(counters.numel() >= B * Hkv, "paged_attn_decode: counters too small");
  c10::cuda::CUDAGuard guard(q.device());
  mb::paged_attn_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr<int>(),
                        context_lens.data_ptr<int>(), out.data_ptr(), scratch.data_ptr<float>(),
                        counters.data_ptr<int>(), (int)B, (int)H, (int)Hkv, (int)D, (int)k_cache.size(1),
                        (int)block_table.size(1), (int)k_cache.size(0), (int)splits, (float)scale,
                        status_ptr(status), cur_stream(), q.stride(0));
}

// q: [total_q, heads, head_dim] (new tokens of all sequences, packed; token stride free); caches [pages, 16, kv_heads, D].
void flash_attn_paged_prefill(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_table,
                              const Tensor& cu_q, const Tensor& kv_lens, Tensor& out, int64_t max_q_len, double scale,
                              const OptTensor& status) {
  chk(q, BF16, "q");
  chk_c(k_cache, BF16, "k_cache");
  chk_c(v_cache, BF16, "v_cache");
  chk_c(block_table, I32, "block_table");
  chk_c(cu_q, I32, "cu_q");
  chk_c(kv_lens, I32, "kv_lens");
  chk(out, BF16, "out");
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && q.stride(1) == q.size(2), "paged prefill: q must be [tokens, heads, head_dim]");
  TORCH_CHECK(out.dim() == 3 && out.stride(2) == 1 && out.stride(1) == out.size(2) && out.size(0) == q.size(0) &&
                  out.size(1) == q.size(1) && out.size(2) == q.size(2), "paged prefill: out must match q");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.size(1) == 16 && k_cache.size(3) == q.size(2) && v_cache.sizes() == k_cache.sizes(),
              "paged prefill: caches must be [pages, 16, kv_heads, head_dim]");
  const int64_t B = kv_lens.numel();
  TORCH_CHECK(cu_q.numel() == B + 1 && block_table.dim() == 2 && block_table.size(0) >= B, "paged prefill: batch metadata");
  c10::cuda::CUDAGuard guard(q.device());
  mb::flash_attn_paged_prefill(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), (int)k_cache.size(0),
                               block_table.data_ptr<int>(), (int)block_table.size(1), cu_q.data_ptr<int>(),
                               kv_lens.data_ptr<int>(), out.data_ptr(), out.stride(0), (int)B, (int)q.size(0),
                               (int)max_q_len, (int)q.size(1), (int)k_cache.size(2), (int)q.size(2), (float)scale,
                               status_ptr(status), cur_stream());
}

void kv_append_int8(const Tensor& k, const Tensor& v, Tensor& k_cache, Tensor& v_cache, Tensor& k_scale, Tensor& v_scale,
                    const Tensor& block_table, const Tensor& positions, const Tensor& seq_ids) {
  chk(k, BF16, "k");
  chk(v, BF16, "v");
  chk_c(k_cache, torch::kInt8, "k_cache");
  chk_c(v_cache, torch::kInt8, "v_cache");
  chk_c(k_scale, F32, "k_scale");
  chk_c(v_scale, F32, "v_scale");
  chk_c(block_table, I32, "block_table");
  chk_c(positions, I32, "positions");
  chk_c(seq_ids, I32, "seq_ids");
  TORCH_CHECK(k.dim() == 3 && k.stride(2) == 1 && k.stride(1) == k.size(2) && k.stride(0) == v.stride(0),
              "kv_append_int8: k/v must be [tokens, kv_heads, head_dim] with a shared token stride");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.size(2) == k.size(1) && k_cache.size(3) == k.size(2),
              "kv_append_int8: cache must be [pages, page_size, kv_heads, head_dim]");
  const int64_t rows = k_cache.size(0) * k_cache.size(1) * k_cache.size(2);
  TORCH_CHECK(k_scale.numel() == rows && v_scale.numel() == rows, "kv_append_int8: one scale per (token, kv head)");
  c10::cuda::CUDAGuard guard(k.device());
  mb::kv_append_int8(k.data_ptr(), v.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), k_scale.data_ptr<float>(),
                     v_scale.data_ptr<float>(), block_table.data_ptr<int>(), positions.data_ptr<int>(),
                     seq_ids.data_ptr<int>(), (int)k.size(0), (int)k.size(1), (int)k.size(2), (int)k_cache.size(1),
                     (int)block_table.size(1), k.stride(0), cur_stream());
}

void paged_attn_decode_int8(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& k_scale,
                            const Tensor& v_scale, const Tensor& block_table, const Tensor& context_lens, Tensor& out,
                            Tensor& scratch, Tensor& counters, int64_t splits, double scale,
                            const OptTensor& status) {
  chk(q, BF16, "q");
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && q.stride(1) == q.size(2),
              "paged_attn_decode_int8: q must be [batch, heads, head_dim] with contiguous heads");
  chk_c(k_cache, torch::kInt8, "k_cache");
  chk_c(v_cache, torch::kInt8, "v_cache");
  chk_c(k_scale, F32, "k_scale");
  chk_c(v_scale, F32, "v_scale");
  chk_c(block_table, I32, "block_table");
  chk_c(context_lens, I32, "context_lens");
  chk_c(out, BF16, "out");
  chk_c(scratch, F32, "scratch");
  chk_c(counters, I32, "counters");
  const int64_t B = q.size(0), H = q.size(1), D = q.size(2), Hkv = k_cache.size(2);
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.size(3) == D, "paged_attn_decode_int8: cache head_dim mismatch");
  const int64_t rows = k_cache.size(0) * k_cache.size(1) * Hkv;
  TORCH_CHECK(k_scale.numel() == rows && v_scale.numel() == rows,
              "paged_attn_decode_int8: one scale per (token, kv head)");
  TORCH_CHECK(scratch.numel() >= B * H * splits * (D + 2), "paged_attn_decode_int8: scratch too small");
  TORCH_CHECK(counters.numel() >= B * Hkv, "paged_attn_decode_int8: counters too small");
  c10::cuda::CUDAGuard guard(q.device());
  mb::paged_attn_decode_int8(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), k_scale.data_ptr<float>(),
                             v_scale.data_ptr<float>(), block_table.data_ptr<int>(), context_lens.data_ptr<int>(),
                             out.data_ptr(), scratch.data_ptr<float>(), counters.data_ptr<int>(), (int)B, (int)H,
                             (int)Hkv, (int)D, (int)k_cache.size(1), (int)block_table.size(1), (int)k_cache.size(0),
                             (int)splits, (float)scale, status_ptr(status), cur_stream(), q.stride(0));
}

void sample_tokens(const Tensor& logits, const OptTensor& history, const OptTensor& allow_mask, double temperature,
                   int64_t top_k, double top_p, double repetition_penalty, int64_t seed, Tensor& out_tokens,
                   OptTensor out_logprob) {
  chk(logits, BF16, "logits");
  chk_c(out_tokens, I32, "out_tokens");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "sample_tokens: logits must be [rows, vocab]");
  const int* hist = nullptr;
  int hist_len = 0;
  if (history.has_value()) {
    chk_c(*history, I32, "history");
    hist = history->data_ptr<int>();
    hist_len = (int)history->size(1);
  }
  mb::SamplerArgs a{(float)temperature, (float)top_p, (float)repetition_penalty, (int)top_k,
                    (unsigned long long)seed};
  c10::cuda::CUDAGuard guard(logits.device());
  mb::sample_tokens(logits.data_ptr(), logits.stride(0), (int)logits.size(0), (int)logits.size(1), hist, hist_len,
                    allow_mask.has_value() ? allow_mask->data_ptr<unsigned char>() : nullptr, a,
                    out_tokens.data_ptr<int>(), out_logprob.has_value() ? out_logprob->data_ptr<float>() : nullptr,
                    nullptr, cur_stream());
}

void peer_add_f32(const Tensor& part, const std::vector<int64_t>& ptrs) {
  chk_c(part, F32, "part");
  c10::cuda::CUDAGuard guard(part.device());
  mb::peer_add_f32(part.data_ptr<float>(), to_peers(ptrs), (int)ptrs.size(), part.numel(), cur_stream());
}
void peer_gather_cols(const Tensor& src, const std::vector<int64_t>& ptrs, int64_t rank, int64_t world) {
  chk_c(src, BF16, "src");
  TORCH_CHECK(src.dim() == 2 && (int64_t)ptrs.size() == world, "peer_gather_cols: src must be [rows, cols]");
  c10::cuda::CUDAGuard guard(src.device());
  mb::peer_gather_cols(src.data_ptr(), to_peers(ptrs), (int)world, (int)rank, src.size(0), (int)src.size(1),
                       cur_stream());
}

void moe_topk(const Tensor& probs, int64_t k, Tensor& topk_idx, Tensor& slot, Tensor& counts) {
  chk_c(probs, F32, "probs");
  chk_c(topk_idx, I32, "topk_idx");
  chk_c(slot, I32, "slot");
  chk_c(counts, I32, "counts");
  c10::cuda::CUDAGuard guard(probs.device());
  mb::moe_topk(probs.data_ptr<float>(), (int)probs.size(0), (int)probs.size(1), (int)k, topk_idx.data_ptr<int>(),
               slot.data_ptr<int>(), counts.data_ptr<int>(), cur_stream());
}
const int* limit_ptr(const OptTensor& send_limit, const Tensor& send_off) {
  if (!send_limit.has_value()) return nullptr;
  chk_c(*send_limit, I32, "send_limit");
  TORCH_CHECK(send_limit->numel() >= send_off.numel(), "send_limit must have an entry per expert");
  return send_limit->data_ptr<int>();
}
void moe_dispatch(const Tensor& x, const Tensor& topk_idx, const Tensor& slot, const Tensor& send_off,
                  const OptTensor& row_scale, const std::vector<int64_t>& recv_ptrs, int64_t experts_per_rank,
                  int64_t rank, int64_t cap, const OptTensor& send_limit) {
  chk_c(x, BF16, "x");
  chk_c(topk_idx, I32, "topk_idx");
  chk_c(slot, I32, "slot");
  chk_c(send_off, I32, "send_off");
  c10::cuda::CUDAGuard guard(x.device());
  mb::moe_dispatch(x.data_ptr(), topk_idx.data_ptr<int>(), slot.data_ptr<int>(), send_off.data_ptr<int>(),
                   row_scale.has_value() ? row_scale->data_ptr<float>() : nullptr, to_peers(recv_ptrs), (int)x.size(0),
                   (int)topk_idx.size(1), (int)x.size(1), (int)experts_per_rank, (int)rank, cap, cur_stream(),
                   limit_ptr(send_limit, send_off));
}
void moe_combine(const std::vector<int64_t>& ybuf_ptrs, const Tensor& topk_idx, const Tensor& slot,
                 const Tensor& send_off, const OptTensor& w, const OptTensor& dout, OptTensor out, OptTensor dw,
                 int64_t dim, int64_t experts_per_rank, int64_t rank, int64_t cap, const OptTensor& send_limit) {
  chk_c(topk_idx, I32, "topk_idx");
  chk_c(slot, I32, "slot");
  chk_c(send_off, I32, "send_off");
  c10::cuda::CUDAGuard guard(topk_idx.device());
  mb::moe_combine(to_peers(ybuf_ptrs), topk_idx.data_ptr<int>(), slot.data_ptr<int>(), send_off.data_ptr<int>(),
                  w.has_value() ? w->data_ptr<float>() : nullptr, cptr(dout), mptr(out),
                  dw.has_value() ? dw->data_ptr<float>() : nullptr, (int)topk_idx.size(0), (int)topk_idx.size(1),
                  (int)dim, (int)experts_per_rank, (int)rank, cap, cur_stream(), limit_ptr(send_limit, send_off));
}

// logits: bf16 [T, ld >= E]. Fills probs [T,E] f32, topk_idx / slot [T,k] i32, w [T,k] f32; adds into counts [E] i32, psum [E] f32.
void moe_route(const Tensor& logits, int64_t E, Tensor& probs, Tensor& topk_idx, Tensor& slot, Tensor& w, Tensor& counts,
               Tensor& psum) {
  chk(logits, BF16, "logits");
  chk_c(probs, F32, "probs");
  chk_c(topk_idx, I32, "topk_idx");
  chk_c(slot, I32, "slot");
  chk_c(w, F32, "w");
  chk_c(counts, I32, "counts");
  chk_c(psum, F32, "psum");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.size(1) >= E, "moe_route: logits [T, >= E]");
  const int64_t T = logits.size(0), k = topk_idx.size(1);
  TORCH_CHECK(probs.numel() == T * E && topk_idx.size(0) == T && slot.numel() == T * k && w.numel() == T * k &&
                  counts.numel() >= E && psum.numel() >= E, "moe_route: output shapes");
  c10::cuda::CUDAGuard guard(logits.device());
  mb::moe_route(logits.data_ptr(), (int)logits.stride(0), (int)T, (int)E, (int)k, probs.data_ptr<float>(),
                topk_idx.data_ptr<int>(), slot.data_ptr<int>(), w.data_ptr<float>(), counts.data_ptr<int>(),
                psum.data_ptr<float>(), cur_stream());
}
void moe_route_bwd(const Tensor& probs, const Tensor& topk_idx, const Tensor& dw, const OptTensor& coef, Tensor& dlogits) {
  chk_c(probs, F32, "probs");
  chk_c(topk_idx, I32, "topk_idx");
  chk_c(dw, F32, "dw");
  chk_c(dlogits, BF16, "dlogits");
  const int64_t T = probs.size(0), E = probs.size(1), k = topk_idx.size(1);
  TORCH_CHECK(dw.numel() == T * k && dlogits.size(0) == T && dlogits.size(1) >= E, "moe_route_bwd: shapes");
  if (coef.has_value()) chk_c(*coef, F32, "coef");
  c10::cuda::CUDAGuard guard(probs.device());
  mb::moe_route_bwd(probs.data_ptr<float>(), topk_idx.data_ptr<int>(), dw.data_ptr<float>(),
                    coef.has_value() ? coef->data_ptr<float>() : nullptr, (int)T, (int)E, (int)k, dlogits.data_ptr(),
                    (int)dlogits.size(1), cur_stream());
}
void moe_publish_counts(const Tensor& counts, const std::vector<int64_t>& table_ptrs, int64_t E, int64_t rank) {
  chk_c(counts, I32, "counts");
  c10::cuda::CUDAGuard guard(counts.device());
  mb::moe_publish_counts(counts.data_ptr<int>(), to_peers(table_ptrs), (int)table_ptrs.size(), (int)E, (int)rank, cur_stream());
}
void moe_offsets(const Tensor& all_counts, int64_t world, int64_t E, int64_t rank, int64_t cap, Tensor& seg_start,
                 Tensor& seg_rows, Tensor& send_base, const OptTensor& status, OptTensor send_limit) {
  chk_c(all_counts, I32, "all_counts");
  chk_c(seg_start, I32, "seg_start");
  chk_c(seg_rows, I32, "seg_rows");
  chk_c(send_base, I32, "send_base");
  TORCH_CHECK(all_counts.numel() >= world * E && send_base.numel() >= E && seg_start.numel() >= E / world &&
                  seg_rows.numel() >= E / world, "moe_offsets: shapes");
  c10::cuda::CUDAGuard guard(all_counts.device());
  mb::moe_offsets(all_counts.data_ptr<int>(), (int)world, (int)E, (int)rank, (int)cap, seg_start.data_ptr<int>(),
                  seg_rows.data_ptr<int>(), send_base.data_ptr<int>(), status_ptr(status), cur_stream(),
                  send_limit.has_value() ? send_limit->data_ptr<int>() : nullptr);
}
void moe_zero_pad(const Tensor& seg_start, const Tensor& seg_rows, int64_t n_seg, OptTensor a, OptTensor b) {
  chk_c(seg_start, I32, "seg_start");
  chk_c(seg_rows, I32, "seg_rows");
  TORCH_CHECK(a.has_value(), "moe_zero_pad: need a buffer");
  chk_c(*a, BF16, "a");
  if (b.has_value()) {
    chk_c(*b, BF16, "b");
    TORCH_CHECK(b->sizes() == a->sizes(), "moe_zero_pad: buffers must have one shape");
  }
  TORCH_CHECK(a->dim() == 2, "moe_zero_pad: [rows, dim] buffers");
  c10::cuda::CUDAGuard guard(a->device());
  mb::moe_zero_pad(seg_start.data_ptr<int>(), seg_rows.data_ptr<int>(), (int)n_seg, (int)a->size(1), mptr(a), mptr(b),
                   (int)a->size(0), cur_stream());
}

// Grouped GEMM over row segments: out[rows of e] = a[rows of e] @ weights[e]^T (weights[e]: [N, K], or [K, N] with b_mn).
void gemm_grouped_rows(const Tensor& a, const std::vector<Tensor>& weights, bool b_mn, OptTensor out, const Tensor& seg_start,
                       const Tensor& seg_rows, int64_t fuse, const OptTensor& aux, OptTensor out2, const OptTensor& status) {
  chk(a, BF16, "a");
  chk_c(seg_start, I32, "seg_start");
  chk_c(seg_rows, I32, "seg_rows");
  TORCH_CHECK(a.dim() == 2 && a.stride(1) == 1 && !weights.empty(), "gemm_grouped_rows: a [rows, K] and weights");
  const int64_t K = a.size(1);
  const int64_t N = b_mn ? weights[0].size(1) : weights[0].size(0);
  std::vector<const void*> bp;
  for (const auto& wt : weights) {
    chk(wt, BF16, "weight");
    TORCH_CHECK(wt.dim() == 2 && wt.stride(1) == 1 && wt.stride(0) == weights[0].stride(0) && wt.sizes() == weights[0].sizes(),
                "gemm_grouped_rows: weights must share one shape");
    TORCH_CHECK((b_mn ? wt.size(0) : wt.size(1)) == K, "gemm_grouped_rows: contraction sizes differ");
    bp.push_back(wt.data_ptr());
  }
  TORCH_CHECK((int64_t)bp.size() <= seg_start.numel() && (int64_t)bp.size() <= seg_rows.numel(), "gemm_grouped_rows: segments");
  if (out.has_value()) {
    chk(*out, BF16, "out");
    TORCH_CHECK(out->dim() == 2 && out->stride(1) == 1 && out->size(0) == a.size(0), "gemm_grouped_rows: out rows");
  }
  if (aux.has_value()) chk(*aux, BF16, "aux");
  if (out2.has_value()) chk(*out2, BF16, "out2");
  c10::cuda::CUDAGuard guard(a.device());
  mb::gemm_grouped_rows(a.data_ptr(), a.stride(0), (int)a.size(0), bp.data(), weights[0].stride(0), b_mn, mptr(out),
                        out.has_value() ? out->stride(0) : (fuse == mb::FUSE_SWIGLU_FWD ? N : 0), (int)N, (int)K,
                        seg_start.data_ptr<int>(), seg_rows.data_ptr<int>(), (int)bp.size(), (int)fuse, cptr(aux),
                        aux.has_value() ? aux->stride(0) : 0, mptr(out2), out2.has_value() ? out2->stride(0) : 0,
                        status_ptr(status), cur_stream());
}
// Grouped weight gradients: grads[e] [M, N] (fp32) += a[rows of e, 0:M]^T @ b[rows of e, 0:N].
void gemm_grouped_k(const Tensor& a, const Tensor& b, const std::vector<Tensor>& grads, const Tensor& seg_start,
                    const Tensor& seg_rows, const OptTensor& status) {
  chk(a, BF16, "a");
  chk(b, BF16, "b");
  chk_c(seg_start, I32, "seg_start");
  chk_c(seg_rows, I32, "seg_rows");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && a.size(0) == b.size(0) && !grads.empty(),
              "gemm_grouped_k: a [rows, M], b [rows, N]");
  std::vector<float*> cp;
  for (const auto& g : grads) {
    chk(g, F32, "grad");
    TORCH_CHECK(g.dim() == 2 && g.stride(1) == 1 && g.size(0) == a.size(1) && g.size(1) == b.size(1) &&
                    g.stride(0) == grads[0].stride(0), "gemm_grouped_k: grads must be [M, N] with one stride");
    cp.push_back(g.data_ptr<float>());
  }
  c10::cuda::CUDAGuard guard(a.device());
  mb::gemm_grouped_k(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), cp.data(), grads[0].stride(0), (int)a.size(1),
                     (int)b.size(1), (int)a.size(0), seg_start.data_ptr<int>(), seg_rows.data_ptr<int>(), (int)cp.size(),
                     status_ptr(status), cur_stream());
}

void tl_gemm(const Tensor& packed, const Tensor& x, Tensor& y, int64_t group) {
  chk_c(packed, U8, "packed");
  chk_c(x, F32, "x");
  chk_c(y, F32, "y");
  TORCH_CHECK(x.dim() == 2 && packed.dim() == 2 && packed.size(1) * 4 == x.size(1) && y.size(0) == x.size(0) &&
                  y.size(1) == packed.size(0), "tl_gemm: x [M, K], packed [N, K/4], y [M, N]");
  c10::cuda::CUDAGuard guard(x.device());
  mb::tl_gemm(packed.data_ptr<uint8_t>(), x.data_ptr<float>(), y.data_ptr<float>(), (int)x.size(0), (int)packed.size(0),
              (int)x.size(1), (int)group, cur_stream());
}

int64_t launch_count() { return mb::launch_count(); }

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "mythos_b200 sm_100a kernels";
  m.def("gemm", &gemm);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("dy"), py::arg("x"), py::arg("gamma"), py::arg("rstd"), py::arg("dx"),
        py::arg("dgamma_partial"), py::arg("dgamma"), py::arg("accumulate"), py::arg("dres") = py::none());
  m.def("gemm_swiglu_fwd", &gemm_swiglu_fwd);
  m.def("gemm_swiglu_bwd", &gemm_swiglu_bwd);
  m.def("gemm_rope", &gemm_rope);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("rope", &rope);
  m.def("swiglu_fused_fwd", &swiglu_fused_fwd);
  m.def("swiglu_fused_bwd", &swiglu_fused_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("relu2_fwd", &relu2_fwd);
  m.def("relu2_bwd", &relu2_bwd);
  m.def("act_fwd", &act_fwd);
  m.def("act_bwd", &act_bwd);
  m.def("softmax_rows_bwd", &softmax_rows_bwd);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("add", &add);
  m.def("softmax_rows", &softmax_rows);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("cross_entropy_fwd_bwd", &cross_entropy_fwd_bwd);
  m.def("cross_entropy_fwd", &cross_entropy_fwd);
  m.def("cross_entropy_shard_stats", &cross_entropy_shard_stats);
  m.def("cross_entropy_shard_grad", &cross_entropy_shard_grad);
  m.def("adamw_step", &adamw_step);
  m.def("sumsq", &sumsq);
  m.def("oil_fake_quant", &oil_fake_quant);
  m.def("i2s_fake_quant", &i2s_fake_quant);
  m.def("cast_f32_to_bf16", &cast_f32_to_bf16);
  m.def("cast_bf16_to_f32", &cast_bf16_to_f32);
  m.def("oil_codebook_stats", &oil_codebook_stats);
  m.def("flash_attn_fwd", &flash_attn_fwd);
  m.def("flash_attn_bwd", &flash_attn_bwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("dout"),
        py::arg("lse"), py::arg("dq"), py::arg("dk"), py::arg("dv"), py::arg("dq_accum"), py::arg("delta"),
        py::arg("causal"), py::arg("scale"), py::arg("status") = py::none(), py::arg("rope_pos") = py::none(),
        py::arg("rope_table") = py::none());
  m.def("dequant_gemm", &dequant_gemm, py::arg("x"), py::arg("packed"), py::arg("codebooks"), py::arg("cb_map"),
        py::arg("scales"), py::arg("fmt"), py::arg("N"), py::arg("K"), py::arg("block_size"), py::arg("out"),
        py::arg("peer_ptrs"), py::arg("k_splits"), py::arg("status"), py::arg("peer_bf16_offset") = -1);
  m.def("tp_push", &tp_push);
  m.def("tp_reduce_slots", &tp_reduce_slots);
  m.def("tp_allreduce_pull", &tp_allreduce_pull);
  m.def("tp_reduce_scatter_pull", &tp_reduce_scatter_pull);
  m.def("sum_residual_rmsnorm", &sum_residual_rmsnorm);
  m.def("tp_sum_residual_rmsnorm", &tp_sum_residual_rmsnorm);
  m.def("qkv_rope_append", &qkv_rope_append, py::arg("acc"), py::arg("pos"), py::arg("seq_ids"), py::arg("block_table"),
        py::arg("q_out"), py::arg("k_cache"), py::arg("v_cache"), py::arg("theta"), py::arg("k_scale") = py::none(),
        py::arg("v_scale") = py::none());
  m.def("finalize_gate", &finalize_gate);
  m.def("gemm_reduce_scatter", &gemm_reduce_scatter);
  m.def("tp_reduce_slots_bcast", &tp_reduce_slots_bcast);
  m.def("finalize_acc", &finalize_acc);
  m.def("dequant_to_bf16", &dequant_to_bf16);
  m.def("dequant_gather_rows", &dequant_gather_rows);
  m.def("i2s_gemv", &i2s_gemv);
  m.def("kv_append", &kv_append);
  m.def("paged_attn_decode", &paged_attn_decode);
  m.def("kv_append_int8", &kv_append_int8);
  m.def("paged_attn_decode_int8", &paged_attn_decode_int8, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"),
        py::arg("k_scale"), py::arg("v_scale"), py::arg("block_table"), py::arg("context_lens"), py::arg("out"),
        py::arg("scratch"), py::arg("counters"), py::arg("splits"), py::arg("scale"), py::arg("status") = py::none());
  m.def("sample_tokens", &sample_tokens);
  m.def("moe_topk", &moe_topk);
  m.def("moe_dispatch", &moe_dispatch, py::arg("x"), py::arg("topk_idx"), py::arg("slot"), py::arg("send_off"),
        py::arg("row_scale"), py::arg("recv_ptrs"), py::arg("experts_per_rank"), py::arg("rank"), py::arg("cap"),
        py::arg("send_limit") = py::none());
  m.def("moe_combine", &moe_combine, py::arg("ybuf_ptrs"), py::arg("topk_idx"), py::arg("slot"), py::arg("send_off"),
        py::arg("w"), py::arg("dout"), py::arg("out"), py::arg("dw"), py::arg("dim"), py::arg("experts_per_rank"),
        py::arg("rank"), py::arg("cap"), py::arg("send_limit") = py::none());
  m.def("peer_add_f32", &peer_add_f32);
  m.def("peer_gather_cols", &peer_gather_cols);
  m.def("symm_barrier", &symm_barrier);
  m.def("gemm_allgather_a", &gemm_allgather_a);
  m.def("gemm_allgather_b", &gemm_allgather_b);
  m.def("comm_barrier_wait_stats", &comm_barrier_wait_stats, py::arg("reset") = true);
  m.def("zero_reduce_scatter", &zero_reduce_scatter, py::arg("grad_ptrs"), py::arg("out"), py::arg("shard_off"),
        py::arg("sumsq"), py::arg("multicast_ptr") = 0, py::arg("max_blocks") = 0, py::arg("scratch") = py::none());
  m.def("tp_allreduce_multimem", &tp_allreduce_multimem);
  m.def("zero_adamw_ste_allgather", &zero_adamw_ste_allgather);
  m.def("comm_set_abort_word", [](const Tensor& status) {
    chk_c(status, I32, "status");
    c10::cuda::CUDAGuard guard(status.device());
    mb::comm_set_abort_word(status.data_ptr<int>());
  });
  m.def("flash_attn_paged_prefill", &flash_attn_paged_prefill);
  m.def("tl_gemm", &tl_gemm);
  m.def("moe_route", &moe_route);
  m.def("moe_route_bwd", &moe_route_bwd);
  m.def("moe_publish_counts", &moe_publish_counts);
  m.def("moe_offsets", &moe_offsets, py::arg("all_counts"), py::arg("world"), py::arg("E"), py::arg("rank"), py::arg("cap"),
        py::arg("seg_start"), py::arg("seg_rows"), py::arg("send_base"), py::arg("status") = py::none(),
        py::arg("send_limit") = py::none());
  m.def("moe_zero_pad", &moe_zero_pad);
  m.def("gemm_grouped_rows", &gemm_grouped_rows);
  m.def("gemm_grouped_k", &gemm_grouped_k);
  m.def("set_gemm_coalesced_epilogue", [](int64_t on) { mb::set_gemm_coalesced_epilogue((int)on); });
  m.def("set_attn_fwd_mode", [](int64_t mode) { mb::set_attn_fwd_mode((int)mode); });
  m.def("get_attn_fwd_mode", []() { return (int64_t)mb::get_attn_fwd_mode(); });
  m.def("set_gemm_mode", [](int64_t mode) { mb::set_gemm_mode((int)mode); });
  m.def("get_gemm_mode", []() { return (int64_t)mb::get_gemm_mode(); });
  m.def("launch_count", &launch_count);
}
