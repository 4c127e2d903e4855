// Plain C ABI over the raw-pointer kernel launchers (kernels/api.h), for callers that do not link
// torch: every function takes device pointers and a CUDA stream, returns 0 on success and a
// non-zero code on failure; mythos_last_error() returns the message of the calling thread's last
// failure. The reference exports its CUDA kernels the same way (27 extern "C" launchers,
// src/kernels/cuda_kernels.cu:423-707); these are the sm_100a counterparts.
#include <exception>
#include <string>

#include "c_abi.h"
#include "kernels/api.h"

namespace {
thread_local std::string g_err;

template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  } catch (...) {
    g_err = "unknown error";
    return 2;
  }
}
}  // namespace

extern "C" {

const char* mythos_last_error(void) { return g_err.c_str(); }

int mythos_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* C,
                     long long ldc, int M, int N, int K, int epilogue, float alpha, int* status, cudaStream_t stream) {
  return guarded([&] {
    mb::gemm_bf16(A, lda, a_mn != 0, B, ldb, b_mn != 0, C, ldc, M, N, K, epilogue, alpha, status, stream);
  });
}

int mythos_rmsnorm_fwd(const void* x, const void* residual, const void* gamma, void* y, void* resid_out, float* rstd,
                       int rows, int dim, float eps, cudaStream_t stream) {
  return guarded([&] { mb::rmsnorm_fwd(x, residual, gamma, y, resid_out, rstd, rows, dim, eps, stream); });
}

int mythos_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, int rows, int dim, float eps,
                         cudaStream_t stream) {
  return guarded([&] { mb::layernorm_fwd(x, gamma, beta, y, rows, dim, eps, stream); });
}

int mythos_rope(void* x, const int* pos, int tokens, int heads, int head_dim, long long token_stride, float theta,
                int inverse, cudaStream_t stream) {
  return guarded([&] { mb::rope_apply(x, pos, tokens, heads, head_dim, token_stride, theta, inverse != 0, stream); });
}

int mythos_swiglu(const void* gate_up, void* out, long long rows, int ffn, cudaStream_t stream) {
  return guarded([&] { mb::swiglu_fused_fwd(gate_up, out, rows, ffn, stream); });
}

int mythos_activation(const void* x, void* out, long long n, int kind, cudaStream_t stream) {
  return guarded([&] { mb::act_fwd(x, out, n, kind, stream); });
}

int mythos_softmax_rows(const void* x, void* y, int rows, int cols, cudaStream_t stream) {
  return guarded([&] { mb::softmax_rows(x, y, rows, cols, stream); });
}

int mythos_embedding(const int* ids, const void* table, void* out, int tokens, int dim, int vocab, cudaStream_t stream) {
  return guarded([&] { mb::embedding_fwd(ids, table, out, tokens, dim, vocab, stream); });
}

int mythos_cross_entropy(void* logits, const int* targets, float* losses, int rows, int vocab, long long ld,
                         float grad_scale, cudaStream_t stream) {
  return guarded([&] { mb::cross_entropy_fwd_bwd(logits, targets, losses, rows, vocab, ld, grad_scale, stream); });
}

int mythos_adamw(float* p, float* m, float* v, const float* g, void* p_bf16, long long n, float lr, float beta1,
                 float beta2, float eps, float weight_decay, int step, float grad_scale, const float* clip_coef,
                 cudaStream_t stream) {
  return guarded([&] {
    mb::AdamWArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
                    grad_scale};
    mb::adamw_step(p, m, v, g, p_bf16, n, a, clip_coef, stream);
  });
}

int mythos_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq,
                          int heads, int kv_heads, int head_dim, int causal, float scale, int* status,
                          cudaStream_t stream) {
  return guarded([&] {
    mb::flash_attn_fwd(q, k, v, o, lse, batch, seq, heads, kv_heads, head_dim, causal != 0, scale, status, stream);
  });
}

int mythos_oil_fake_quant(const float* w, const float* codebooks, const int* cb_map, int cb_size, int block_size,
                          long long n, void* w_bf16, unsigned char* idx, cudaStream_t stream) {
  return guarded([&] { mb::oil_fake_quant(w, codebooks, cb_map, cb_size, block_size, n, w_bf16, idx, stream); });
}

}  // extern "C"
