/* C ABI of the sm_100a kernel library (libmythos_kernels.so). Pointers are device pointers;
 * bf16 tensors are passed as void*. Return value 0 = launched, otherwise see mythos_last_error(). */
#pragma once
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif
const char* mythos_last_error(void);
/* C[M,N] (+)= alpha * op(A) * op(B)^T; epilogue: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate, 3 fp32 atomic. */
int mythos_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* C,
                     long long ldc, int M, int N, int K, int epilogue, float alpha, int* status, cudaStream_t stream);
int mythos_rmsnorm_fwd(const void* x, const void* residual, const void* gamma, void* y, void* resid_out, float* rstd,
                       int rows, int dim, float eps, cudaStream_t stream);
int mythos_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, int rows, int dim, float eps,
                         cudaStream_t stream);
int mythos_rope(void* x, const int* pos, int tokens, int heads, int head_dim, long long token_stride, float theta,
                int inverse, cudaStream_t stream);
int mythos_swiglu(const void* gate_up, void* out, long long rows, int ffn, cudaStream_t stream);
int mythos_activation(const void* x, void* out, long long n, int kind, cudaStream_t stream);
int mythos_softmax_rows(const void* x, void* y, int rows, int cols, cudaStream_t stream);
int mythos_embedding(const int* ids, const void* table, void* out, int tokens, int dim, int vocab, cudaStream_t stream);
int mythos_cross_entropy(void* logits, const int* targets, float* losses, int rows, int vocab, long long ld,
                         float grad_scale, cudaStream_t stream);
int mythos_adamw(float* p, float* m, float* v, const float* g, void* p_bf16, long long n, float lr, float beta1,
                 float beta2, float eps, float weight_decay, int step, float grad_scale, const float* clip_coef,
                 cudaStream_t stream);
int mythos_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq,
                          int heads, int kv_heads, int head_dim, int causal, float scale, int* status,
                          cudaStream_t stream);
int mythos_oil_fake_quant(const float* w, const float* codebooks, const int* cb_map, int cb_size, int block_size,
                          long long n, void* w_bf16, unsigned char* idx, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
