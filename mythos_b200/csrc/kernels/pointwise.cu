// Memory-bound pointwise kernels: rotary embedding, SwiGLU / squared-ReLU gates, generic
// activations, residual add, row softmax, embedding gather / scatter-add, fused cross-entropy.
// bf16 storage, fp32 math, 128-bit accesses.
//
// Formula parity with the reference:
//   RoPE  inv_freq_j = theta^(-2j/D), pairs (d, d+D/2)          src/transformer.cpp:108-135
//   SiLU  x/(1+e^-x); SwiGLU = silu(gate)*up                    src/transformer.cpp:373-387
//   GELU  exact erf (src/math.cpp:107-117) and tanh form (src/kernels/cuda_kernels.cu:119-126)
//   CE    mean of logsumexp - logit[target]; grad (softmax-onehot)/rows   src/autograd.cpp:1166-1215
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace mb {
namespace {

// ------------------------------------------------------------------------------ RoPE
// One thread per (token, 8-wide group of pairs) loops over a chunk of heads (blockIdx.y picks the
// chunk), so each cos/sin is computed once per chunk; few-token launches (decode) use many chunks.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos, int tokens, int heads,
                            int heads_per_chunk, int head_dim, long long token_stride, float log2_theta,
                            int inverse) {
  const int half = head_dim >> 1;
  const int groups = half >> 3;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)tokens * groups) return;
  const int t = (int)(gid / groups), g = (int)(gid % groups);
  const float p = (float)pos[t];
  float cs[8], sn[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int j = g * 8 + i;
    const float inv_freq = exp2f(-2.0f * (float)j / (float)head_dim * log2_theta);
    sincosf(p * inv_freq, &sn[i], &cs[i]);
    if (inverse) sn[i] = -sn[i];
  }
  __nv_bfloat16* base = x + (long long)t * token_stride;
  const int h_begin = blockIdx.y * heads_per_chunk;
  const int h_end = min(heads, h_begin + heads_per_chunk);
  for (int h = h_begin; h < h_end; ++h) {
    __nv_bfloat16* hp = base + (long long)h * head_dim;
    float a[8], b[8];
    unpack8(ldg8(hp, g * 8), a);
    unpack8(ldg8(hp, half + g * 8), b);
    float ra[8], rb[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ra[i] = a[i] * cs[i] - b[i] * sn[i];
      rb[i] = a[i] * sn[i] + b[i] * cs[i];
    }
    stg8(hp, g * 8, pack8(ra));
    stg8(hp, half + g * 8, pack8(rb));
  }
}

// ------------------------------------------------------------------------------ gates
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                  __nv_bfloat16* __restrict__ out, long long rows, int ffn, long long ld_in) {
  const int per_row = ffn >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c = (int)(i % per_row) * 8;
    float g[8], u[8], o[8];
    unpack8(ldg8(gate, r * ld_in + c), g);
    unpack8(ldg8(up, r * ld_in + c), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = silu_f(g[k]) * u[k];
    stg8(out, r * ffn + c, pack8(o));
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                  const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dgate,
                                  __nv_bfloat16* __restrict__ dup, long long rows, int ffn, long long ld_in) {
  const int per_row = ffn >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c = (int)(i % per_row) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(ldg8(gate, r * ld_in + c), g);
    unpack8(ldg8(up, r * ld_in + c), u);
    unpack8(ldg8(dout, r * ffn + c), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = sigmoid_f(g[k]);
      const float sl = g[k] * s;
      du[k] = d[k] * sl;
      dg[k] = d[k] * u[k] * (s + sl * (1.f - s));
    }
    stg8(dgate, r * ld_in + c, pack8(dg));
    stg8(dup, r * ld_in + c, pack8(du));
  }
}

__global__ void relu2_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float v[8];
    unpack8(ldg8(x, i * 8), v);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float r = fmaxf(v[k], 0.f);
      v[k] = r * r;
    }
    stg8(out, i * 8, pack8(v));
  }
}
__global__ void relu2_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dout,
                                 __nv_bfloat16* __restrict__ dx, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float v[8], d[8];
    unpack8(ldg8(x, i * 8), v);
    unpack8(ldg8(dout, i * 8), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = 2.f * fmaxf(v[k], 0.f) * d[k];
    stg8(dx, i * 8, pack8(v));
  }
}

__device__ __forceinline__ float act_apply(float x, int kind) {
  switch (kind) {
    case ACT_RELU: return fmaxf(x, 0.f);
    case ACT_GELU_ERF: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case ACT_GELU_TANH: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    case ACT_SILU: return silu_f(x);
    case ACT_SIGMOID: return sigmoid_f(x);
    default: return tanhf(x);
  }
}
__global__ void act_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, long long n8, int kind) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float v[8];
    unpack8(ldg8(x, i * 8), v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = act_apply(v[k], kind);
    stg8(out, i * 8, pack8(v));
  }
}
// d act(x) / dx for the same table of activations.
__device__ __forceinline__ float act_grad(float x, int kind) {
  switch (kind) {
    case ACT_RELU: return x > 0.f ? 1.f : 0.f;
    case ACT_GELU_ERF:   // Phi(x) + x phi(x)
      return 0.5f * (1.f + erff(x * 0.70710678118654752f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
    case ACT_GELU_TANH: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      const float t = tanhf(u);
      return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * 0.7978845608028654f * (1.f + 0.134145f * x * x);
    }
    case ACT_SILU: {
      const float sg = sigmoid_f(x);
      return sg * (1.f + x * (1.f - sg));
    }
    case ACT_SIGMOID: {
      const float sg = sigmoid_f(x);
      return sg * (1.f - sg);
    }
    default: {
      const float t = tanhf(x);
      return 1.f - t * t;
    }
  }
}
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dout,
                               __nv_bfloat16* __restrict__ dx, long long n8, int kind) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float v[8], d[8];
    unpack8(ldg8(x, i * 8), v);
    unpack8(ldg8(dout, i * 8), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = act_grad(v[k], kind) * d[k];
    stg8(dx, i * 8, pack8(v));
  }
}
__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ out, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float x[8], y[8];
    unpack8(ldg8(a, i * 8), x);
    unpack8(ldg8(b, i * 8), y);
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] += y[k];
    stg8(out, i * 8, pack8(x));
  }
}

// ------------------------------------------------------------------------------ softmax (generic rows)
__global__ void softmax_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int cols) {
  __shared__ float scratch[32];
  const __nv_bfloat16* xr = x + (long long)blockIdx.x * cols;
  __nv_bfloat16* yr = y + (long long)blockIdx.x * cols;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, __bfloat162float(xr[c]));
  m = block_max(m, scratch);
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s += __expf(__bfloat162float(xr[c]) - m);
  s = block_sum(s, scratch);
  const float inv = 1.f / s;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) yr[c] = __float2bfloat16(__expf(__bfloat162float(xr[c]) - m) * inv);
}

// dx = y * (dy - sum_c dy_c y_c), one CTA per row.
__global__ void softmax_bwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ dy,
                                   __nv_bfloat16* __restrict__ dx, int cols) {
  __shared__ float scratch[32];
  const long long base = (long long)blockIdx.x * cols;
  float dot = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dot += __bfloat162float(y[base + c]) * __bfloat162float(dy[base + c]);
  dot = block_sum(dot, scratch);
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    dx[base + c] = __float2bfloat16(__bfloat162float(y[base + c]) * (__bfloat162float(dy[base + c]) - dot));
}

// ------------------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int tokens, int dim, int vocab) {
  const int per_row = dim >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)tokens * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / per_row), c = (int)(i % per_row) * 8;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    stg8(out, (long long)t * dim + c, ldg8(table, (long long)id * dim + c));
  }
}
__global__ void embedding_bwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dtable, int tokens, int dim, int vocab) {
  const int per_row = dim >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)tokens * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / per_row), c = (int)(i % per_row) * 8;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    float d[8];
    unpack8(ldg8(dout, (long long)t * dim + c), d);
    float* p = dtable + (long long)id * dim + c;
    atomicAdd(reinterpret_cast<float4*>(p), make_float4(d[0], d[1], d[2], d[3]));
    atomicAdd(reinterpret_cast<float4*>(p + 4), make_float4(d[4], d[5], d[6], d[7]));
  }
}

// ------------------------------------------------------------------------------ cross-entropy
// One CTA per row. Pass 1: online max / sum-exp. Pass 2 (WRITE_GRAD): overwrite logits with
// (softmax - onehot) * grad_scale. Targets are clamped to [0, vocab-1]; target < 0 with
// ignore semantics is expressed by the caller through grad_scale.
// Block-wide max and sum of exp(x - max) over one row of bf16 logits (online, one pass).
__device__ __forceinline__ void row_max_sumexp(const __nv_bfloat16* __restrict__ row, int vocab, float* scratch,
                                               float& gm, float& gs) {
  const int nchunk = vocab >> 3;
  float m = -INFINITY, s = 0.f;
  for (int ch = threadIdx.x; ch < nchunk; ch += blockDim.x) {
    float v[8];
    unpack8(ldg8(row, ch * 8), v);
    float cm = v[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) cm = fmaxf(cm, v[k]);
    const float nm = fmaxf(m, cm);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc += __expf(v[k] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int c = nchunk * 8 + threadIdx.x; c < vocab; c += blockDim.x) {
    const float v = __bfloat162float(row[c]);
    const float nm = fmaxf(m, v);
    s = s * __expf(m - nm) + __expf(v - nm);
    m = nm;
  }
  gm = block_max(m, scratch);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  gs = block_sum(s, scratch);
}

template <bool WRITE_GRAD>
__global__ void ce_kernel(__nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                          float* __restrict__ losses, int vocab, long long ld, float grad_scale) {
  __shared__ float scratch[32];
  __nv_bfloat16* row = logits + (long long)blockIdx.x * ld;
  const int nchunk = vocab >> 3;
  float gm, gs;
  row_max_sumexp(row, vocab, scratch, gm, gs);
  int tgt = targets[blockIdx.x];
  tgt = tgt < 0 ? 0 : (tgt >= vocab ? vocab - 1 : tgt);
  const float lse = gm + logf(gs);
  if (threadIdx.x == 0) losses[blockIdx.x] = lse - __bfloat162float(row[tgt]);
  if (WRITE_GRAD) {
    __syncthreads();  // the target logit has been read before anyone overwrites it
    const float inv = 1.f / gs;
    for (int ch = threadIdx.x; ch < nchunk; ch += blockDim.x) {
      float v[8];
      unpack8(ldg8(row, ch * 8), v);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float p = __expf(v[k] - gm) * inv;
        v[k] = (p - ((ch * 8 + k) == tgt ? 1.f : 0.f)) * grad_scale;
      }
      stg8(row, ch * 8, pack8(v));
    }
    for (int c = nchunk * 8 + threadIdx.x; c < vocab; c += blockDim.x) {
      const float p = __expf(__bfloat162float(row[c]) - gm) * inv;
      row[c] = __float2bfloat16((p - (c == tgt ? 1.f : 0.f)) * grad_scale);
    }
  }
}

// Vocabulary-parallel cross-entropy: every rank holds the columns [vocab_offset, vocab_offset +
// vocab) of the logits. Step 1 (this kernel, one CTA per row) writes stats[row] = {local max, local
// sum of exp(x - local max), target logit if this shard owns the target else 0}. The ranks then
// exchange the 12-byte records, merge them (max, rescaled sums, target) into the global
// log-sum-exp, and step 2 overwrites the local logits with their gradient.
__global__ void ce_shard_stats_kernel(const __nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                                      float* __restrict__ stats, int vocab, long long ld, int vocab_offset,
                                      int vocab_total) {
  __shared__ float scratch[32];
  const __nv_bfloat16* row = logits + (long long)blockIdx.x * ld;
  float gm, gs;
  row_max_sumexp(row, vocab, scratch, gm, gs);
  if (threadIdx.x == 0) {
    int tgt = targets[blockIdx.x];
    tgt = tgt < 0 ? 0 : (tgt >= vocab_total ? vocab_total - 1 : tgt);
    const int local = tgt - vocab_offset;
    float* o = stats + (long long)blockIdx.x * 3;
    o[0] = gm;
    o[1] = gs;
    o[2] = (local >= 0 && local < vocab) ? __bfloat162float(row[local]) : 0.f;
  }
}
__global__ void ce_shard_grad_kernel(__nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                                     const float* __restrict__ lse, int vocab, long long ld, int vocab_offset,
                                     int vocab_total, float grad_scale) {
  __nv_bfloat16* row = logits + (long long)blockIdx.x * ld;
  int tgt = targets[blockIdx.x];
  tgt = tgt < 0 ? 0 : (tgt >= vocab_total ? vocab_total - 1 : tgt);
  const int local = tgt - vocab_offset;     // outside [0, vocab) when another shard owns the target
  const float l = lse[blockIdx.x];
  const int nchunk = vocab >> 3;
  for (int ch = threadIdx.x; ch < nchunk; ch += blockDim.x) {
    float v[8];
    unpack8(ldg8(row, ch * 8), v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = (__expf(v[k] - l) - ((ch * 8 + k) == local ? 1.f : 0.f)) * grad_scale;
    stg8(row, ch * 8, pack8(v));
  }
  for (int c = nchunk * 8 + threadIdx.x; c < vocab; c += blockDim.x)
    row[c] = __float2bfloat16((__expf(__bfloat162float(row[c]) - l) - (c == local ? 1.f : 0.f)) * grad_scale);
}

inline int ew_grid(long long work, int threads) {
  long long g = (work + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

void rope_apply(void* x, const int* pos, int tokens, int heads, int head_dim, long long token_stride, float theta,
                bool inverse, cudaStream_t stream) {
  MB_REQUIRE(head_dim % 16 == 0, "rope: head_dim must be a multiple of 16");
  MB_REQUIRE(token_stride % 8 == 0, "rope: token stride must be a multiple of 8 elements");
  if (tokens == 0) return;
  const long long work = (long long)tokens * (head_dim / 16);
  // enough head chunks to put about two waves of threads on the machine
  long long chunks = ((long long)sm_count() * 2048 + work - 1) / work;
  if (chunks > heads) chunks = heads;
  if (chunks < 1) chunks = 1;
  const int hpc = (int)((heads + chunks - 1) / chunks);
  const dim3 grid((unsigned)ceil_div(work, 128), (unsigned)((heads + hpc - 1) / hpc));
  rope_kernel<<<grid, 128, 0, stream>>>((__nv_bfloat16*)x, pos, tokens, heads, hpc, head_dim, token_stride,
                                        log2f(theta), inverse ? 1 : 0);
  count_launch();
  check_launch();
}

void swiglu_fwd(const void* gate, const void* up, void* out, long long n, cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0, "swiglu: element count must be a multiple of 8");
  if (n == 0) return;
  swiglu_fwd_kernel<<<ew_grid(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)up,
                                                             (__nv_bfloat16*)out, n / 8, 8, 8);
  count_launch();
  check_launch();
}
void swiglu_bwd(const void* gate, const void* up, const void* dout, void* dgate, void* dup, long long n,
                cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0, "swiglu: element count must be a multiple of 8");
  if (n == 0) return;
  swiglu_bwd_kernel<<<ew_grid(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)up,
                                                             (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgate,
                                                             (__nv_bfloat16*)dup, n / 8, 8, 8);
  count_launch();
  check_launch();
}
void swiglu_fused_fwd(const void* gate_up, void* out, long long rows, int ffn, cudaStream_t stream) {
  MB_REQUIRE(ffn % 8 == 0, "swiglu: ffn must be a multiple of 8");
  if (rows == 0) return;
  const __nv_bfloat16* g = (const __nv_bfloat16*)gate_up;
  swiglu_fwd_kernel<<<ew_grid(rows * ffn / 8, 256), 256, 0, stream>>>(g, g + ffn, (__nv_bfloat16*)out, rows, ffn,
                                                                      2LL * ffn);
  count_launch();
  check_launch();
}
void swiglu_fused_bwd(const void* gate_up, const void* dout, void* dgate_up, long long rows, int ffn,
                      cudaStream_t stream) {
  MB_REQUIRE(ffn % 8 == 0, "swiglu: ffn must be a multiple of 8");
  if (rows == 0) return;
  const __nv_bfloat16* g = (const __nv_bfloat16*)gate_up;
  __nv_bfloat16* d = (__nv_bfloat16*)dgate_up;
  swiglu_bwd_kernel<<<ew_grid(rows * ffn / 8, 256), 256, 0, stream>>>(g, g + ffn, (const __nv_bfloat16*)dout, d,
                                                                      d + ffn, rows, ffn, 2LL * ffn);
  count_launch();
  check_launch();
}
void relu2_fwd(const void* x, void* out, long long n, cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0, "relu2: element count must be a multiple of 8");
  if (n == 0) return;
  relu2_fwd_kernel<<<ew_grid(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n / 8);
  count_launch();
  check_launch();
}
void relu2_bwd(const void* x, const void* dout, void* dx, long long n, cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0, "relu2: element count must be a multiple of 8");
  if (n == 0) return;
  relu2_bwd_kernel<<<ew_grid(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dout,
                                                            (__nv_bfloat16*)dx, n / 8);
  count_launch();
  check_launch();
}
void act_fwd(const void* x, void* out, long long n, int kind, cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0, "act: element count must be a multiple of 8");
  if (n == 0) return;
  act_kernel<<<ew_grid(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n / 8, kind);
  count_launch();
  check_launch();
}
void add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0, "add: element count must be a multiple of 8");
  if (n == 0) return;
  add_kernel<<<ew_grid(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                      (__nv_bfloat16*)out, n / 8);
  count_launch();
  check_launch();
}
void act_bwd(const void* x, const void* dout, void* dx, long long n, int kind, cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0, "act: element count must be a multiple of 8");
  if (n == 0) return;
  act_bwd_kernel<<<ew_grid(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dout,
                                                          (__nv_bfloat16*)dx, n / 8, kind);
  count_launch();
  check_launch();
}
void softmax_rows_bwd(const void* y, const void* dy, void* dx, int rows, int cols, cudaStream_t stream) {
  if (rows == 0) return;
  softmax_bwd_kernel<<<rows, 256, 0, stream>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, cols);
  count_launch();
  check_launch();
}
void softmax_rows(const void* x, void* y, int rows, int cols, cudaStream_t stream) {
  if (rows == 0) return;
  softmax_kernel<<<rows, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, cols);
  count_launch();
  check_launch();
}

void embedding_fwd(const int* ids, const void* table, void* out, int tokens, int dim, int vocab, cudaStream_t stream) {
  MB_REQUIRE(dim % 8 == 0, "embedding: dim must be a multiple of 8");
  if (tokens == 0) return;
  embedding_fwd_kernel<<<ew_grid((long long)tokens * dim / 8, 256), 256, 0, stream>>>(
      ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, tokens, dim, vocab);
  count_launch();
  check_launch();
}
void embedding_bwd(const int* ids, const void* dout, float* dtable, int tokens, int dim, int vocab, cudaStream_t stream) {
  MB_REQUIRE(dim % 8 == 0, "embedding: dim must be a multiple of 8");
  if (tokens == 0) return;
  embedding_bwd_kernel<<<ew_grid((long long)tokens * dim / 8, 256), 256, 0, stream>>>(
      ids, (const __nv_bfloat16*)dout, dtable, tokens, dim, vocab);
  count_launch();
  check_launch();
}

void cross_entropy_fwd_bwd(void* logits, const int* targets, float* losses, int rows, int vocab, long long ld,
                           float grad_scale, cudaStream_t stream) {
  MB_REQUIRE(ld % 8 == 0, "cross_entropy: row stride must be a multiple of 8 elements");
  if (rows == 0) return;
  ce_kernel<true><<<rows, 512, 0, stream>>>((__nv_bfloat16*)logits, targets, losses, vocab, ld, grad_scale);
  count_launch();
  check_launch();
}
void cross_entropy_fwd(const void* logits, const int* targets, float* losses, int rows, int vocab, long long ld,
                       cudaStream_t stream) {
  MB_REQUIRE(ld % 8 == 0, "cross_entropy: row stride must be a multiple of 8 elements");
  if (rows == 0) return;
  ce_kernel<false><<<rows, 512, 0, stream>>>((__nv_bfloat16*)const_cast<void*>(logits), targets, losses, vocab, ld, 0.f);
  count_launch();
  check_launch();
}

void cross_entropy_shard_stats(const void* logits, const int* targets, float* stats, int rows, int vocab, long long ld,
                               int vocab_offset, int vocab_total, cudaStream_t stream) {
  MB_REQUIRE(ld % 8 == 0, "cross_entropy_shard_stats: row stride must be a multiple of 8 elements");
  if (rows == 0) return;
  ce_shard_stats_kernel<<<rows, 512, 0, stream>>>((const __nv_bfloat16*)logits, targets, stats, vocab, ld, vocab_offset,
                                                  vocab_total);
  count_launch();
  check_launch();
}
void cross_entropy_shard_grad(void* logits, const int* targets, const float* lse, int rows, int vocab, long long ld,
                              int vocab_offset, int vocab_total, float grad_scale, cudaStream_t stream) {
  MB_REQUIRE(ld % 8 == 0, "cross_entropy_shard_grad: row stride must be a multiple of 8 elements");
  if (rows == 0) return;
  ce_shard_grad_kernel<<<rows, 512, 0, stream>>>((__nv_bfloat16*)logits, targets, lse, vocab, ld, vocab_offset,
                                                 vocab_total, grad_scale);
  count_launch();
  check_launch();
}

long long launch_count() { return launch_counter().load(); }

}  // namespace mb
