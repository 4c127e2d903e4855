// Paged KV cache kernels for decoding.
//
//   kv_append          scatter new K/V vectors into 16-token (or any size) pages through a block table
//   paged_attn_decode  one query token per sequence against its paged context: split-KV flash
//                      decoding, all query heads of a GQA group share each K/V load, the partial
//                      results of the splits are merged by the last CTA to finish (no waiting)
//   i2s_gemv           single-token GEMV over packed I2_S trits
//
// Reference counterparts: PagedAttention::forward (src/inference_opt.cpp:58-107, no causal mask,
// no partial last block), flash_decoding (:594-664), KVCache::append (src/kv_cache.cpp:78-137),
// i2s_gemv (src/kernel_i2s.cpp:32-40). Partial last pages and per-sequence context lengths are
// handled here.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace mb {
namespace {

__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                 __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                 const int* __restrict__ block_table, const int* __restrict__ positions,
                                 const int* __restrict__ seq_ids, int tokens, int kv_heads, int head_dim,
                                 int page_size, int max_pages, long long kv_tok_stride) {
  const int row = kv_heads * head_dim;
  const int per_tok = row >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)tokens * per_tok;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / per_tok), c = (int)(i % per_tok) * 8;
    const int pos = positions[t], seq = seq_ids[t];
    const int page = block_table[(long long)seq * max_pages + pos / page_size];
    if (page < 0) continue;
    const long long dst = ((long long)page * page_size + pos % page_size) * row + c;
    stg8(k_cache, dst, ldg8(k, (long long)t * kv_tok_stride + c));
    stg8(v_cache, dst, ldg8(v, (long long)t * kv_tok_stride + c));
  }
}

// grid (batch, kv_heads, splits); block 128 threads. G = query heads per kv head, D = head_dim.
template <int G, int D>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                    const int* __restrict__ context_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ scratch,
                    int* __restrict__ counters, int heads, int kv_heads, int page_size, int max_pages, int splits,
                    float scale_log2) {
  constexpr int LPT = D / 8;        // lanes per token (each lane holds 8 elements)
  constexpr int TPW = 32 / LPT;     // tokens per warp iteration
  constexpr int NSTATE = 4 * TPW;   // online-softmax states per CTA
  __shared__ float s_m[NSTATE][G], s_l[NSTATE][G];
  __shared__ float s_acc[NSTATE][G][D];
  __shared__ int s_last;
  const int b = blockIdx.x, hkv = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPT, li = lane % LPT;  // token slot inside the warp, lane inside the token
  const int ctx = context_lens[b];
  const int per = (ctx + splits - 1) / splits;
  const int t0 = split * per, t1 = min(ctx, t0 + per);
  const int row = kv_heads * D;

  float qv[G][8], acc[G][8], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    unpack8(ldg8(q, ((long long)b * heads + hkv * G + g) * D + li * 8), qv[g]);
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }
  const int* bt = block_table + (long long)b * max_pages;
  // Every lane of a warp runs the same number of iterations (the shuffles below need the full
  // warp); a token slot past the end of the range contributes nothing.
  for (int tb = t0 + warp * TPW; tb < t1; tb += 4 * TPW) {
    const int t = tb + sub;
    const bool valid = t < t1;
    float kf[8], vf[8];
    if (valid) {
      const int page = bt[t / page_size];
      const long long off = ((long long)page * page_size + t % page_size) * row + (long long)hkv * D + li * 8;
      unpack8(ldg8(k_cache, off), kf);
      unpack8(ldg8(v_cache, off), vf);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) kf[i] = vf[i] = 0.f;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s += qv[g][i] * kf[i];
#pragma unroll
      for (int o = LPT / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (valid) {
        s *= scale_log2;
        const float mn = fmaxf(m[g], s);
        const float a = exp2f(m[g] - mn), p = exp2f(s - mn);
        l[g] = l[g] * a + p;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * a + p * vf[i];
        m[g] = mn;
      }
    }
  }
  // publish the per-slot states
  const int st = warp * TPW + sub;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (li == 0) {
      s_m[st][g] = m[g];
      s_l[st][g] = l[g];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s_acc[st][g][li * 8 + i] = acc[g][i];
  }
  __syncthreads();
  // merge the CTA's states: thread d handles column d of every head of the group
  const int stride = D + 2;
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float M = -INFINITY;
    for (int s = 0; s < NSTATE; ++s) M = fmaxf(M, s_m[s][g]);
    float L = 0.f, A = 0.f;
    for (int s = 0; s < NSTATE; ++s) {
      const float w = (s_m[s][g] == -INFINITY) ? 0.f : exp2f(s_m[s][g] - M);
      L += w * s_l[s][g];
      A += w * s_acc[s][g][d];
    }
    float* part = scratch + (((long long)b * heads + hkv * G + g) * splits + split) * stride;
    part[d] = A;
    if (d == 0) {
      part[D] = M;
      part[D + 1] = L;
    }
  }
  // the last CTA of this (sequence, kv head) merges the splits
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&counters[b * kv_heads + hkv], 1);
    s_last = (prev == splits - 1) ? 1 : 0;
    if (s_last) counters[b * kv_heads + hkv] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    const float* base = scratch + ((long long)b * heads + hkv * G + g) * splits * stride;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, base[s * stride + D]);
    float L = 0.f, A = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = base[s * stride + D];
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
      L += w * base[s * stride + D + 1];
      A += w * base[s * stride + d];
    }
    out[((long long)b * heads + hkv * G + g) * D + d] = __float2bfloat16(L > 0.f ? A / L : 0.f);
  }
}

// One warp per output row; x staged in shared memory as fp32.
__global__ void i2s_gemv_kernel(const __nv_bfloat16* __restrict__ x, DequantWeights w, __nv_bfloat16* __restrict__ y) {
  extern __shared__ float xs[];
  for (int k = threadIdx.x; k < w.K; k += blockDim.x) xs[k] = __bfloat162float(x[k]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const int chunks = w.K / 64;  // 16 bytes = 64 trits per chunk
  for (long long n = (long long)blockIdx.x * wpb + warp; n < w.N; n += (long long)gridDim.x * wpb) {
    float total = 0.f;
    for (int c = lane; c < chunks; c += 32) {
      const long long elem = n * w.K + c * 64;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(w.packed + elem / 4));
      const uint32_t words[4] = {v.x, v.y, v.z, v.w};
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int p = 0; p < 16; ++p) {
          const int code = (words[j] >> (2 * p)) & 3;
          const float xv = xs[c * 64 + j * 16 + p];
          s += (code == 2) ? xv : ((code == 0) ? -xv : 0.f);
        }
      }
      total += s * w.scales[elem / w.block_size];
    }
    total = warp_sum(total);
    if (lane == 0) y[n] = __float2bfloat16(total);
  }
}

}  // namespace

void kv_append(const void* k, const void* v, void* k_cache, void* v_cache, const int* block_table,
               const int* positions, const int* seq_ids, int tokens, int kv_heads, int head_dim, int page_size,
               int max_pages, long long kv_tok_stride, cudaStream_t stream) {
  MB_REQUIRE(head_dim % 8 == 0 && kv_tok_stride % 8 == 0, "kv_append: head_dim and stride must be multiples of 8");
  if (tokens == 0) return;
  const long long work = (long long)tokens * kv_heads * head_dim / 8;
  long long g = (work + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  kv_append_kernel<<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                               (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, block_table, positions,
                                               seq_ids, tokens, kv_heads, head_dim, page_size, max_pages, kv_tok_stride);
  count_launch();
  check_launch();
}

void paged_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                       const int* context_lens, void* out, float* scratch, int* counters, int batch, int heads,
                       int kv_heads, int head_dim, int page_size, int max_pages, int splits, float scale,
                       cudaStream_t stream) {
  MB_REQUIRE(heads % kv_heads == 0, "paged_attn_decode: heads must be a multiple of kv_heads");
  MB_REQUIRE(splits >= 1, "paged_attn_decode: need at least one split");
  if (batch == 0) return;
  const int G = heads / kv_heads;
  const dim3 grid(batch, kv_heads, splits);
  const float sl2 = scale * 1.4426950408889634f;
#define MB_PD(GG, DD)                                                                                         \
  paged_decode_kernel<GG, DD><<<grid, 128, 0, stream>>>(                                                      \
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table,     \
      context_lens, (__nv_bfloat16*)out, scratch, counters, heads, kv_heads, page_size, max_pages, splits, sl2)
  if (head_dim == 128) {
    if (G == 1) MB_PD(1, 128);
    else if (G == 2) MB_PD(2, 128);
    else if (G == 4) MB_PD(4, 128);
    else MB_REQUIRE(false, "paged_attn_decode: GQA group must be 1, 2 or 4");
  } else if (head_dim == 64) {
    if (G == 1) MB_PD(1, 64);
    else if (G == 2) MB_PD(2, 64);
    else if (G == 4) MB_PD(4, 64);
    else MB_REQUIRE(false, "paged_attn_decode: GQA group must be 1, 2 or 4");
  } else {
    MB_REQUIRE(false, "paged_attn_decode: head_dim must be 64 or 128");
  }
#undef MB_PD
  count_launch();
  check_launch();
}

void i2s_gemv(const void* x, const DequantWeights& w, void* y, cudaStream_t stream) {
  MB_REQUIRE(w.fmt == QFMT_I2S, "i2s_gemv: weights must be I2_S");
  MB_REQUIRE(w.K % 64 == 0 && w.block_size % 64 == 0, "i2s_gemv: K and block size must be multiples of 64");
  MB_REQUIRE((size_t)w.K * 4 <= 200 * 1024, "i2s_gemv: K too large for the shared-memory activation copy");
  long long g = ((long long)w.N + 7) / 8;
  const long long cap = (long long)sm_count() * 4;
  if (g > cap) g = cap;
  static bool configured = false;
  if (!configured) {
    MB_CUDA_CHECK(cudaFuncSetAttribute(i2s_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured = true;
  }
  i2s_gemv_kernel<<<(int)g, 256, (size_t)w.K * 4, stream>>>((const __nv_bfloat16*)x, w, (__nv_bfloat16*)y);
  count_launch();
  check_launch();
}

}  // namespace mb
