// Paged KV cache kernels for decoding.
//
//   kv_append          scatter new K/V vectors into 16-token (or any size) pages through a block table
//   paged_attn_decode  one query token per sequence against its paged context: split-KV flash
//                      decoding, all query heads of a GQA group share each K/V load, the partial
//                      results of the splits are merged by the last CTA to finish (no waiting).
//                      16-token pages take the tensor-core path: each warp streams whole pages
//                      through its own TMA ring (the kernel is bound by the KV bytes in flight)
//                      and does QK^T and PV with warp-level MMAs (the query group is 1-8 rows, so
//                      the arithmetic is far below the memory time either way); other page sizes
//                      use the scalar kernel.
//   i2s_gemv           single-token GEMV over packed I2_S trits
//
// Reference counterparts: PagedAttention::forward (src/inference_opt.cpp:58-107, no causal mask,
// no partial last block), flash_decoding (:594-664), KVCache::append (src/kv_cache.cpp:78-137),
// i2s_gemv (src/kernel_i2s.cpp:32-40). Partial last pages and per-sequence context lengths are
// handled here.
#include <cuda_fp16.h>

#include "api.h"
#include "common.cuh"
#include "host_util.h"
#include "tc.cuh"

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

// int8 pages: every (token, kv head) row of head_dim values is stored as int8 with one fp32 scale
// = max|x| / 127 (k_scale / v_scale: [pages * page_size, kv_heads]). The head_dim / 8 threads that
// share a row find the maximum with shuffles; a thread quantises and stores 8 values (8 bytes).
__global__ void kv_append_int8_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                      signed char* __restrict__ k_cache, signed char* __restrict__ v_cache,
                                      float* __restrict__ k_scale, float* __restrict__ v_scale,
                                      const int* __restrict__ block_table, const int* __restrict__ positions,
                                      const int* __restrict__ seq_ids, int tokens, int kv_heads, int head_dim,
                                      int page_size, int max_pages, long long kv_tok_stride) {
  const int row = kv_heads * head_dim;
  const int per_tok = row >> 3;
  const int lpt = head_dim >> 3;      // 8 or 16 lanes per row, aligned inside the warp
  const long long total = (long long)tokens * per_tok;
  const long long padded = (total + 31) / 32 * 32;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < padded;
       i += (long long)gridDim.x * blockDim.x) {
    const bool valid = i < total;
    const int t = valid ? (int)(i / per_tok) : 0, c = valid ? (int)(i % per_tok) * 8 : 0;
    float kf[8], vf[8];
    unpack8(ldg8(k, (long long)t * kv_tok_stride + c), kf);
    unpack8(ldg8(v, (long long)t * kv_tok_stride + c), vf);
    float ka = 0.f, va = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      ka = fmaxf(ka, fabsf(kf[j]));
      va = fmaxf(va, fabsf(vf[j]));
    }
    for (int o = lpt / 2; o > 0; o >>= 1) {
      ka = fmaxf(ka, __shfl_xor_sync(0xffffffffu, ka, o));
      va = fmaxf(va, __shfl_xor_sync(0xffffffffu, va, o));
    }
    if (!valid) continue;
    const int pos = positions[t], seq = seq_ids[t];
    const int page = block_table[(long long)seq * max_pages + pos / page_size];
    if (page < 0) continue;
    const long long tokrow = (long long)page * page_size + pos % page_size;
    const float kinv = ka > 0.f ? 127.f / ka : 0.f, vinv = va > 0.f ? 127.f / va : 0.f;
    uint32_t kw[2] = {0u, 0u}, vw[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int kq = max(-127, min(127, __float2int_rn(kf[j] * kinv)));
      const int vq = max(-127, min(127, __float2int_rn(vf[j] * vinv)));
      kw[j >> 2] |= (uint32_t)(kq & 0xFF) << (8 * (j & 3));
      vw[j >> 2] |= (uint32_t)(vq & 0xFF) << (8 * (j & 3));
    }
    *reinterpret_cast<uint2*>(k_cache + tokrow * row + c) = make_uint2(kw[0], kw[1]);
    *reinterpret_cast<uint2*>(v_cache + tokrow * row + c) = make_uint2(vw[0], vw[1]);
    if ((c % head_dim) == 0) {
      const int head = c / head_dim;
      k_scale[tokrow * kv_heads + head] = ka / 127.f;
      v_scale[tokrow * kv_heads + head] = va / 127.f;
    }
  }
}

__device__ __forceinline__ void unpack8_int8(uint2 w, float (&f)[8]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[j] = (float)(int)(signed char)((w.x >> (8 * j)) & 0xFF);
    f[4 + j] = (float)(int)(signed char)((w.y >> (8 * j)) & 0xFF);
  }
}

// Merge `nstate` online-softmax states of a CTA (s_m/s_l: [nstate][gstride]; s_acc: state s at
// s_acc + s * acc_stride, laid out [gstride][D]) for the G heads of one (sequence, kv head), publish the partial result of
// this split, and let the last CTA of the (sequence, kv head) combine all splits into `out`.
template <int D>
__device__ __forceinline__ void merge_and_finish(const float* s_m, const float* s_l, const float* s_acc,
                                                 long long acc_stride, int nstate, int gstride, int G, int* s_last, float* __restrict__ scratch,
                                                 int* __restrict__ counters, __nv_bfloat16* __restrict__ out, int b,
                                                 int hkv, int split, int heads, int kv_heads, int splits) {
  const int stride = D + 2;
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float M = -INFINITY;
    for (int s = 0; s < nstate; ++s) M = fmaxf(M, s_m[s * gstride + g]);
    float L = 0.f, A = 0.f;
    for (int s = 0; s < nstate; ++s) {
      const float ms = s_m[s * gstride + g];
      if (ms == -INFINITY) continue;   // empty state: its accumulator may hold anything
      const float w = exp2f(ms - M);
      L += w * s_l[s * gstride + g];
      A += w * s_acc[s * acc_stride + (long long)g * D + d];
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
    *s_last = (prev == splits - 1) ? 1 : 0;
    if (*s_last) counters[b * kv_heads + hkv] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    const float* base = scratch + ((long long)b * heads + hkv * G + g) * splits * stride;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, base[s * stride + D]);
    float L = 0.f, A = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = base[s * stride + D];
      if (ms == -INFINITY) continue;
      const float w = exp2f(ms - M);
      L += w * base[s * stride + D + 1];
      A += w * base[s * stride + d];
    }
    out[((long long)b * heads + hkv * G + g) * D + d] = __float2bfloat16(L > 0.f ? A / L : 0.f);
  }
}

// grid (batch, kv_heads, splits); block 128 threads. G = query heads per kv head, D = head_dim.
// INT8: the pages hold int8 rows with one fp32 scale per (token, kv head) in k_scale / v_scale; a
// lane then loads 8 bytes per token instead of 16 and the scales are folded into the score and
// into the probability.
template <int G, int D, bool INT8>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const void* __restrict__ k_cache_v,
                    const void* __restrict__ v_cache_v, const float* __restrict__ k_scale,
                    const float* __restrict__ v_scale, const int* __restrict__ block_table,
                    const int* __restrict__ context_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ scratch,
                    int* __restrict__ counters, int heads, int kv_heads, int page_size, int max_pages, int splits,
                    float scale_log2, long long q_tok_stride) {
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
  const __nv_bfloat16* k_cache = static_cast<const __nv_bfloat16*>(k_cache_v);
  const __nv_bfloat16* v_cache = static_cast<const __nv_bfloat16*>(v_cache_v);
  const signed char* k_cache8 = static_cast<const signed char*>(k_cache_v);
  const signed char* v_cache8 = static_cast<const signed char*>(v_cache_v);

  float qv[G][8], acc[G][8], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    unpack8(ldg8(q, (long long)b * q_tok_stride + (long long)(hkv * G + g) * D + li * 8), qv[g]);
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }
  const int* bt = block_table + (long long)b * max_pages;
  // Every lane of a warp runs the same number of iterations (the shuffles below need the full
  // warp); a token slot past the end of the range contributes nothing. Each iteration first issues
  // the K/V loads of U token slots, then does the arithmetic, so a warp keeps 2*U 16-byte loads
  // per lane in flight: decode attention is bound by how much of the KV stream is in flight.
  constexpr int U = 4;   // (8 slots for int8 rows measured slower: 700 against 906 GB/s at 32k context)
  for (int tb = t0 + warp * TPW; tb < t1; tb += 4 * TPW * U) {
    bf16x8 kq[U], vq[U];
    uint2 k8[U], v8[U];
    float ks[U], vs[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = tb + u * 4 * TPW + sub;
      valid[u] = t < t1;
      if (valid[u]) {
        const int page = bt[t / page_size];
        const long long tokrow = (long long)page * page_size + t % page_size;
        const long long off = tokrow * row + (long long)hkv * D + li * 8;
        if (INT8) {
          k8[u] = __ldg(reinterpret_cast<const uint2*>(k_cache8 + off));
          v8[u] = __ldg(reinterpret_cast<const uint2*>(v_cache8 + off));
          ks[u] = __ldg(k_scale + tokrow * kv_heads + hkv);
          vs[u] = __ldg(v_scale + tokrow * kv_heads + hkv);
        } else {
          kq[u] = ldg8(k_cache, off);
          vq[u] = ldg8(v_cache, off);
        }
      } else {
        const float z[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        kq[u] = vq[u] = pack8(z);
        k8[u] = v8[u] = make_uint2(0u, 0u);
        ks[u] = vs[u] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[8], vf[8];
      if (INT8) {
        unpack8_int8(k8[u], kf);
        unpack8_int8(v8[u], vf);
      } else {
        unpack8(kq[u], kf);
        unpack8(vq[u], vf);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s += qv[g][i] * kf[i];
#pragma unroll
        for (int o = LPT / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (valid[u]) {
          s *= INT8 ? scale_log2 * ks[u] : scale_log2;
          const float mn = fmaxf(m[g], s);
          const float a = exp2f(m[g] - mn), p = exp2f(s - mn);
          l[g] = l[g] * a + p;
          const float pv = INT8 ? p * vs[u] : p;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * a + pv * vf[i];
          m[g] = mn;
        }
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
  merge_and_finish<D>(&s_m[0][0], &s_l[0][0], &s_acc[0][0][0], (long long)G * D, NSTATE, G, G, &s_last, scratch, counters, out, b, hkv,
                      split, heads, kv_heads, splits);
}

// ---------------------------------------------------------------------------------------------
// Tensor-core decode attention for 16-token pages.
//
// grid (batch, kv_heads, splits), 4 warps. A warp owns every fourth page of the split and streams
// them through a private ring of PD_STAGES shared-memory stages filled by TMA (K and V of one page
// and one kv head: two [16 tokens x 64 dims] 128B-swizzled boxes each). Per page the warp computes
// S = Q K^T with m16n8k16 MMAs (the G <= 8 query heads of the group are rows 0..G-1 of the 16-row
// A operand, loaded once into registers), an online softmax on the accumulator fragments, and
// O += P V with the V fragments read through ldmatrix.trans. Nothing but the page bytes moves.
constexpr int PD_STAGES = 2;

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int D>
struct PdSmem {
  static constexpr int CHUNKS = D / 64;                 // 64-dim boxes per K or V page
  static constexpr int TILE = 16 * 128;                 // one box: 16 tokens x 128 B
  static constexpr int STAGE = 2 * CHUNKS * TILE;       // K + V
  static constexpr int WARP_BYTES = PD_STAGES * STAGE;
  static constexpr int OFF_BAR = 4 * WARP_BYTES;
  static constexpr int OFF_MERGE = OFF_BAR + 4 * PD_STAGES * 8 + 16;   // s_m[4][8], s_l[4][8]
  static constexpr int BYTES = OFF_MERGE + 64 * 4 + 1024;
  static_assert(8 * D * 4 <= WARP_BYTES, "a warp's output state is staged in its own (drained) ring");
};

template <int D>
__global__ void __launch_bounds__(128)
paged_decode_mma_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                        const __nv_bfloat16* __restrict__ q, const int* __restrict__ block_table,
                        const int* __restrict__ context_lens, __nv_bfloat16* __restrict__ out,
                        float* __restrict__ scratch, int* __restrict__ counters, int heads, int kv_heads, int G,
                        int max_pages, int splits, float scale_log2, long long q_tok_stride, int* status) {
  using S = PdSmem<D>;
  constexpr int KS = D / 16;   // k-steps of Q K^T
  constexpr int NT = D / 8;    // n-tiles of P V
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x, hkv = blockIdx.y, split = blockIdx.z;
  uint8_t* wsm = smem + warp * S::WARP_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR) + warp * PD_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::OFF_BAR + 4 * PD_STAGES * 8);
  int* s_last = const_cast<int*>(abort_flag) + 1;
  float* s_m = reinterpret_cast<float*>(smem + S::OFF_MERGE);
  float* s_l = s_m + 32;
  float* w_acc = reinterpret_cast<float*>(wsm);   // this warp's [8][D] output state, written after its ring drained

  if (threadIdx.x == 0) *abort_flag = 0;
  if (lane == 0) {
    for (int s = 0; s < PD_STAGES; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();

  const int ctx = context_lens[b];
  const int n_pages = (ctx + 15) >> 4;
  const int per = (n_pages + splits - 1) / splits;
  const int p0 = split * per, p1 = min(n_pages, p0 + per);
  const int my_pages = (p1 - p0 - warp + 3) >> 2;   // pages p0 + warp, p0 + warp + 4, ... (<= 0: none)
  const int* bt = block_table + (long long)b * max_pages;

  auto issue = [&](int i) {   // lane 0: load the warp's i-th page into stage i % PD_STAGES
    const int st = i % PD_STAGES;
    const int page = bt[p0 + warp + 4 * i];
    uint8_t* dst = wsm + st * S::STAGE;
    mbar_arrive_expect_tx(&full[st], S::STAGE);
#pragma unroll
    for (int c = 0; c < S::CHUNKS; ++c) {
      tma_load_2d(dst + c * S::TILE, &tm_k, &full[st], hkv * D + c * 64, page * 16);
      tma_load_2d(dst + (S::CHUNKS + c) * S::TILE, &tm_v, &full[st], hkv * D + c * 64, page * 16);
    }
  };
  if (lane == 0)
    for (int i = 0; i < PD_STAGES && i < my_pages; ++i) issue(i);

  // Q fragments: row r = lane / 4 of the group (zero rows beyond G), columns 2t, 2t+1 (+8) of each k-step
  const int r = lane >> 2, t = lane & 3;
  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    qa[ks][0] = qa[ks][1] = qa[ks][2] = qa[ks][3] = 0u;
    if (r < G) {
      const __nv_bfloat16* qp = q + (long long)b * q_tok_stride + (long long)(hkv * G + r) * D + ks * 16 + 2 * t;
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(qp);
      qa[ks][2] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
  }
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  // per-lane ldmatrix row selectors
  const int k_tok = ((lane >> 4) << 3) + (lane & 7), k_unit = (lane >> 3) & 1;   // K: matrices by (token half, unit)
  const int v_tok = (((lane >> 3) & 1) << 3) + (lane & 7), v_unit = lane >> 4;   // V: matrices by (unit, token half)
  const uint32_t wsm_addr = smem_u32(wsm);
  bool ok = true;
  for (int i = 0; i < my_pages; ++i) {
    const int st = i % PD_STAGES;
    ok = mbar_wait(&full[st], (i / PD_STAGES) & 1, abort_flag, status, 70);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const uint32_t kbase = wsm_addr + st * S::STAGE, vbase = kbase + S::CHUNKS * S::TILE;
    // ---- S = Q K^T : two n-tiles of 8 tokens
    float sc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int unit = ((ks & 3) << 1) + k_unit;
      uint32_t kb[4];
      ldmatrix_x4(kbase + (ks >> 2) * S::TILE + k_tok * 128 + ((unit ^ (k_tok & 7)) << 4), kb);
      mma_bf16_16816(sc[0], qa[ks], kb[0], kb[1]);
      mma_bf16_16816(sc[1], qa[ks], kb[2], kb[3]);
    }
    // ---- online softmax on rows 0..7 (fragment elements 0, 1); tokens past the context are masked
    const int tok0 = (p0 + warp + 4 * i) * 16 + 2 * t;
    float pv[2][2];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float v = (tok0 + j * 8 + e < ctx) ? sc[j][e] * scale_log2 : -INFINITY;
        pv[j][e] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);   // finite: every page of the range holds a valid token
    const float alpha = exp2f(m_run - m_new);
    float psum = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        pv[j][e] = exp2f(pv[j][e] - m_new);
        psum += pv[j][e];
      }
    l_run = l_run * alpha + psum;
    m_run = m_new;
    uint32_t pa[4];
    pa[0] = pack_bf16x2(pv[0][0], pv[0][1]);
    pa[1] = 0u;
    pa[2] = pack_bf16x2(pv[1][0], pv[1][1]);
    pa[3] = 0u;
    // ---- O = O * alpha + P V
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      const int unit = ((np & 3) << 1) + v_unit;
      uint32_t vb[4];
      ldmatrix_x4_trans(vbase + (np >> 2) * S::TILE + v_tok * 128 + ((unit ^ (v_tok & 7)) << 4), vb);
      o[2 * np][0] *= alpha;
      o[2 * np][1] *= alpha;
      o[2 * np + 1][0] *= alpha;
      o[2 * np + 1][1] *= alpha;
      mma_bf16_16816(o[2 * np], pa, vb[0], vb[1]);
      mma_bf16_16816(o[2 * np + 1], pa, vb[2], vb[3]);
    }
    __syncwarp();
    if (lane == 0 && i + PD_STAGES < my_pages) issue(i + PD_STAGES);
  }

  // ---- publish the warp's state (rows 0..G-1), merge warps, then splits
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (t == 0) {
    s_m[warp * 8 + r] = ok ? m_run : -INFINITY;   // a warp that gave up contributes nothing
    s_l[warp * 8 + r] = l_run;
  }
  if (ok) {   // every load this warp issued has landed and been consumed
#pragma unroll
    for (int n = 0; n < NT; ++n)
      *reinterpret_cast<float2*>(&w_acc[r * D + n * 8 + 2 * t]) = make_float2(o[n][0], o[n][1]);
  }
  __syncthreads();
  merge_and_finish<D>(s_m, s_l, reinterpret_cast<const float*>(smem), S::WARP_BYTES / 4, 4, 8, G, s_last, scratch, counters, out, b, hkv, split, heads, kv_heads,
                      splits);
}

// ---------------------------------------------------------------------------------------------
// Tensor-core decode attention over int8 pages (16-token pages, head_dim 128).
//
// Same grid, warp roles and split merge as the bf16 kernel above. A warp's 16 KB of shared memory
// hold a ring of PD_STAGES raw stages (K and V of one page as [16 tokens x 128 B] int8 boxes,
// filled by TMA) and one pair of expanded tiles (K and V as fp16 in the 128B-swizzled layout that
// the ldmatrix addressing below expects). Per page the warp expands the raw stage (16 bytes per
// lane and step: int8 -> fp16 is exact and costs one byte permute and one subtract per pair of
// values), hands the raw stage back to TMA at once, and runs the same m16n8k16 products in fp16.
// The fp32 scales (one per token and kv head) never touch the tiles: the K scale multiplies the
// score, the V scale the probability, both in fp32 on the accumulator fragments.
__device__ __forceinline__ void mma_f16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Four int8 in `w` -> two fp16x2 words (values 0,1 and 2,3). x ^ 0x80 is the value + 128 as an
// unsigned byte u; 0x6400 | u is the fp16 number 1024 + u; subtracting 1152 leaves the value.
__device__ __forceinline__ void int8x4_to_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t x = w ^ 0x80808080u;
  uint32_t l = __byte_perm(x, 0x64646464u, 0x4140), h = __byte_perm(x, 0x64646464u, 0x4342);
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
  __half2 lv = __hsub2(*reinterpret_cast<__half2*>(&l), bias), hv = __hsub2(*reinterpret_cast<__half2*>(&h), bias);
  lo = *reinterpret_cast<uint32_t*>(&lv);
  hi = *reinterpret_cast<uint32_t*>(&hv);
}

__global__ void __launch_bounds__(128)
paged_decode_mma_int8_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                             const __nv_bfloat16* __restrict__ q, const float* __restrict__ k_scale,
                             const float* __restrict__ v_scale, const int* __restrict__ block_table,
                             const int* __restrict__ context_lens, __nv_bfloat16* __restrict__ out,
                             float* __restrict__ scratch, int* __restrict__ counters, int heads, int kv_heads, int G,
                             int max_pages, int splits, float scale_log2, long long q_tok_stride, int* status) {
  constexpr int D = 128;
  using S = PdSmem<D>;
  constexpr int KS = D / 16, NT = D / 8;
  constexpr int RAW_HALF = 16 * D;            // K (or V) of one page as int8
  constexpr int RAW = 2 * RAW_HALF;
  constexpr int CONV_OFF = PD_STAGES * RAW;   // expanded tiles behind the raw ring
  static_assert(CONV_OFF + 2 * S::CHUNKS * S::TILE == S::WARP_BYTES, "raw ring + expanded tiles fill the warp's share");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x, hkv = blockIdx.y, split = blockIdx.z;
  uint8_t* wsm = smem + warp * S::WARP_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR) + warp * PD_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::OFF_BAR + 4 * PD_STAGES * 8);
  int* s_last = const_cast<int*>(abort_flag) + 1;
  float* s_m = reinterpret_cast<float*>(smem + S::OFF_MERGE);
  float* s_l = s_m + 32;
  float* w_acc = reinterpret_cast<float*>(wsm);   // [8][D] output state, written after the ring drained

  if (threadIdx.x == 0) *abort_flag = 0;
  if (lane == 0) {
    for (int s = 0; s < PD_STAGES; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();

  const int ctx = context_lens[b];
  const int n_pages = (ctx + 15) >> 4;
  const int per = (n_pages + splits - 1) / splits;
  const int p0 = split * per, p1 = min(n_pages, p0 + per);
  const int my_pages = (p1 - p0 - warp + 3) >> 2;
  const int* bt = block_table + (long long)b * max_pages;

  auto issue = [&](int i) {   // lane 0: the warp's i-th page into raw stage i % PD_STAGES
    const int st = i % PD_STAGES;
    const int page = bt[p0 + warp + 4 * i];
    uint8_t* dst = wsm + st * RAW;
    mbar_arrive_expect_tx(&full[st], RAW);
    tma_load_2d(dst, &tm_k, &full[st], hkv * D, page * 16);
    tma_load_2d(dst + RAW_HALF, &tm_v, &full[st], hkv * D, page * 16);
  };
  if (lane == 0)
    for (int i = 0; i < PD_STAGES && i < my_pages; ++i) issue(i);

  const int r = lane >> 2, t = lane & 3;
  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    qa[ks][0] = qa[ks][1] = qa[ks][2] = qa[ks][3] = 0u;
    if (r < G) {
      const __nv_bfloat16* qp = q + (long long)b * q_tok_stride + (long long)(hkv * G + r) * D + ks * 16 + 2 * t;
      qa[ks][0] = pack_f16x2(__bfloat162float(qp[0]), __bfloat162float(qp[1]));
      qa[ks][2] = pack_f16x2(__bfloat162float(qp[8]), __bfloat162float(qp[9]));
    }
  }
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  const int k_tok = ((lane >> 4) << 3) + (lane & 7), k_unit = (lane >> 3) & 1;
  const int v_tok = (((lane >> 3) & 1) << 3) + (lane & 7), v_unit = lane >> 4;
  const uint32_t conv_addr = smem_u32(wsm) + CONV_OFF;
  uint8_t* convk = wsm + CONV_OFF;
  uint8_t* convv = convk + S::CHUNKS * S::TILE;
  bool ok = true;
  for (int i = 0; i < my_pages; ++i) {
    const int st = i % PD_STAGES;
    const int lpage = p0 + warp + 4 * i;
    // scales of the four tokens this lane's score / probability fragments cover; issued before the
    // wait so that their latency hides behind it. Tokens past the context are never used.
    const long long tokrow0 = (long long)bt[lpage] * 16;
    const int tok0 = lpage * 16 + 2 * t;
    float ksc[2][2], vsc[2][2];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const bool live = tok0 + j * 8 + e < ctx;
        const long long idx = (tokrow0 + 2 * t + j * 8 + e) * kv_heads + hkv;
        ksc[j][e] = live ? __ldg(k_scale + idx) : 0.f;
        vsc[j][e] = live ? __ldg(v_scale + idx) : 0.f;
      }
    ok = mbar_wait(&full[st], (i / PD_STAGES) & 1, abort_flag, status, 71);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    // ---- expand the raw stage: chunk c = 16 dims of token c / 8
    const uint8_t* rawk = wsm + st * RAW;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const int c = lane + 32 * kk;
      const int tok = c >> 3, g = c & 7;
      const uint4 kr = *reinterpret_cast<const uint4*>(rawk + c * 16);
      const uint4 vr = *reinterpret_cast<const uint4*>(rawk + RAW_HALF + c * 16);
      uint4 k0, k1, v0, v1;
      int8x4_to_f16x4(kr.x, k0.x, k0.y);
      int8x4_to_f16x4(kr.y, k0.z, k0.w);
      int8x4_to_f16x4(kr.z, k1.x, k1.y);
      int8x4_to_f16x4(kr.w, k1.z, k1.w);
      int8x4_to_f16x4(vr.x, v0.x, v0.y);
      int8x4_to_f16x4(vr.y, v0.z, v0.w);
      int8x4_to_f16x4(vr.z, v1.x, v1.y);
      int8x4_to_f16x4(vr.w, v1.z, v1.w);
      const int off = (g >> 2) * S::TILE + tok * 128;
      const int u0 = (g & 3) << 1;
      const int a0 = off + ((u0 ^ (tok & 7)) << 4), a1 = off + (((u0 + 1) ^ (tok & 7)) << 4);
      *reinterpret_cast<uint4*>(convk + a0) = k0;
      *reinterpret_cast<uint4*>(convk + a1) = k1;
      *reinterpret_cast<uint4*>(convv + a0) = v0;
      *reinterpret_cast<uint4*>(convv + a1) = v1;
    }
    __syncwarp();   // raw stage consumed by every lane; expanded tiles visible to the warp
    if (lane == 0 && i + PD_STAGES < my_pages) issue(i + PD_STAGES);
    const uint32_t kbase = conv_addr, vbase = conv_addr + S::CHUNKS * S::TILE;
    // ---- S = Q K^T
    float sc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int unit = ((ks & 3) << 1) + k_unit;
      uint32_t kb[4];
      ldmatrix_x4(kbase + (ks >> 2) * S::TILE + k_tok * 128 + ((unit ^ (k_tok & 7)) << 4), kb);
      mma_f16_16816(sc[0], qa[ks], kb[0], kb[1]);
      mma_f16_16816(sc[1], qa[ks], kb[2], kb[3]);
    }
    // ---- online softmax; the K scale enters here, the V scale goes into the probabilities
    float pv[2][2];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float v = (tok0 + j * 8 + e < ctx) ? sc[j][e] * ksc[j][e] * scale_log2 : -INFINITY;
        pv[j][e] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float alpha = exp2f(m_run - m_new);
    float psum = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float pe = exp2f(pv[j][e] - m_new);   // 0 for masked tokens
        psum += pe;
        pv[j][e] = (tok0 + j * 8 + e < ctx) ? pe * vsc[j][e] : 0.f;
      }
    l_run = l_run * alpha + psum;
    m_run = m_new;
    uint32_t pa[4];
    pa[0] = pack_f16x2(pv[0][0], pv[0][1]);
    pa[1] = 0u;
    pa[2] = pack_f16x2(pv[1][0], pv[1][1]);
    pa[3] = 0u;
    // ---- O = O * alpha + P V
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      const int unit = ((np & 3) << 1) + v_unit;
      uint32_t vb[4];
      ldmatrix_x4_trans(vbase + (np >> 2) * S::TILE + v_tok * 128 + ((unit ^ (v_tok & 7)) << 4), vb);
      o[2 * np][0] *= alpha;
      o[2 * np][1] *= alpha;
      o[2 * np + 1][0] *= alpha;
      o[2 * np + 1][1] *= alpha;
      mma_f16_16816(o[2 * np], pa, vb[0], vb[1]);
      mma_f16_16816(o[2 * np + 1], pa, vb[2], vb[3]);
    }
    __syncwarp();   // the expanded tiles are free for the next page
  }

  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (t == 0) {
    s_m[warp * 8 + r] = ok ? m_run : -INFINITY;
    s_l[warp * 8 + r] = l_run;
  }
  if (ok) {
#pragma unroll
    for (int n = 0; n < NT; ++n)
      *reinterpret_cast<float2*>(&w_acc[r * D + n * 8 + 2 * t]) = make_float2(o[n][0], o[n][1]);
  }
  __syncthreads();
  merge_and_finish<D>(s_m, s_l, reinterpret_cast<const float*>(smem), S::WARP_BYTES / 4, 4, 8, G, s_last, scratch, counters, out, b, hkv,
                      split, heads, kv_heads, splits);
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
                       int kv_heads, int head_dim, int page_size, int max_pages, int cache_pages, int splits,
                       float scale, int* status, cudaStream_t stream, long long q_tok_stride) {
  if (q_tok_stride <= 0) q_tok_stride = (long long)heads * head_dim;
  MB_REQUIRE(q_tok_stride % 8 == 0, "paged_attn_decode: query token stride must be a multiple of 8 elements");
  MB_REQUIRE(heads % kv_heads == 0, "paged_attn_decode: heads must be a multiple of kv_heads");
  MB_REQUIRE(splits >= 1, "paged_attn_decode: splits must be positive");
  if (batch == 0) return;
  const int G = heads / kv_heads;
  const dim3 grid(batch, kv_heads, splits);
  const float sl2 = scale * 1.4426950408889634f;
  if (page_size == 16 && G <= 8 && (head_dim == 64 || head_dim == 128)) {
    // K / V cache as [cache_pages * 16 tokens, kv_heads * head_dim]; one box = 16 tokens x 64 dims
    uint64_t dims[2] = {(uint64_t)kv_heads * head_dim, (uint64_t)cache_pages * 16};
    uint64_t strides[1] = {(uint64_t)kv_heads * head_dim * 2};
    uint32_t box[2] = {64, 16};
    const CUtensorMap tk = make_tensor_map(k_cache, TmaDType::BF16, 2, dims, strides, box, true);
    const CUtensorMap tv = make_tensor_map(v_cache, TmaDType::BF16, 2, dims, strides, box, true);
#define MB_PDM(DD)                                                                                                 \
  do {                                                                                                             \
    static bool configured = false;                                                                                \
    if (!configured) {                                                                                             \
      MB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_mma_kernel<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         PdSmem<DD>::BYTES));                                                      \
      configured = true;                                                                                           \
    }                                                                                                              \
    paged_decode_mma_kernel<DD><<<grid, 128, PdSmem<DD>::BYTES, stream>>>(                                         \
        tk, tv, (const __nv_bfloat16*)q, block_table, context_lens, (__nv_bfloat16*)out, scratch, counters, heads, \
        kv_heads, G, max_pages, splits, sl2, q_tok_stride, status);                                                              \
  } while (0)
    if (head_dim == 128) MB_PDM(128);
    else MB_PDM(64);
#undef MB_PDM
    count_launch();
    check_launch();
    return;
  }
#define MB_PD(GG, DD)                                                                                         \
  paged_decode_kernel<GG, DD, false><<<grid, 128, 0, stream>>>(                                               \
      (const __nv_bfloat16*)q, k_cache, v_cache, nullptr, nullptr, block_table, context_lens,                 \
      (__nv_bfloat16*)out, scratch, counters, heads, kv_heads, page_size, max_pages, splits, sl2, q_tok_stride)
  if (head_dim == 128) {
    if (G == 1) MB_PD(1, 128);
    else if (G == 2) MB_PD(2, 128);
    else if (G == 4) MB_PD(4, 128);
    else MB_REQUIRE(false, "paged_attn_decode: GQA group must be 1, 2 or 4 for this page size");
  } else if (head_dim == 64) {
    if (G == 1) MB_PD(1, 64);
    else if (G == 2) MB_PD(2, 64);
    else if (G == 4) MB_PD(4, 64);
    else MB_REQUIRE(false, "paged_attn_decode: GQA group must be 1, 2 or 4 for this page size");
  } else {
    MB_REQUIRE(false, "paged_attn_decode: head_dim must be 64 or 128");
  }
#undef MB_PD
  count_launch();
  check_launch();
}

void kv_append_int8(const void* k, const void* v, void* k_cache, void* v_cache, float* k_scale, float* v_scale,
                    const int* block_table, const int* positions, const int* seq_ids, int tokens, int kv_heads,
                    int head_dim, int page_size, int max_pages, long long kv_tok_stride, cudaStream_t stream) {
  MB_REQUIRE(head_dim == 64 || head_dim == 128, "kv_append_int8: head_dim must be 64 or 128");
  MB_REQUIRE(kv_tok_stride % 8 == 0, "kv_append_int8: token stride must be a multiple of 8 elements");
  if (tokens == 0) return;
  const long long work = ((long long)tokens * kv_heads * head_dim / 8 + 31) / 32 * 32;
  long long g = (work + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  kv_append_int8_kernel<<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                    (signed char*)k_cache, (signed char*)v_cache, k_scale, v_scale,
                                                    block_table, positions, seq_ids, tokens, kv_heads, head_dim,
                                                    page_size, max_pages, kv_tok_stride);
  count_launch();
  check_launch();
}

void paged_attn_decode_int8(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                            const float* v_scale, const int* block_table, const int* context_lens, void* out,
                            float* scratch, int* counters, int batch, int heads, int kv_heads, int head_dim,
                            int page_size, int max_pages, int cache_pages, int splits, float scale, int* status,
                            cudaStream_t stream, long long q_tok_stride) {
  if (q_tok_stride <= 0) q_tok_stride = (long long)heads * head_dim;
  MB_REQUIRE(q_tok_stride % 8 == 0, "paged_attn_decode_int8: query token stride must be a multiple of 8 elements");
  MB_REQUIRE(heads % kv_heads == 0, "paged_attn_decode_int8: heads must be a multiple of kv_heads");
  MB_REQUIRE(splits >= 1, "paged_attn_decode_int8: splits must be positive");
  if (batch == 0) return;
  const int G = heads / kv_heads;
  const dim3 grid(batch, kv_heads, splits);
  const float sl2 = scale * 1.4426950408889634f;
  if (page_size == 16 && G <= 8 && head_dim == 128) {
    // Measured faster than the scalar kernel below for every group size (1, 2 and 4 query heads per
    // kv head: 3.2 / 2.8 / 2.6 TB/s of int8 bytes against 2.4 / 1.4 / 0.9 at 32k context).
    // K / V cache as [cache_pages * 16 tokens, kv_heads * 128] bytes; one box = 16 tokens x 128 B
    uint64_t dims[2] = {(uint64_t)kv_heads * head_dim, (uint64_t)cache_pages * 16};
    uint64_t strides[1] = {(uint64_t)kv_heads * head_dim};
    uint32_t box[2] = {128, 16};
    const CUtensorMap tk = make_tensor_map(k_cache, TmaDType::U8, 2, dims, strides, box, false);
    const CUtensorMap tv = make_tensor_map(v_cache, TmaDType::U8, 2, dims, strides, box, false);
    static bool configured = false;
    if (!configured) {
      MB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_mma_int8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         PdSmem<128>::BYTES));
      configured = true;
    }
    paged_decode_mma_int8_kernel<<<grid, 128, PdSmem<128>::BYTES, stream>>>(
        tk, tv, (const __nv_bfloat16*)q, k_scale, v_scale, block_table, context_lens, (__nv_bfloat16*)out, scratch,
        counters, heads, kv_heads, G, max_pages, splits, sl2, q_tok_stride, status);
    count_launch();
    check_launch();
    return;
  }
#define MB_PD8(GG, DD)                                                                                        \
  paged_decode_kernel<GG, DD, true><<<grid, 128, 0, stream>>>(                                                \
      (const __nv_bfloat16*)q, k_cache, v_cache, k_scale, v_scale, block_table, context_lens,                 \
      (__nv_bfloat16*)out, scratch, counters, heads, kv_heads, page_size, max_pages, splits, sl2, q_tok_stride)
  if (head_dim == 128) {
    if (G == 1) MB_PD8(1, 128);
    else if (G == 2) MB_PD8(2, 128);
    else if (G == 4) MB_PD8(4, 128);
    else MB_REQUIRE(false, "paged_attn_decode_int8: GQA group must be 1, 2 or 4");
  } else if (head_dim == 64) {
    if (G == 1) MB_PD8(1, 64);
    else if (G == 2) MB_PD8(2, 64);
    else if (G == 4) MB_PD8(4, 64);
    else MB_REQUIRE(false, "paged_attn_decode_int8: GQA group must be 1, 2 or 4");
  } else {
    MB_REQUIRE(false, "paged_attn_decode_int8: head_dim must be 64 or 128");
  }
#undef MB_PD8
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
