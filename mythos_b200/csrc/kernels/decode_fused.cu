// Fused epilogue kernels of the decode step. A decode step at tensor-parallel width 8 is bound by
// launch latency (a dozen small kernels per layer), so the kernels that only reshuffle a few hundred
// kilobytes are merged:
//
//   sum_residual_rmsnorm   [split-K fp32 accumulator | W bf16 all-reduce slots] + residual stream
//                          -> new residual stream, RMS-normalised activations     (replaces finalize /
//                          tp_reduce_slots followed by the fused add + RMSNorm kernel)
//   qkv_rope_append        fp32 accumulator of the fused QKV projection -> rotated Q (bf16), rotated K
//                          and V written straight into their KV-cache pages         (replaces finalize,
//                          RoPE and kv_append)
//   finalize_gate          fp32 accumulator of the gate/up projection -> act(gate) * up (bf16)
//   tp_sum_residual_rmsnorm   the tensor-parallel form of the first: push this rank's partial row to
//                          every peer, signal a per-row flag, wait for the peers' flags of the same
//                          row, then sum + residual + RMSNorm, all in one launch (replaces push
//                          kernel, barrier kernel and sum kernel)
//
// Accumulators are zeroed as they are read (they are shared split-K scratch). Reference formulas:
// rms_norm (src/math.cpp:182-205), RotaryEmbedding::apply (src/transformer.cpp:118-139), FFN
// (src/transformer.cpp:373-387), KVCache::append (src/kv_cache.cpp:78-137).
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace mb {
namespace {

constexpr int SRN_THREADS = 512;
constexpr int SRN_MAX_VEC = 4;   // 8-element vectors per thread: rows up to 512 * 8 * 4 = 16384 wide

__device__ __forceinline__ bf16x8 ldcg8(const void* base, long long elem_index) {
  const uint4 v = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem_index));
  return *reinterpret_cast<const bf16x8*>(&v);
}

// One CTA per row.
__global__ void __launch_bounds__(SRN_THREADS)
sum_residual_rmsnorm_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ slots, int n_slots,
                            long long slot_stride, const __nv_bfloat16* __restrict__ residual,
                            const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ stream_out,
                            __nv_bfloat16* __restrict__ normed, int dim, float eps) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const int nvec = dim >> 3;
  float vals[SRN_MAX_VEC][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < SRN_MAX_VEC; ++it) {
    const int v = threadIdx.x + it * SRN_THREADS;
    if (v < nvec) {
      const long long e = row * dim + (long long)v * 8;
      float (&x)[8] = vals[it];
      if (acc) {
        float4* a = reinterpret_cast<float4*>(acc + e);
        const float4 lo = a[0], hi = a[1];
        a[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        a[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w; x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = 0.f;
        for (int s = 0; s < n_slots; ++s) {   // written by peers: read through L2
          float f[8];
          unpack8(ldcg8(slots, s * slot_stride + e), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] += f[j];
        }
      }
      if (residual) {
        float f[8];
        unpack8(ldg8(residual, e), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] += f[j];
      }
      // the stream is stored in bf16; normalise what is stored so both outputs agree
      const bf16x8 h = pack8(x);
      stg8(stream_out, e, h);
      unpack8(h, x);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int it = 0; it < SRN_MAX_VEC; ++it) {
    const int v = threadIdx.x + it * SRN_THREADS;
    if (v < nvec) {
      float g[8], y[8];
      unpack8(ldg8(gamma, (long long)v * 8), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = vals[it][j] * rstd * g[j];
      stg8(normed, row * dim + (long long)v * 8, pack8(y));
    }
  }
}

__device__ __forceinline__ void st_release_sys_i32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Tensor-parallel sum of a decode-sized activation fused with the residual add and RMSNorm.
// One CTA per row; rows are independent, so no CTA ever waits on another CTA of its own grid.
//   1. (acc != null) the row of this rank's fp32 partial is rounded to bf16 and stored into slot
//      `rank` of the staging buffer of every rank (acc is zeroed for the next split-K GEMM);
//      with acc == null the GEMM before this launch has already stored the slots.
//   2. thread r < world announces the row to rank r: flags[r][parity][rank][row] = epoch (release at
//      system scope, after a system fence that covers the row's stores), then waits for
//      flags[me][parity][r][row] >= epoch with a cycle limit; on expiry the status word is set
//      and the row is left alone.
//   3. the world's slots of the row are read through L2, summed with the residual, stored as the
//      new residual stream and normalised.
// The epoch lives on the device (one increment per launch, done by the CTA that is last to have
// read it), so the launch can be replayed from a CUDA graph.
__global__ void __launch_bounds__(SRN_THREADS)
tp_sum_residual_rmsnorm_kernel(float* __restrict__ acc, PeerPtrs staging, PeerPtrs flags, int rank, int world,
                               long long slot_stride, long long flag_base, int max_rows,
                               const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ gamma,
                               __nv_bfloat16* __restrict__ stream_out, __nv_bfloat16* __restrict__ normed, int dim,
                               float eps, int* epoch_dev, int* arrive, long long limit_cycles, int* status) {
  __shared__ float scratch[32];
  __shared__ int s_epoch, s_ok;
  const long long row = blockIdx.x;
  const int nvec = dim >> 3;
  if (threadIdx.x == 0) {
    const int e = *reinterpret_cast<volatile int*>(epoch_dev) + 1;
    s_epoch = e;
    s_ok = 1;
    __threadfence();
    if (atomicAdd(arrive, 1) == (int)gridDim.x - 1) {   // every CTA has read the old epoch
      *arrive = 0;
      *epoch_dev = e;
    }
  }
  if (acc) {
#pragma unroll
    for (int it = 0; it < SRN_MAX_VEC; ++it) {
      const int v = threadIdx.x + it * SRN_THREADS;
      if (v < nvec) {
        const long long e = row * dim + (long long)v * 8;
        float4* a = reinterpret_cast<float4*>(acc + e);
        const float4 lo = a[0], hi = a[1];
        a[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        a[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        const float x[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        const bf16x8 h = pack8(x);
        for (int r = 0; r < world; ++r) {
          const int dst = (rank + r) % world;
          stg8(staging.p[dst], (long long)rank * slot_stride + e, h);
        }
      }
    }
  }
  // The row's stores are ordered before the barrier (CTA scope); the signalling threads then fence at
  // system scope before their release store, which carries the whole CTA's stores with it. A system
  // fence in every thread costs about 5 us per launch here.
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const int r = threadIdx.x, e = s_epoch;
    __threadfence_system();
    st_release_sys_i32(reinterpret_cast<int*>(flags.p[r]) + flag_base + (long long)rank * max_rows + row, e);
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + flag_base + (long long)r * max_rows + row;
    const long long t0 = clock64();
    while (ld_acquire_sys_i32(mine) < e) {
      if (clock64() - t0 > limit_cycles) {
        if (status) atomicCAS(status, 0, 1 | (41 << 16));
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const __nv_bfloat16* slots = reinterpret_cast<const __nv_bfloat16*>(staging.p[rank]);
  float vals[SRN_MAX_VEC][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < SRN_MAX_VEC; ++it) {
    const int v = threadIdx.x + it * SRN_THREADS;
    if (v < nvec) {
      const long long e = row * dim + (long long)v * 8;
      float (&x)[8] = vals[it];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = 0.f;
      for (int s = 0; s < world; ++s) {   // written by peers: read through L2
        float f[8];
        unpack8(ldcg8(slots, s * slot_stride + e), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] += f[j];
      }
      if (residual) {
        float f[8];
        unpack8(ldg8(residual, e), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] += f[j];
      }
      const bf16x8 h = pack8(x);
      stg8(stream_out, e, h);
      unpack8(h, x);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int it = 0; it < SRN_MAX_VEC; ++it) {
    const int v = threadIdx.x + it * SRN_THREADS;
    if (v < nvec) {
      float g[8], y[8];
      unpack8(ldg8(gamma, (long long)v * 8), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = vals[it][j] * rstd * g[j];
      stg8(normed, row * dim + (long long)v * 8, pack8(y));
    }
  }
}

// One thread per (token, head slot, 8-wide group of the first half of the head): handles the pair
// group (d, d + D/2). Head slots [0, H) are Q, [H, H + Hkv) K, [H + Hkv, H + 2 Hkv) V.
// With k_cache8 / v_cache8 set the pages are int8: the head_dim / 16 threads of a head slot (adjacent
// lanes, aligned in the warp) find max|x| with shuffles and store 8 + 8 bytes each plus one fp32
// scale = max|x| / 127 per (token, kv head). Every lane of a warp reaches the shuffles: lanes past
// the end of the work carry zeros and store nothing.
__global__ void qkv_rope_append_kernel(float* __restrict__ acc, const int* __restrict__ pos,
                                       const int* __restrict__ seq_ids, const int* __restrict__ block_table,
                                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                                       __nv_bfloat16* __restrict__ v_cache, signed char* __restrict__ k_cache8,
                                       signed char* __restrict__ v_cache8, float* __restrict__ k_scale,
                                       float* __restrict__ v_scale, int tokens, int heads, int kv_heads,
                                       int head_dim, int page_size, int max_pages, float log2_theta) {
  const int half = head_dim >> 1, groups = half >> 3, slots = heads + 2 * kv_heads;
  const long long raw_gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool valid = raw_gid < (long long)tokens * slots * groups;
  const long long gid = valid ? raw_gid : 0;
  const int g = (int)(gid % groups);
  const int hs = (int)((gid / groups) % slots);
  const int t = (int)(gid / ((long long)groups * slots));
  float* src = acc + ((long long)t * slots + hs) * head_dim;
  float a[8], b[8];
  if (valid) {
    float4* pa = reinterpret_cast<float4*>(src + g * 8);
    float4* pb = reinterpret_cast<float4*>(src + half + g * 8);
    const float4 a0 = pa[0], a1 = pa[1], b0 = pb[0], b1 = pb[1];
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    pa[0] = z; pa[1] = z; pb[0] = z; pb[1] = z;
    a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w; a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
    b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = b[i] = 0.f;
  }
  const int p = pos[t];
  if (hs < heads + kv_heads && log2_theta > 0.f) {   // Q and K are rotated
    // the projection result is rounded to bf16 first, as the unfused path does
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a[i] = __bfloat162float(__float2bfloat16(a[i]));
      b[i] = __bfloat162float(__float2bfloat16(b[i]));
      const int j = g * 8 + i;
      const float inv_freq = exp2f(-2.0f * (float)j / (float)head_dim * log2_theta);
      float sn, cs;
      sincosf((float)p * inv_freq, &sn, &cs);
      const float ra = a[i] * cs - b[i] * sn, rb = a[i] * sn + b[i] * cs;
      a[i] = ra;
      b[i] = rb;
    }
  }
  float amax = 0.f;
  if (k_cache8 != nullptr) {   // same for every thread of the grid
    // quantise what the bf16 path would have stored
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a[i] = __bfloat162float(__float2bfloat16(a[i]));
      b[i] = __bfloat162float(__float2bfloat16(b[i]));
      amax = fmaxf(amax, fmaxf(fabsf(a[i]), fabsf(b[i])));
    }
    for (int o = groups >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  }
  if (!valid) return;
  if (hs < heads) {
    __nv_bfloat16* dst = q_out + ((long long)t * heads + hs) * head_dim;
    stg8(dst, g * 8, pack8(a));
    stg8(dst, half + g * 8, pack8(b));
    return;
  }
  const int seq = seq_ids[t];
  const int page = block_table[(long long)seq * max_pages + p / page_size];
  if (page < 0) return;
  const bool is_k = hs < heads + kv_heads;
  const int kvh = is_k ? hs - heads : hs - heads - kv_heads;
  const long long row = ((long long)page * page_size + p % page_size) * kv_heads + kvh;
  if (k_cache8 != nullptr) {
    const float inv = amax > 0.f ? 127.f / amax : 0.f;
    uint32_t wa[2] = {0u, 0u}, wb[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int qa = max(-127, min(127, __float2int_rn(a[i] * inv)));
      const int qb = max(-127, min(127, __float2int_rn(b[i] * inv)));
      wa[i >> 2] |= (uint32_t)(qa & 0xFF) << (8 * (i & 3));
      wb[i >> 2] |= (uint32_t)(qb & 0xFF) << (8 * (i & 3));
    }
    signed char* dst8 = (is_k ? k_cache8 : v_cache8) + row * head_dim;
    *reinterpret_cast<uint2*>(dst8 + g * 8) = make_uint2(wa[0], wa[1]);
    *reinterpret_cast<uint2*>(dst8 + half + g * 8) = make_uint2(wb[0], wb[1]);
    if (g == 0) (is_k ? k_scale : v_scale)[row] = amax / 127.f;
    return;
  }
  __nv_bfloat16* dst = (is_k ? k_cache : v_cache) + row * head_dim;
  stg8(dst, g * 8, pack8(a));
  stg8(dst, half + g * 8, pack8(b));
}

// out[r, c] = act(acc[r, c]) * acc[r, ffn + c]; kind 0 = SiLU, 1 = squared ReLU.
__global__ void finalize_gate_kernel(float* __restrict__ acc, __nv_bfloat16* __restrict__ out, long long rows,
                                     int ffn, int kind) {
  const int per_row = ffn >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c = (int)(i % per_row) * 8;
    float4* pg = reinterpret_cast<float4*>(acc + r * 2 * ffn + c);
    float4* pu = reinterpret_cast<float4*>(acc + r * 2 * ffn + ffn + c);
    const float4 g0 = pg[0], g1 = pg[1], u0 = pu[0], u1 = pu[1];
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    pg[0] = z; pg[1] = z; pu[0] = z; pu[1] = z;
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
    float y[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // gate and up are rounded to bf16 first, as the unfused path stores them
      const float gj = __bfloat162float(__float2bfloat16(g[j])), uj = __bfloat162float(__float2bfloat16(u[j]));
      const float act = kind == 0 ? gj / (1.f + __expf(-gj)) : (gj > 0.f ? gj * gj : 0.f);
      y[j] = act * uj;
    }
    stg8(out, r * ffn + c, pack8(y));
  }
}

}  // namespace

void sum_residual_rmsnorm(float* acc, const void* slots, int n_slots, long long slot_stride, const void* residual,
                          const void* gamma, void* stream_out, void* normed, int rows, int dim, float eps,
                          cudaStream_t stream) {
  MB_REQUIRE((acc != nullptr) != (slots != nullptr), "sum_residual_rmsnorm: exactly one of accumulator / slots");
  MB_REQUIRE(dim % 8 == 0 && dim <= SRN_THREADS * 8 * SRN_MAX_VEC, "sum_residual_rmsnorm: unsupported row width");
  MB_REQUIRE(slots == nullptr || slot_stride % 8 == 0, "sum_residual_rmsnorm: slot stride must be a multiple of 8");
  if (rows == 0) return;
  sum_residual_rmsnorm_kernel<<<rows, SRN_THREADS, 0, stream>>>(
      acc, (const __nv_bfloat16*)slots, n_slots, slot_stride, (const __nv_bfloat16*)residual,
      (const __nv_bfloat16*)gamma, (__nv_bfloat16*)stream_out, (__nv_bfloat16*)normed, dim, eps);
  count_launch();
  check_launch();
}

void tp_sum_residual_rmsnorm(float* acc, const PeerPtrs& staging, const PeerPtrs& flags, int rank, int world,
                             long long slot_stride, int parity, int max_rows, const void* residual, const void* gamma,
                             void* stream_out, void* normed, int rows, int dim, float eps, int* epoch_dev, int* arrive,
                             long long limit_cycles, int* status, cudaStream_t stream) {
  MB_REQUIRE(world >= 1 && world <= MAX_PEERS, "tp_sum_residual_rmsnorm: world size out of range");
  MB_REQUIRE(dim % 8 == 0 && dim <= SRN_THREADS * 8 * SRN_MAX_VEC, "tp_sum_residual_rmsnorm: unsupported row width");
  MB_REQUIRE(slot_stride % 8 == 0 && slot_stride >= (long long)rows * dim,
             "tp_sum_residual_rmsnorm: slot stride must hold the rows and be a multiple of 8");
  MB_REQUIRE(rows <= max_rows && (parity == 0 || parity == 1), "tp_sum_residual_rmsnorm: rows exceed the flag array");
  MB_REQUIRE(epoch_dev != nullptr && arrive != nullptr, "tp_sum_residual_rmsnorm: epoch and arrival counters are required");
  if (rows == 0) return;
  tp_sum_residual_rmsnorm_kernel<<<rows, SRN_THREADS, 0, stream>>>(
      acc, staging, flags, rank, world, slot_stride, (long long)parity * world * max_rows, max_rows,
      (const __nv_bfloat16*)residual, (const __nv_bfloat16*)gamma, (__nv_bfloat16*)stream_out, (__nv_bfloat16*)normed,
      dim, eps, epoch_dev, arrive, limit_cycles, status);
  count_launch();
  check_launch();
}

void qkv_rope_append(float* acc, const int* pos, const int* seq_ids, const int* block_table, void* q_out,
                     void* k_cache, void* v_cache, int tokens, int heads, int kv_heads, int head_dim, int page_size,
                     int max_pages, float theta, cudaStream_t stream, float* k_scale, float* v_scale) {
  MB_REQUIRE(head_dim % 16 == 0, "qkv_rope_append: head_dim must be a multiple of 16");
  const bool int8 = k_scale != nullptr;
  MB_REQUIRE(int8 == (v_scale != nullptr), "qkv_rope_append: int8 pages need both scale arrays");
  MB_REQUIRE(!int8 || head_dim == 64 || head_dim == 128 || head_dim == 256,
             "qkv_rope_append: int8 pages need head_dim / 16 lanes per head to be a power of two up to 16");
  if (tokens == 0) return;
  const long long work = (long long)tokens * (heads + 2 * kv_heads) * (head_dim / 16);
  qkv_rope_append_kernel<<<(unsigned)ceil_div(work, 128), 128, 0, stream>>>(
      acc, pos, seq_ids, block_table, (__nv_bfloat16*)q_out, int8 ? nullptr : (__nv_bfloat16*)k_cache,
      int8 ? nullptr : (__nv_bfloat16*)v_cache, int8 ? (signed char*)k_cache : nullptr,
      int8 ? (signed char*)v_cache : nullptr, k_scale, v_scale, tokens, heads, kv_heads, head_dim, page_size, max_pages,
      theta > 0.f ? log2f(theta) : 0.f);
  count_launch();
  check_launch();
}

void finalize_gate(float* acc, void* out, long long rows, int ffn, int kind, cudaStream_t stream) {
  MB_REQUIRE(ffn % 8 == 0, "finalize_gate: ffn must be a multiple of 8");
  if (rows == 0) return;
  long long g = (rows * (ffn / 8) + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  finalize_gate_kernel<<<(int)g, 256, 0, stream>>>(acc, (__nv_bfloat16*)out, rows, ffn, kind);
  count_launch();
  check_launch();
}

}  // namespace mb
