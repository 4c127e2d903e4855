// Data-parallel collectives fused with compute, over NVLink peer memory.
//
// Every rank maps the other ranks' buffers (symmetric memory) and the kernels issue plain
// peer loads and stores; nothing here goes through a library collective.
//
//   symm_barrier        flag barrier between ranks (st.release.sys / ld.acquire.sys on peer
//                       memory), optionally carrying one float per rank (the partial gradient
//                       norm). The wait is bounded and reports a timeout in the status word.
//   zero_reduce_scatter rank r sums slice r of every rank's fp32 gradient buffer in fixed rank
//                       order (deterministic), keeps the result locally and accumulates its
//                       sum of squares: reduce-scatter + global-norm partial in one pass.
//   zero_adamw_ste_allgather
//                       on the local shard: clip coefficient from the gathered norm partials,
//                       AdamW on the fp32 master, STE fake-quantisation of the updated weights
//                       (OIL8 / OIL4 nearest centroid in a sorted codebook, I2_S absmean ternary,
//                       or plain cast) and the bf16 result stored straight into every rank's
//                       compute buffer: optimizer + quantiser + all-gather in one pass.
//
// The reference's counterpart is DDPWrapper::sync_gradients (src/distributed.cpp:102-138): one
// blocking all-reduce per parameter through a mutex-protected host buffer, followed by a
// separate optimizer loop.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace mb {
namespace {

// Two-shot all-reduce through NVLS: this rank's slice is summed inside the switch (one multicast load
// per 16 bytes) and broadcast to every rank with one multicast store.
__global__ void tp_allreduce_mc_kernel(const __nv_bfloat16* part_mc, __nv_bfloat16* out_mc, long long begin8,
                                       long long end8, const int* abort_word);

const int* g_abort_word[64] = {nullptr};
const int* abort_word_for_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  return g_abort_word[dev];
}

// A kernel that consumes what a barrier guarded reads the status word first: once a bounded wait
// has expired somewhere on this device the data may be incomplete, so the kernel returns without
// writing anything (no poisoned update is applied or broadcast); the host sees the word afterwards.
__device__ __forceinline__ bool aborted(const int* abort_word) {
  return abort_word != nullptr && *reinterpret_cast<const volatile int*>(abort_word) != 0;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Wait statistics of the flag barriers launched on this device: [0] number of barriers, [1] sum and
// [2] maximum of the cycles between this rank's arrival and the last peer's (the slowest of the
// per-peer waits of a launch). Read and cleared by comm_barrier_wait_stats.
__device__ unsigned long long g_barrier_wait[3];

// One thread per peer. flags[r] on every rank is an int array of `world` slots; slot s of rank r
// holds the last epoch that rank s announced to rank r.
__global__ void symm_barrier_kernel(PeerPtrs flags, PeerPtrs slots, const float* send_val, int rank, int world,
                                    int epoch, int* epoch_ptr, long long limit_cycles, int* status) {
  const int p = threadIdx.x;
  // With epoch_ptr the epoch lives on the device and advances by one per launch, so the same
  // launch can be replayed from a CUDA graph.
  if (epoch_ptr) epoch = *epoch_ptr + 1;
  __syncwarp();
  if (p == 0 && epoch_ptr) *epoch_ptr = epoch;
  long long waited = 0;
  if (p < world) {
    __threadfence_system();
    if (send_val) reinterpret_cast<float*>(slots.p[p])[rank] = *send_val;
    st_release_sys(reinterpret_cast<int*>(flags.p[p]) + rank, epoch);
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + p;
    const long long t0 = clock64();
    while (ld_acquire_sys(mine) < epoch) {
      if (clock64() - t0 > limit_cycles) {
        if (status) atomicCAS(status, 0, 1 | (40 << 16));
        break;
      }
    }
    waited = clock64() - t0;
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) waited = max(waited, __shfl_xor_sync(0xffffffffu, waited, m));
  if (p == 0) {
    atomicAdd(&g_barrier_wait[0], 1ull);
    atomicAdd(&g_barrier_wait[1], (unsigned long long)waited);
    atomicMax(&g_barrier_wait[2], (unsigned long long)waited);
  }
}

// NVLS: one load from the multicast address of a symmetric buffer returns the sum over every rank's
// copy, added inside the NVSwitch (fp32), so a rank receives one value per element instead of one per peer.
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// NVLS: one store to the multicast address writes the 16 bytes into every rank's copy.
__device__ __forceinline__ void multimem_st_b128(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}
// Sum of bf16 pairs over every rank's copy, accumulated in fp32 inside the switch.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

__global__ void zero_reduce_scatter_kernel(PeerPtrs grads, float* __restrict__ out, long long shard_off, long long n,
                                           int world, float* __restrict__ sumsq, const int* abort_word,
                                           const float* mc, float* __restrict__ block_partials) {
  __shared__ float scratch[32];
  if (aborted(abort_word)) return;
  float ss = 0.f;
  const long long n4 = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (mc != nullptr) {
      acc = multimem_ld_reduce_f32x4(mc + shard_off + 4 * i);
    } else {
#pragma unroll 8
      for (int r = 0; r < world; ++r) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + shard_off) + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    reinterpret_cast<float4*>(out)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0 && sumsq) {
    if (block_partials == nullptr) {
      atomicAdd(sumsq, ss);                      // order of the additions varies from launch to launch
    } else {
      // bit-reproducible norm: every block leaves its partial, the block that finishes last adds them
      // in index order (the ticket lives behind the partials and is reset for the next launch)
      unsigned* ticket = reinterpret_cast<unsigned*>(block_partials + gridDim.x);
      block_partials[blockIdx.x] = ss;
      __threadfence();
      if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
        __threadfence();
        float tot = 0.f;
        for (unsigned b = 0; b < gridDim.x; ++b) tot += reinterpret_cast<volatile float*>(block_partials)[b];
        atomicAdd(sumsq, tot);
        *ticket = 0u;
      }
    }
  }
}

template <int CB>
__device__ __forceinline__ int nearest_sorted_dev(const float* cb, float w) {
  int lo = 0;
#pragma unroll
  for (int step = CB >> 1; step > 0; step >>= 1)
    if (cb[lo + step - 1] < w) lo += step;
  if (lo < CB && cb[lo] < w) ++lo;
  int j;
  if (lo == 0) j = 0;
  else if (lo >= CB) j = CB - 1;
  else j = (w - cb[lo - 1] <= cb[lo] - w) ? lo - 1 : lo;
  while (j > 0 && cb[j - 1] == cb[j]) --j;
  return j;
}

// One warp per 256-element segment of the local shard.
__global__ void zero_adamw_ste_allgather_kernel(ZeroFusedArgs a, const int* abort_word) {
  if (aborted(abort_word)) return;
  extern __shared__ float cb_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  float* cb = cb_smem + warp * 256;
  float total = 0.f;
  for (int r = 0; r < a.world; ++r) total += a.norm_partials[r];
  const float norm = sqrtf(total);
  const float clip = (a.max_norm > 0.f && norm > a.max_norm) ? a.max_norm / (norm + 1e-8f) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0 && a.grad_norm_out) *a.grad_norm_out = norm;
  const float gs = a.opt.grad_scale * clip;
  const long long nseg = a.n >> 8;
  int cached = -1;
  for (long long seg = (long long)blockIdx.x * wpb + warp; seg < nseg; seg += (long long)gridDim.x * wpb) {
    const long long base = seg * 256 + lane * 8;
    float p[8], m[8], v[8], g[8];
    *reinterpret_cast<float4*>(p) = *reinterpret_cast<const float4*>(a.p + base);
    *reinterpret_cast<float4*>(p + 4) = *reinterpret_cast<const float4*>(a.p + base + 4);
    *reinterpret_cast<float4*>(m) = *reinterpret_cast<const float4*>(a.m + base);
    *reinterpret_cast<float4*>(m + 4) = *reinterpret_cast<const float4*>(a.m + base + 4);
    *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(a.v + base);
    *reinterpret_cast<float4*>(v + 4) = *reinterpret_cast<const float4*>(a.v + base + 4);
    *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(a.g + base);
    *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(a.g + base + 4);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = g[k] * gs;
      p[k] -= a.opt.lr * a.opt.weight_decay * p[k];
      m[k] = a.opt.beta1 * m[k] + (1.f - a.opt.beta1) * gk;
      v[k] = a.opt.beta2 * v[k] + (1.f - a.opt.beta2) * gk * gk;
      p[k] -= a.opt.lr * (m[k] / a.opt.bc1) / (sqrtf(v[k] / a.opt.bc2) + a.opt.eps);
    }
    *reinterpret_cast<float4*>(a.p + base) = *reinterpret_cast<float4*>(p);
    *reinterpret_cast<float4*>(a.p + base + 4) = *reinterpret_cast<float4*>(p + 4);
    *reinterpret_cast<float4*>(a.m + base) = *reinterpret_cast<float4*>(m);
    *reinterpret_cast<float4*>(a.m + base + 4) = *reinterpret_cast<float4*>(m + 4);
    *reinterpret_cast<float4*>(a.v + base) = *reinterpret_cast<float4*>(v);
    *reinterpret_cast<float4*>(a.v + base + 4) = *reinterpret_cast<float4*>(v + 4);

    const long long gseg = (a.shard_off >> 8) + seg;  // segment index in the full flat buffer
    const int fmt = a.seg_fmt ? a.seg_fmt[gseg] : ZERO_FMT_CAST;
    float q[8];
    if (fmt == ZERO_FMT_OIL8 || fmt == ZERO_FMT_OIL4) {
      const int cbi = a.seg_cb[gseg];
      const int key = cbi * 2 + (fmt == ZERO_FMT_OIL4 ? 1 : 0);
      if (key != cached) {
        __syncwarp();
        if (fmt == ZERO_FMT_OIL8) {
          for (int i = lane; i < 256; i += 32) cb[i] = a.codebooks8[(long long)cbi * 256 + i];
        } else if (lane < 16) {
          cb[lane] = a.codebooks4[(long long)cbi * 16 + lane];
        }
        cached = key;
        __syncwarp();
      }
#pragma unroll
      for (int k = 0; k < 8; ++k)
        q[k] = (fmt == ZERO_FMT_OIL8) ? cb[nearest_sorted_dev<256>(cb, p[k])] : cb[nearest_sorted_dev<16>(cb, p[k])];
    } else if (fmt == ZERO_FMT_I2S) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) s += fabsf(p[k]);
      s = warp_sum(s);
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(p[k]));
      amax = warp_max(amax);
      int exact = 1;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (p[k] != 0.f && fabsf(p[k]) != amax) exact = 0;
      exact = __all_sync(0xffffffffu, exact);
      const float scale = exact ? amax : s * (1.f / 256.f);  // already-ternary blocks keep their scale
      const float inv = scale > 0.f ? 1.f / scale : 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) q[k] = fminf(1.f, fmaxf(-1.f, rintf(p[k] * inv))) * scale;
    } else if (fmt == ZERO_FMT_BINARY) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) s += fabsf(p[k]);
      s = warp_sum(s) * (1.f / 256.f);           // mean |w| of the 256-weight block
#pragma unroll
      for (int k = 0; k < 8; ++k) q[k] = p[k] > 0.f ? s : -s;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) q[k] = p[k];
    }
    const bf16x8 packed = pack8(q);
    const long long gelem = a.shard_off + base;
    if (a.compute_mc != nullptr) {
      // one multicast store reaches every rank's compute buffer (this rank's own included)
      multimem_st_b128(reinterpret_cast<__nv_bfloat16*>(a.compute_mc) + gelem, *reinterpret_cast<const uint4*>(&packed));
    } else {
      for (int r = 0; r < a.world; ++r) {
        const int dst = (a.rank + r) % a.world;  // start with the local copy, then fan out
        stg8(a.compute.p[dst], gelem, packed);
      }
    }
  }
}

}  // namespace

void symm_barrier(const PeerPtrs& flags, const PeerPtrs& slots, const float* send_val, int rank, int world, int epoch,
                  int* epoch_ptr, long long limit_cycles, int* status, cudaStream_t stream) {
  MB_REQUIRE(world >= 1 && world <= MAX_PEERS, "symm_barrier: world size out of range");
  symm_barrier_kernel<<<1, 32, 0, stream>>>(flags, slots, send_val, rank, world, epoch, epoch_ptr, limit_cycles, status);
  count_launch();
  check_launch();
}

void comm_barrier_wait_stats(unsigned long long out[3], bool reset) {
  MB_CUDA_CHECK(cudaMemcpyFromSymbol(out, g_barrier_wait, 3 * sizeof(unsigned long long)));
  if (reset) {
    const unsigned long long zero[3] = {0ull, 0ull, 0ull};
    MB_CUDA_CHECK(cudaMemcpyToSymbol(g_barrier_wait, zero, sizeof(zero)));
  }
}

void zero_reduce_scatter(const PeerPtrs& grads, float* out, long long shard_off, long long n, int world, float* sumsq,
                         cudaStream_t stream, const float* grads_multicast, int max_blocks, float* block_partials,
                         long long n_block_partials) {
  MB_REQUIRE(n % 4 == 0 && shard_off % 4 == 0, "zero_reduce_scatter: shard must be a multiple of 4 elements");
  if (n == 0) return;
  long long grid = (n / 4 + 255) / 256;
  long long cap = (long long)sm_count() * 8;
  if (max_blocks > 0 && max_blocks < cap) cap = max_blocks;   // a small grid when it runs beside the backward pass
  if (grid > cap) grid = cap;
  if (block_partials != nullptr && grid + 1 > n_block_partials) grid = n_block_partials - 1;
  MB_REQUIRE(grid >= 1, "zero_reduce_scatter: scratch for the block partials is too small");
  zero_reduce_scatter_kernel<<<(int)grid, 256, 0, stream>>>(grads, out, shard_off, n, world, sumsq,
                                                            abort_word_for_current_device(), grads_multicast,
                                                            block_partials);
  count_launch();
  check_launch();
}

void zero_adamw_ste_allgather(const ZeroFusedArgs& a, cudaStream_t stream) {
  MB_REQUIRE(a.n % 256 == 0 && a.shard_off % 256 == 0, "zero_adamw_ste_allgather: shard must be 256-aligned");
  if (a.n == 0) return;
  const int threads = 256, wpb = threads / 32;
  long long grid = ((a.n >> 8) + wpb - 1) / wpb;
  const long long cap = (long long)sm_count() * 8;
  if (grid > cap) grid = cap;
  zero_adamw_ste_allgather_kernel<<<(int)grid, threads, wpb * 256 * sizeof(float), stream>>>(
      a, abort_word_for_current_device());
  count_launch();
  check_launch();
}

namespace {

__global__ void peer_add_kernel(const float* __restrict__ part, PeerPtrs dst, int n_peers, long long n4) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(part)[i];
    for (int p = 0; p < n_peers; ++p) atomicAdd(reinterpret_cast<float4*>(dst.p[p]) + i, v);
  }
}

// dst_r[b, rank*cols + j] = src[b, j] for every rank r (cols is a multiple of 8).
__global__ void peer_gather_cols_kernel(const __nv_bfloat16* __restrict__ src, PeerPtrs dst, int n_peers, int rank,
                                        long long rows, int cols) {
  const int per_row = cols >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c = (int)(i % per_row) * 8;
    const bf16x8 v = ldg8(src, r * cols + c);
    const long long off = r * ((long long)cols * n_peers) + (long long)rank * cols + c;
    for (int p = 0; p < n_peers; ++p) stg8(dst.p[(rank + p) % n_peers], off, v);
  }
}


// ---- tensor-parallel all-reduce of bf16 activations over peer memory
//
// One-shot (few tokens, latency bound): every rank stores its partial into slot `rank` of every
// peer's staging buffer (tp_push_kernel, or the dequant-GEMM epilogue directly), one barrier, then
// every rank sums the W slots of its own staging buffer (tp_reduce_slots_kernel). One NVLink hop.
//
// Two-shot (prefill-sized, bandwidth bound): after a barrier every rank pulls ITS slice of the
// elements from all W partial buffers with peer loads, sums in fp32 and stores the bf16 result into
// every peer's output buffer (tp_allreduce_pull_kernel); a second barrier publishes the result.
// Each element crosses NVLink once in each direction per rank pair, the minimum for an all-reduce.

// acc fp32 [n] (zeroed afterwards) -> bf16 -> dst_p[slot_off + i] for every peer p.
__global__ void tp_push_kernel(float* __restrict__ acc, PeerPtrs dst, int n_peers, int rank, long long slot_off,
                               long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float4* a = reinterpret_cast<float4*>(acc) + 2 * i;
    const float4 lo = a[0], hi = a[1];
    a[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    a[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    const float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    const bf16x8 v = pack8(f);
    for (int p = 0; p < n_peers; ++p) stg8(dst.p[(rank + p) % n_peers], slot_off + i * 8, v);
  }
}

// Loads of memory that another GPU wrote (or owns) bypass L1: a line cached by an earlier round
// would otherwise be served stale. L2 is the coherence point for NVLink traffic.
__device__ __forceinline__ bf16x8 ld_l2_8(const void* base, long long elem_index) {
  const uint4 v = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem_index));
  return *reinterpret_cast<const bf16x8*>(&v);
}

// out[i] = bf16(sum_s staging[s * slot_stride + i] (+ residual[i]))
__global__ void tp_reduce_slots_kernel(const __nv_bfloat16* __restrict__ staging, int slots, long long slot_stride,
                                       const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out,
                                       long long n8, const int* abort_word) {
  if (aborted(abort_word)) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bf16x8 v[MAX_PEERS];
#pragma unroll
    for (int s = 0; s < MAX_PEERS; ++s)
      if (s < slots) v[s] = ld_l2_8(staging, s * slot_stride + i * 8);   // all loads in flight before the adds
#pragma unroll
    for (int s = 0; s < MAX_PEERS; ++s)
      if (s < slots) {
        float f[8];
        unpack8(v[s], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    if (residual) {
      float f[8];
      unpack8(ldg8(residual, i * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    stg8(out, i * 8, pack8(acc));
  }
}

// out_p[out_off + i] = bf16(sum_s staging[s * slot_stride + i]) for every peer p.
__global__ void tp_reduce_slots_bcast_kernel(const __nv_bfloat16* __restrict__ staging, int slots, long long slot_stride,
                                             PeerPtrs out, int n_peers, int rank, long long out_off, long long n8,
                                             const int* abort_word) {
  if (aborted(abort_word)) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bf16x8 v[MAX_PEERS];
#pragma unroll
    for (int s = 0; s < MAX_PEERS; ++s)
      if (s < slots) v[s] = ld_l2_8(staging, s * slot_stride + i * 8);
#pragma unroll
    for (int s = 0; s < MAX_PEERS; ++s)
      if (s < slots) {
        float f[8];
        unpack8(v[s], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    const bf16x8 r = pack8(acc);
    for (int p = 0; p < n_peers; ++p) stg8(out.p[(rank + p) % n_peers], out_off + i * 8, r);
  }
}

// Elements [begin8, end8) (units of 8) are this rank's slice: out_p[i] = bf16(sum_q part_q[i]) for
// every p. Partials are summed in rank order, so the value does not depend on which rank owns it.
// With local_out the sum of the slice is stored there only (element 0 = first element of the slice): a
// reduce-scatter by peer loads.
__global__ void tp_allreduce_pull_kernel(PeerPtrs part, PeerPtrs out, int n_peers, int rank, long long begin8,
                                         long long end8, const int* abort_word, __nv_bfloat16* __restrict__ local_out) {
  if (aborted(abort_word)) return;
  for (long long i = begin8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < end8;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bf16x8 v[MAX_PEERS];
#pragma unroll
    for (int q = 0; q < MAX_PEERS; ++q)
      if (q < n_peers) v[q] = ld_l2_8(part.p[q], i * 8);
#pragma unroll
    for (int q = 0; q < MAX_PEERS; ++q)
      if (q < n_peers) {
        float f[8];
        unpack8(v[q], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    const bf16x8 r = pack8(acc);
    if (local_out != nullptr) {
      stg8(local_out, (i - begin8) * 8, r);
    } else {
      for (int p = 0; p < n_peers; ++p) stg8(out.p[(rank + p) % n_peers], i * 8, r);
    }
  }
}

__global__ void tp_allreduce_mc_kernel(const __nv_bfloat16* part_mc, __nv_bfloat16* out_mc, long long begin8,
                                       long long end8, const int* abort_word) {
  if (aborted(abort_word)) return;
  for (long long i = begin8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < end8;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = multimem_ld_reduce_bf16x8(part_mc + i * 8);
    multimem_st_b128(out_mc + i * 8, v);
  }
}

}  // namespace

void tp_allreduce_multimem(const void* part_mc, void* out_mc, int n_peers, int rank, long long n, cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0 && n_peers >= 1 && part_mc != nullptr && out_mc != nullptr, "tp_allreduce_multimem: bad arguments");
  const long long n8 = n / 8;
  const long long per = (n8 + n_peers - 1) / n_peers;
  const long long begin = per * rank, end = begin + per < n8 ? begin + per : n8;
  if (begin >= end) return;
  long long g = (end - begin + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  tp_allreduce_mc_kernel<<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)part_mc, (__nv_bfloat16*)out_mc, begin, end,
                                                     abort_word_for_current_device());
  count_launch();
  check_launch();
}

void comm_set_abort_word(const int* status) {
  int dev = 0;
  MB_CUDA_CHECK(cudaGetDevice(&dev));
  MB_REQUIRE(dev >= 0 && dev < 64, "comm_set_abort_word: device index out of range");
  g_abort_word[dev] = status;
}

void peer_add_f32(const float* part, const PeerPtrs& dst, int n_peers, long long n, cudaStream_t stream) {
  MB_REQUIRE(n % 4 == 0, "peer_add_f32: element count must be a multiple of 4");
  if (n == 0) return;
  long long g = (n / 4 + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  peer_add_kernel<<<(int)g, 256, 0, stream>>>(part, dst, n_peers, n / 4);
  count_launch();
  check_launch();
}

void peer_gather_cols(const void* src, const PeerPtrs& dst, int n_peers, int rank, long long rows, int cols,
                      cudaStream_t stream) {
  MB_REQUIRE(cols % 8 == 0, "peer_gather_cols: column count must be a multiple of 8");
  if (rows == 0) return;
  long long g = (rows * (cols / 8) + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  peer_gather_cols_kernel<<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)src, dst, n_peers, rank, rows, cols);
  count_launch();
  check_launch();
}

void tp_push(float* acc, const PeerPtrs& dst, int n_peers, int rank, long long slot_off, long long n,
             cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0 && slot_off % 8 == 0, "tp_push: counts and offsets must be multiples of 8");
  if (n == 0) return;
  long long g = (n / 8 + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  tp_push_kernel<<<(int)g, 256, 0, stream>>>(acc, dst, n_peers, rank, slot_off, n / 8);
  count_launch();
  check_launch();
}

void tp_reduce_slots(const void* staging, int slots, long long slot_stride, const void* residual, void* out,
                     long long n, cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0 && slot_stride % 8 == 0, "tp_reduce_slots: counts and strides must be multiples of 8");
  if (n == 0) return;
  long long g = (n / 8 + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  tp_reduce_slots_kernel<<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)staging, slots, slot_stride,
                                                     (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, n / 8,
                                                     abort_word_for_current_device());
  count_launch();
  check_launch();
}

void tp_reduce_slots_bcast(const void* staging, int slots, long long slot_stride, const PeerPtrs& out, int n_peers,
                           int rank, long long out_off, long long n, cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0 && slot_stride % 8 == 0 && out_off % 8 == 0,
             "tp_reduce_slots_bcast: counts, strides and offsets must be multiples of 8");
  if (n == 0) return;
  long long g = (n / 8 + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  tp_reduce_slots_bcast_kernel<<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)staging, slots, slot_stride, out,
                                                           n_peers, rank, out_off, n / 8,
                                                           abort_word_for_current_device());
  count_launch();
  check_launch();
}

void tp_allreduce_pull(const PeerPtrs& part, const PeerPtrs& out, int n_peers, int rank, long long n,
                       cudaStream_t stream) {
  MB_REQUIRE(n % 8 == 0, "tp_allreduce_pull: element count must be a multiple of 8");
  MB_REQUIRE(n_peers >= 1 && n_peers <= MAX_PEERS, "tp_allreduce_pull: bad peer count");
  const long long n8 = n / 8;
  const long long per = (n8 + n_peers - 1) / n_peers;
  const long long begin = per * rank < n8 ? per * rank : n8;
  const long long end = begin + per < n8 ? begin + per : n8;
  if (end <= begin) return;
  long long g = (end - begin + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  tp_allreduce_pull_kernel<<<(int)g, 256, 0, stream>>>(part, out, n_peers, rank, begin, end,
                                                       abort_word_for_current_device(), nullptr);
  count_launch();
  check_launch();
}

void tp_reduce_scatter_pull(const PeerPtrs& part, int n_peers, int rank, long long n, void* out_local, cudaStream_t stream) {
  MB_REQUIRE(n % (8LL * n_peers) == 0, "tp_reduce_scatter_pull: element count must be a multiple of 8 x ranks");
  MB_REQUIRE(n_peers >= 1 && n_peers <= MAX_PEERS, "tp_reduce_scatter_pull: bad peer count");
  const long long per = n / 8 / n_peers;
  if (per == 0) return;
  long long g = (per + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  tp_allreduce_pull_kernel<<<(int)g, 256, 0, stream>>>(part, PeerPtrs{}, n_peers, rank, per * rank, per * (rank + 1),
                                                       abort_word_for_current_device(), (__nv_bfloat16*)out_local);
  count_launch();
  check_launch();
}

}  // namespace mb
