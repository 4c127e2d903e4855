// bf16 GEMM with paired SMs: tcgen05.mma.cta_group::2 computes a 256x256 output tile on a
// cluster of two CTAs. Each CTA loads only its own 128 rows of A and its own 128 columns of B
// (32 KB per 64-deep k-block instead of 48 KB for the single-CTA 128x256 tile), so six pipeline
// stages fit in shared memory and the L2 -> SM traffic per FLOP drops by a third; the single-CTA
// kernel was limited by the bytes it can keep in flight per SM.
//
// Protocol (leader = CTA rank 0 of the pair):
//   * every CTA's TMA producer loads its A and B halves; both producers complete the transaction
//     count on the LEADER's full barrier (the load carries .cta_group::2 so it may signal the peer);
//   * the leader's MMA thread waits on its full barrier, issues the paired MMAs, then commits to the
//     empty barrier of BOTH CTAs (two plain commits: own address and the peer's cluster address);
//   * accumulators live in each CTA's own TMEM (128 lanes x 256 columns, double buffered); the
//     leader commits "accumulator full" to both CTAs; epilogue warps of both CTAs arrive on the
//     leader's "accumulator empty" barrier.
// No load in this file fans out to several CTAs: every CTA fetches its own tiles.
#include "api.h"
#include "host_util.h"
#include "tc.cuh"

namespace mb {
namespace {

constexpr int T_BM = 256;        // tile rows per cluster (128 per CTA)
constexpr int T_BN = 256;        // tile columns per cluster (each CTA stages 128 of them)
constexpr int T_BK = 64;
constexpr int T_STAGES = 6;
constexpr int T_THREADS = 192;
constexpr int T_GROUP_M = 8;

struct Cfg2 {
  static constexpr int A_BYTES = 128 * T_BK * 2;  // 16 KB
  static constexpr int B_BYTES = 128 * T_BK * 2;  // 16 KB
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = T_STAGES * STAGE_BYTES;
  static constexpr int NUM_BARS = 2 * T_STAGES + 4;
  static constexpr int EPI_STAGE_OFFSET = BAR_OFFSET + 256;       // [4 epilogue warps][32 rows][128 B]
  static constexpr int SMEM_BYTES = EPI_STAGE_OFFSET + 4 * 4096 + 1024;
  static_assert(NUM_BARS * 8 + 16 <= 256, "barrier region");
  static constexpr int TMEM_COLS = 512;  // two 256-column accumulators
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* m, uint32_t leader_bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(leader_bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
      "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

struct Work2 {
  int m0, n0, kb0, kb1;
};
__device__ __forceinline__ Work2 decode2(int w, int tiles_m, int tiles_n, int k_splits, int kblocks) {
  const int tiles = tiles_m * tiles_n;
  const int split = w / tiles;
  const int t = w - split * tiles;
  const int per_group = T_GROUP_M * tiles_n;
  const int g = t / per_group;
  const int first_m = g * T_GROUP_M;
  const int gsz = min(T_GROUP_M, tiles_m - first_m);
  const int r = t - g * per_group;
  const int tm = first_m + r % gsz;
  const int tn = r / gsz;
  const int base = kblocks / k_splits, rem = kblocks % k_splits;
  const int kb0 = split * base + min(split, rem);
  const int kb1 = kb0 + base + (split < rem ? 1 : 0);
  return {tm * T_BM, tn * T_BN, kb0, kb1};
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T_THREADS, 1)
gemm_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 void* __restrict__ Cout, int M, int N, int K, long long ldc, int tiles_m, int tiles_n, int k_splits,
                 int epi, int vec_ok, float alpha, int* status, PeerPtrs scatter, int n_scatter,
                 long long rows_per_rank, long long slot_off) {
  using Cfg = Cfg2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFFSET);
  uint64_t* empty = full + T_STAGES;
  uint64_t* tfull = empty + T_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const bool leader = cta == 0;
  const int kblocks = (K + T_BK - 1) / T_BK;
  const int total = tiles_m * tiles_n * k_splits;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T_STAGES; ++s) {
      mbar_init(&full[s], 1);   // leader: its own arrive.expect_tx (bytes of both CTAs)
      mbar_init(&empty[s], 1);  // one commit from the leader's MMA thread
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 8);   // leader: four epilogue warps of each CTA
    mbar_init(&tempty[1], 8);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr)),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = cluster_id; w < total && ok; w += n_clusters) {
        const Work2 wi = decode2(w, tiles_m, tiles_n, k_splits, kblocks);
        const int my_m = wi.m0 + (int)cta * 128, my_n = wi.n0 + (int)cta * 128;
        for (int kb = wi.kb0; kb < wi.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, status, 51)) { ok = false; break; }
          const uint32_t lbar = map_to_cta(smem_u32(&full[stage]), 0);
          if (leader) mbar_arrive_expect_tx(&full[stage], 2 * Cfg::STAGE_BYTES);
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          if (!A_MN) {
            tma_load_2d_pair(sa, &tma_a, lbar, kb * T_BK, my_m);
          } else {
            tma_load_2d_pair(sa, &tma_a, lbar, my_m, kb * T_BK);
            tma_load_2d_pair(sa + 8192, &tma_a, lbar, my_m + 64, kb * T_BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tma_b, lbar, kb * T_BK, my_n);
          } else {
            tma_load_2d_pair(sb, &tma_b, lbar, my_n, kb * T_BK);
            tma_load_2d_pair(sb + 8192, &tma_b, lbar, my_n + 64, kb * T_BK);
          }
          if (++stage == T_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && leader) {
      constexpr uint32_t IDESC = umma_idesc_bf16(T_BM, T_BN, A_MN, B_MN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int w = cluster_id; w < total && ok; w += n_clusters) {
        const Work2 wi = decode2(w, tiles_m, tiles_n, k_splits, kblocks);
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, status, 52)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * T_BN;
        for (int kb = wi.kb0; kb < wi.kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, status, 53)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < T_BK / 16; ++k) {
            const uint64_t ad = A_MN ? umma_desc_sw128(a_addr + k * 2048, 8192, 1024)
                                     : umma_desc_sw128(a_addr + k * 32, 0, 1024);
            const uint64_t bd = B_MN ? umma_desc_sw128(b_addr + k * 2048, 8192, 1024)
                                     : umma_desc_sw128(b_addr + k * 32, 0, 1024);
            umma_f16_pair(d_tmem, ad, bd, IDESC, (kb > wi.kb0 || k > 0) ? 1u : 0u);
          }
          const uint32_t e_local = smem_u32(&empty[stage]);
          umma_commit_pair(map_to_cta(e_local, 0));
          umma_commit_pair(map_to_cta(e_local, 1));
          if (++stage == T_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        const uint32_t f_local = smem_u32(&tfull[acc]);
        umma_commit_pair(map_to_cta(f_local, 0));
        umma_commit_pair(map_to_cta(f_local, 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int w = cluster_id; w < total; w += n_clusters) {
      const Work2 wi = decode2(w, tiles_m, tiles_n, k_splits, kblocks);
      bool ok = mbar_wait(&tfull[acc], acc_phase, abort_flag, status, 54);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = wi.m0 + (int)cta * 128 + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * T_BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < T_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = wi.n0 + c * 32;
        if (n_scatter > 0) {
          // Fused reduce-scatter (bf16): the rows go to the rank that owns them, into the slot of
          // the sending rank. A thread holds one row; stored from registers, every warp store would
          // be 32 separate 16-byte peer writes. The warp therefore transposes 32 rows x 64 columns
          // through shared memory and writes full 128-byte lines over NVLink.
          uint8_t* stg = smem + Cfg::EPI_STAGE_OFFSET + q * 4096;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 0]), alpha * __uint_as_float(r[8 * j + 1]));
            v.y = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 2]), alpha * __uint_as_float(r[8 * j + 3]));
            v.z = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 4]), alpha * __uint_as_float(r[8 * j + 5]));
            v.w = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 6]), alpha * __uint_as_float(r[8 * j + 7]));
            const int piece = (c & 1) * 4 + j;
            *reinterpret_cast<uint4*>(stg + lane * 128 + ((piece ^ (lane & 7)) << 4)) = v;
          }
          if (c & 1) {
            __syncwarp();
            const int col0 = wi.n0 + (c - 1) * 32;
            const int row0 = wi.m0 + (int)cta * 128 + q * 32;
            if (col0 < N && row0 < M) {
              const long long owner = row0 / rows_per_rank;   // 256-row tiles never straddle two owners
              __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(scatter.p[owner]) + slot_off +
                                    (row0 - owner * rows_per_rank) * ldc + col0;
#pragma unroll
              for (int it = 0; it < 8; ++it) {
                const int rr = it * 4 + (lane >> 3), piece = lane & 7;
                if (row0 + rr < M)
                  *reinterpret_cast<uint4*>(base + (long long)rr * ldc + piece * 8) =
                      *reinterpret_cast<const uint4*>(stg + rr * 128 + ((piece ^ (rr & 7)) << 4));
              }
            }
            __syncwarp();
          }
          continue;
        }
        if (row < M && col < N) {
          const int ncols = min(32, N - col);
          if (epi == EPI_BF16) {
            __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(Cout) + (long long)row * ldc + col;
            if (ncols == 32 && vec_ok) {
              uint4* p4 = reinterpret_cast<uint4*>(p);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 0]), alpha * __uint_as_float(r[8 * j + 1]));
                v.y = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 2]), alpha * __uint_as_float(r[8 * j + 3]));
                v.z = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 4]), alpha * __uint_as_float(r[8 * j + 5]));
                v.w = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 6]), alpha * __uint_as_float(r[8 * j + 7]));
                p4[j] = v;
              }
            } else {
              for (int j = 0; j < ncols; ++j) p[j] = __float2bfloat16(alpha * __uint_as_float(r[j]));
            }
          } else {
            float* p = reinterpret_cast<float*>(Cout) + (long long)row * ldc + col;
            if (ncols == 32 && vec_ok) {
              float4* p4 = reinterpret_cast<float4*>(p);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(alpha * __uint_as_float(r[4 * j]), alpha * __uint_as_float(r[4 * j + 1]),
                                       alpha * __uint_as_float(r[4 * j + 2]), alpha * __uint_as_float(r[4 * j + 3]));
                if (epi == EPI_F32) {
                  p4[j] = v;
                } else if (epi == EPI_F32_ACC) {
                  float4 o = p4[j];
                  p4[j] = make_float4(o.x + v.x, o.y + v.y, o.z + v.z, o.w + v.w);
                } else {
                  atomicAdd(p4 + j, v);
                }
              }
            } else {
              for (int j = 0; j < ncols; ++j) {
                const float v = alpha * __uint_as_float(r[j]);
                if (epi == EPI_F32) p[j] = v;
                else if (epi == EPI_F32_ACC) p[j] += v;
                else atomicAdd(p + j, v);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 10000000LL) {}
    __syncthreads();
  }
  tc_fence_before();
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while the peer may still touch it
  tc_fence_after();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
}

template <bool A_MN, bool B_MN>
void launch2(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc, int k_splits,
             int epi, int vec_ok, float alpha, int* status, cudaStream_t stream, const PeerPtrs& scatter,
             int n_scatter, long long rows_per_rank, long long slot_off) {
  auto kern = gemm_2cta_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    MB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg2::SMEM_BYTES));
    configured = true;
  }
  const int tiles_m = (M + T_BM - 1) / T_BM, tiles_n = (N + T_BN - 1) / T_BN;
  const int total = tiles_m * tiles_n * k_splits;
  int clusters = sm_count() / 2;
  if (total < clusters) clusters = total;
  kern<<<clusters * 2, T_THREADS, Cfg2::SMEM_BYTES, stream>>>(ta, tb, C, M, N, K, ldc, tiles_m, tiles_n, k_splits, epi,
                                                              vec_ok, alpha, status, scatter, n_scatter, rows_per_rank,
                                                              slot_off);
  count_launch();
  check_launch();
}

}  // namespace

// Relative cost estimate (in 256-wide tile-waves) of the paired kernel; used by the dispatcher.
double gemm_2cta_waves(int M, int N, int sms) {
  const long long tiles = (long long)((M + T_BM - 1) / T_BM) * ((N + T_BN - 1) / T_BN);
  const int clusters = sms / 2;
  return (double)((tiles + clusters - 1) / clusters);
}

void gemm_bf16_2cta(const void* A, long long lda, bool a_mn, const void* B, long long ldb, bool b_mn, void* C,
                    long long ldc, int M, int N, int K, int epi, float alpha, int* status, cudaStream_t stream) {
  gemm_bf16_2cta_scatter(A, lda, a_mn, B, ldb, b_mn, C, ldc, M, N, K, epi, alpha, status, stream, nullptr, 0, 0, 0);
}

void gemm_bf16_2cta_scatter(const void* A, long long lda, bool a_mn, const void* B, long long ldb, bool b_mn, void* C,
                            long long ldc, int M, int N, int K, int epi, float alpha, int* status,
                            cudaStream_t stream, const PeerPtrs* scatter, int n_scatter, long long rows_per_rank,
                            long long slot_off) {
  MB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem");
  PeerPtrs sc{};
  if (n_scatter > 0) {
    MB_REQUIRE(scatter != nullptr && epi == EPI_BF16, "gemm: scattered output needs peers and the bf16 epilogue");
    MB_REQUIRE(rows_per_rank > 0 && (long long)n_scatter * rows_per_rank >= M, "gemm: scattered rows exceed the peers");
    MB_REQUIRE((slot_off * 2) % 16 == 0, "gemm: slot offset must keep 16-byte alignment");
    MB_REQUIRE(N % 64 == 0 && ldc % 8 == 0 && rows_per_rank % 256 == 0,
               "gemm: scattered output needs N % 64 == 0, ldc % 8 == 0 and 256-row ownership blocks");
    sc = *scatter;
  }
  MB_REQUIRE(!(a_mn && !b_mn), "gemm: MN-major A with K-major B is not instantiated");
  MB_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "gemm: operand row strides must be multiples of 8 elements");
  const int esz = (epi == EPI_BF16) ? 2 : 4;
  const int vec_ok = ((ldc * esz) % 16 == 0 && (n_scatter > 0 || (reinterpret_cast<uintptr_t>(C) & 15) == 0)) ? 1 : 0;
  const int kblocks = (K + T_BK - 1) / T_BK;
  int k_splits = 1;
  if (epi == EPI_F32_ATOMIC) {
    const int clusters = sm_count() / 2;
    const long long tiles = (long long)((M + T_BM - 1) / T_BM) * ((N + T_BN - 1) / T_BN);
    double best = 1e30;
    for (int s = 1; s <= 8; ++s) {
      if (kblocks / s < 8 && s > 1) break;
      const double waves = (double)((tiles * s + clusters - 1) / clusters) / s;
      if (waves < best * 0.97) { best = waves; k_splits = s; }
    }
  }
  uint64_t adims[2], astr[1], bdims[2], bstr[1];
  uint32_t abox[2], bbox[2];
  if (!a_mn) { adims[0] = K; adims[1] = M; abox[0] = T_BK; abox[1] = 128; }
  else       { adims[0] = M; adims[1] = K; abox[0] = 64; abox[1] = T_BK; }
  astr[0] = (uint64_t)lda * 2;
  if (!b_mn) { bdims[0] = K; bdims[1] = N; bbox[0] = T_BK; bbox[1] = 128; }
  else       { bdims[0] = N; bdims[1] = K; bbox[0] = 64; bbox[1] = T_BK; }
  bstr[0] = (uint64_t)ldb * 2;
  const CUtensorMap ta = make_tensor_map(A, TmaDType::BF16, 2, adims, astr, abox, true);
  const CUtensorMap tb = make_tensor_map(B, TmaDType::BF16, 2, bdims, bstr, bbox, true);
  if (!a_mn && !b_mn)
    launch2<false, false>(ta, tb, C, M, N, K, ldc, k_splits, epi, vec_ok, alpha, status, stream, sc, n_scatter,
                          rows_per_rank, slot_off);
  else if (!a_mn && b_mn)
    launch2<false, true>(ta, tb, C, M, N, K, ldc, k_splits, epi, vec_ok, alpha, status, stream, sc, n_scatter,
                         rows_per_rank, slot_off);
  else
    launch2<true, true>(ta, tb, C, M, N, K, ldc, k_splits, epi, vec_ok, alpha, status, stream, sc, n_scatter,
                        rows_per_rank, slot_off);
}

}  // namespace mb
