// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM),
// operands staged by TMA into 128-byte-swizzled shared-memory tiles, persistent over
// output tiles with a double-buffered accumulator so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
//   C[M,N] (+)= A * B^T      A: [M,K] (K-major) or stored transposed [K,M] (MN-major)
//                            B: [N,K] (K-major) or stored transposed [K,N] (MN-major)
//
// The three operand layouts cover a linear layer's forward (K/K), input gradient (K/MN)
// and weight gradient (MN/MN) without a transpose pass. This replaces the reference's
// scalar triple loop (src/kernel_i2s.cpp:91-102) and its autograd MatMul backward
// (src/autograd.cpp:94-127).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..5 = epilogue (each reads its own 32-lane quarter of TMEM).
#include "api.h"
#include "host_util.h"
#include "tc.cuh"

namespace mb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 16;  // raster: GROUP_M row-tiles share each column panel in L2

template <int BN, int STAGES>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int SMEM_BYTES = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;
  static constexpr int TMEM_COLS = 2 * BN;
};

struct WorkItem {
  int m0, n0, kb0, kb1;
};

__device__ __forceinline__ WorkItem decode_work(int w, int tiles_m, int tiles_n, int k_splits, int kblocks) {
  const int tiles = tiles_m * tiles_n;
  const int split = w / tiles;
  const int t = w - split * tiles;
  const int per_group = GROUP_M * tiles_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(GROUP_M, tiles_m - first_m);
  const int r = t - g * per_group;
  const int tm = first_m + r % gsz;
  const int tn = r / gsz;
  const int base = kblocks / k_splits, rem = kblocks % k_splits;
  const int kb0 = split * base + min(split, rem);
  const int kb1 = kb0 + base + (split < rem ? 1 : 0);
  return {tm * BM, tn, kb0, kb1};
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               void* __restrict__ Cout, int M, int N, int K, long long ldc, int tiles_m, int tiles_n,
               int k_splits, int epi, int vec_ok, float alpha, int* status) {
  using Cfg = GemmCfg<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (K + BK - 1) / BK;
  const int total = tiles_m * tiles_n * k_splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 4);
    mbar_init(&tempty[1], 4);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const WorkItem wi = decode_work(w, tiles_m, tiles_n, k_splits, kblocks);
        const int n0 = wi.n0 * BN;
        for (int kb = wi.kb0; kb < wi.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, status, 1)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          if (!A_MN) {
            tma_load_2d(sa, &tma_a, &full[stage], kb * BK, wi.m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * 8192, &tma_a, &full[stage], wi.m0 + c * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tma_b, &full[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * 8192, &tma_b, &full[stage], n0 + c * 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const WorkItem wi = decode_work(w, tiles_m, tiles_n, k_splits, kblocks);
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = wi.kb0; kb < wi.kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, status, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = A_MN ? umma_desc_sw128(a_addr + k * 2048, 8192, 1024)
                                     : umma_desc_sw128(a_addr + k * 32, 0, 1024);
            const uint64_t bd = B_MN ? umma_desc_sw128(b_addr + k * 2048, 8192, 1024)
                                     : umma_desc_sw128(b_addr + k * 32, 0, 1024);
            umma_f16(d_tmem, ad, bd, IDESC, (kb > wi.kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x) {
      const WorkItem wi = decode_work(w, tiles_m, tiles_n, k_splits, kblocks);
      const int n0 = wi.n0 * BN;
      bool ok = mbar_wait(&tfull[acc], acc_phase, abort_flag, status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = wi.m0 + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
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
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up: let copies and MMAs in flight land before shared memory and TMEM go away.
    const long long t0 = clock64();
    while (clock64() - t0 < 10000000LL) {}
    __syncthreads();
  }
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
void launch_cfg(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc,
                int k_splits, int epi, int vec_ok, float alpha, int* status, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, STAGES>;
  auto kern = gemm_tc_kernel<BN, STAGES, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    MB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    configured = true;
  }
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int total = tiles_m * tiles_n * k_splits;
  const int grid = total < sm_count() ? total : sm_count();
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, C, M, N, K, ldc, tiles_m, tiles_n, k_splits, epi,
                                                        vec_ok, alpha, status);
  count_launch();
  check_launch();
}

// Relative cost of running `tiles` equal tiles of width bn on `sms` SMs.
inline double wave_cost(long long tiles, int bn, int sms) { return (double)((tiles + sms - 1) / sms) * bn; }

int g_gemm_mode = 0;

}  // namespace

void set_gemm_mode(int mode) { g_gemm_mode = mode; }
int get_gemm_mode() { return g_gemm_mode; }

void gemm_bf16(const void* A, long long lda, bool a_mn, const void* B, long long ldb, bool b_mn, void* C,
               long long ldc, int M, int N, int K, int epi, float alpha, int* status, cudaStream_t stream) {
  MB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem");
  MB_REQUIRE(epi >= EPI_BF16 && epi <= EPI_F32_ATOMIC, "gemm: bad epilogue id");
  MB_REQUIRE(!(a_mn && !b_mn), "gemm: MN-major A with K-major B is not instantiated");
  MB_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "gemm: operand row strides must be multiples of 8 elements");
  const int esz = (epi == EPI_BF16) ? 2 : 4;
  const int vec_ok = ((ldc * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
  const int sms = sm_count();
  const long long tm = (M + BM - 1) / BM;
  const long long t256 = tm * ((N + 255) / 256), t128 = tm * ((N + 127) / 128);
  // A 128-wide tile reads as many shared-memory bytes per MMA as the unit can deliver and
  // measured ~0.72x the throughput of the 256-wide tile, so it only wins on small problems.
  const bool use256 = N > 128 && wave_cost(t256, 256, sms) <= wave_cost(t128, 128, sms) / 0.72;
  const int BN = use256 ? 256 : 128;
  const long long tiles = use256 ? t256 : t128;
  // Paired-SM kernel: one 256x256 tile per SM pair costs the time of one 128x256 tile per SM and
  // streams a third fewer bytes per FLOP, which measured faster whenever its wave count is close.
  if (g_gemm_mode != 1 && M >= 256 && N >= 256) {
    const double c2 = gemm_2cta_waves(M, N, sms) * 256.0;
    const double c1 = use256 ? wave_cost(t256, 256, sms) : wave_cost(t128, 128, sms) / 0.72;
    // Measured on B200 (all three operand layouts, forward / dgrad / wgrad shapes of the 1.3B
    // model): the paired kernel is 8-16 % faster than the single-CTA one whenever its wave count
    // is close, e.g. K/MN 16384x5504x2048 1385 vs 1196 TFLOP/s, MN/MN 6144x2048x16384 1416 vs 1251.
    if (g_gemm_mode == 2 || c2 <= c1 * 1.15) {
      gemm_bf16_2cta(A, lda, a_mn, B, ldb, b_mn, C, ldc, M, N, K, epi, alpha, status, stream);
      return;
    }
  }
  const int kblocks = (K + BK - 1) / BK;
  int k_splits = 1;
  if (epi == EPI_F32_ATOMIC) {
    double best = 1e30;
    for (int s = 1; s <= 8; ++s) {
      if (s > 1 && (kblocks / s < 8 || tiles >= 6LL * sms)) break;
      const double waves = (double)((tiles * s + sms - 1) / sms) / s * (1.0 + 0.02 * (s - 1));
      if (waves < best * 0.97) { best = waves; k_splits = s; }
    }
    if (k_splits == 1) epi = EPI_F32_ACC;  // one tile per output block: same sum, no atomic traffic
  }
  uint64_t adims[2], astr[1], bdims[2], bstr[1];
  uint32_t abox[2], bbox[2];
  if (!a_mn) { adims[0] = K; adims[1] = M; abox[0] = BK; abox[1] = BM; }
  else       { adims[0] = M; adims[1] = K; abox[0] = 64; abox[1] = BK; }
  astr[0] = (uint64_t)lda * 2;
  if (!b_mn) { bdims[0] = K; bdims[1] = N; bbox[0] = BK; bbox[1] = (uint32_t)BN; }
  else       { bdims[0] = N; bdims[1] = K; bbox[0] = 64; bbox[1] = BK; }
  bstr[0] = (uint64_t)ldb * 2;
  const CUtensorMap ta = make_tensor_map(A, TmaDType::BF16, 2, adims, astr, abox, true);
  const CUtensorMap tb = make_tensor_map(B, TmaDType::BF16, 2, bdims, bstr, bbox, true);

#define MB_GEMM_DISPATCH(AMN, BMN)                                                                            \
  do {                                                                                                        \
    if (use256) launch_cfg<256, 4, AMN, BMN>(ta, tb, C, M, N, K, ldc, k_splits, epi, vec_ok, alpha, status, stream); \
    else launch_cfg<128, 6, AMN, BMN>(ta, tb, C, M, N, K, ldc, k_splits, epi, vec_ok, alpha, status, stream);  \
  } while (0)
  if (!a_mn && !b_mn) MB_GEMM_DISPATCH(false, false);
  else if (!a_mn && b_mn) MB_GEMM_DISPATCH(false, true);
  else MB_GEMM_DISPATCH(true, true);
#undef MB_GEMM_DISPATCH
}

}  // namespace mb
