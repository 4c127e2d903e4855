// Codebook-dequant GEMM for inference: y[M,N] = x[M,K] * dequant(W)[N,K]^T with W stored in an
// OIL format (OIL8 byte indices, OIL4 nibble indices, I2_S 2-bit trits + per-block scale).
//
// The weight matrix is the A operand of tcgen05.mma (128 weight rows per CTA), the activations
// are the B operand (up to 256 tokens, TMA-loaded), so the accumulator in TMEM is y^T: lane =
// output feature, column = token. Four producer warps expand indices through the codebook into a
// 128-byte-swizzled bf16 shared tile (one thread per weight row, 64 weights = one 128-byte row per
// k-block) that the tensor core consumes directly; the packed weights are read from HBM exactly
// once, which is what a decode step is bound by. Split-K CTAs fill the machine when N is small
// (tensor-parallel shards) and combine with fp32 reductions.
//
// Fused collective: with `peers` set, every CTA adds its fp32 partial tile straight into the
// accumulation buffer of EVERY rank (peer red.add over NVLink), so a row-parallel projection
// leaves the all-reduced result on all ranks without a separate collective.
//
// Semantics follow the reference reader's dequantisation (src/oil_format.cpp:434-455) followed
// by a GEMM; the reference's own quantised "GEMMs" (src/kernel_oil8.cpp:14-71,
// src/kernel_oil4.cpp:31-125, src/kernel_i2s.cpp:32-65) use a distinct index row per output
// element and are only called from tests, so the weight-shared layout is used here.
#include "api.h"
#include "host_util.h"
#include "tc.cuh"

namespace mb {
namespace {

constexpr int DQ_BM = 128;  // weight rows per CTA
constexpr int DQ_BK = 64;
constexpr int DQ_THREADS = 192;
constexpr int DQ_STAGES = 4;

struct DqSmem {
  static constexpr int A_BYTES = DQ_BM * DQ_BK * 2;     // 16 KB
  static constexpr int B_BYTES_MAX = 256 * DQ_BK * 2;   // 32 KB
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES_MAX;
  static constexpr int BAR_OFFSET = DQ_STAGES * STAGE_BYTES;
  static constexpr int NUM_BARS = 3 * DQ_STAGES + 1;
  static constexpr int CB_SLOTS = 16;                                // codebooks cached per producer warp
  static constexpr int CB_OFFSET = (BAR_OFFSET + NUM_BARS * 8 + 16 + 15) / 16 * 16; // [4 warps][CB_SLOTS][256] bf16
  static constexpr int SMEM_BYTES = CB_OFFSET + 4 * CB_SLOTS * 256 * 2 + 1024;
  static_assert(SMEM_BYTES <= 232448, "dequant GEMM shared memory exceeds the per-CTA limit");
};

__device__ __forceinline__ uint32_t bf16_bits(float v) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16(v));
}

template <bool SMEM>
__device__ __forceinline__ uint32_t cb_at(const unsigned short* cb, uint32_t i) {
  return SMEM ? (uint32_t)cb[i] : (uint32_t)__ldg(cb + i);
}

// Expand 64 weights of one row into 8 packed uint4 (8 bf16 each). `cb` is the row's codebook for
// this k-block: a shared-memory copy (SMEM) or the table in global memory.
template <int FMT, bool SMEM>
__device__ __forceinline__ void dequant_row64(const DequantWeights& w, long long row, int k0,
                                              const unsigned short* cb, uint4 (&out)[8]) {
  const long long elem = row * w.K + k0;
  if (FMT == QFMT_OIL8) {
    const uint4* ip = reinterpret_cast<const uint4*>(w.packed + elem);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 v = __ldg(ip + c);
      const uint32_t words[4] = {v.x, v.y, v.z, v.w};
      uint32_t o[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t x = words[j];
        o[2 * j] = cb_at<SMEM>(cb, x & 0xFF) | (cb_at<SMEM>(cb, (x >> 8) & 0xFF) << 16);
        o[2 * j + 1] = cb_at<SMEM>(cb, (x >> 16) & 0xFF) | (cb_at<SMEM>(cb, x >> 24) << 16);
      }
      out[2 * c] = make_uint4(o[0], o[1], o[2], o[3]);
      out[2 * c + 1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
  } else if (FMT == QFMT_OIL4) {
    const uint4* ip = reinterpret_cast<const uint4*>(w.packed + elem / 2);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint4 v = __ldg(ip + c);
      const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // one 32-bit word = 8 nibbles = 8 weights, even index in the low nibble
        const uint32_t x = words[j];
        uint32_t o[4];
#pragma unroll
        for (int p = 0; p < 4; ++p)
          o[p] = cb_at<SMEM>(cb, (x >> (8 * p)) & 0xF) | (cb_at<SMEM>(cb, (x >> (8 * p + 4)) & 0xF) << 16);
        out[4 * c + j] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  } else {  // I2_S: code = trit + 1 in 2 bits, LSB first; value = (code - 1) * scale
    const float scale = w.scales[elem / w.block_size];
    const uint32_t lut[4] = {bf16_bits(-scale), 0u, bf16_bits(scale), 0u};
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(w.packed + elem / 4));
    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // one word = 16 weights = two uint4 outputs
      const uint32_t x = words[j];
      uint32_t o[8];
#pragma unroll
      for (int p = 0; p < 8; ++p) o[p] = lut[(x >> (4 * p)) & 3] | (lut[(x >> (4 * p + 2)) & 3] << 16);
      out[2 * j] = make_uint4(o[0], o[1], o[2], o[3]);
      out[2 * j + 1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
  }
}

template <int FMT>
__global__ void __launch_bounds__(DQ_THREADS, 1)
dequant_gemm_kernel(const __grid_constant__ CUtensorMap tma_x, DequantWeights w, int M, int mt, int k_splits,
                    __nv_bfloat16* __restrict__ out_bf16, float* __restrict__ out_f32, PeerPtrs peers, int n_peers,
                    long long ld_out, int* status) {
  using S = DqSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full_a = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* full_b = full_a + DQ_STAGES;
  uint64_t* empty = full_b + DQ_STAGES;
  uint64_t* done = empty + DQ_STAGES;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * DQ_BM;
  const int split = blockIdx.y;
  const int m0 = blockIdx.z * mt;
  const int kblocks = w.K / DQ_BK;
  const int base = kblocks / k_splits, rem = kblocks % k_splits;
  const int kb0 = split * base + min(split, rem);
  const int kb1 = kb0 + base + (split < rem ? 1 : 0);
  const uint32_t tmem_cols = mt <= 32 ? 32 : (mt <= 64 ? 64 : (mt <= 128 ? 128 : 256));

  if (threadIdx.x == 0) {
    for (int s = 0; s < DQ_STAGES; ++s) {
      mbar_init(&full_a[s], 128);
      mbar_init(&full_b[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = kb0, it = 0; kb < kb1; ++kb, ++it) {
        const int st = it % DQ_STAGES;
        const uint32_t ph = (it / DQ_STAGES) & 1;
        if (!mbar_wait(&empty[st], ph ^ 1, abort_flag, status, 61)) break;
        mbar_arrive_expect_tx(&full_b[st], (uint32_t)mt * 128u);
        tma_load_2d(smem + st * S::STAGE_BYTES + S::A_BYTES, &tma_x, &full_b[st], kb * DQ_BK, m0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(DQ_BM, mt, false, false);
      bool ok = true;
      for (int kb = kb0, it = 0; kb < kb1 && ok; ++kb, ++it) {
        const int st = it % DQ_STAGES;
        const uint32_t ph = (it / DQ_STAGES) & 1;
        if (!mbar_wait(&full_a[st], ph, abort_flag, status, 62)) { ok = false; break; }
        if (!mbar_wait(&full_b[st], ph, abort_flag, status, 63)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + st * S::STAGE_BYTES);
        const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
        for (int k = 0; k < DQ_BK / 16; ++k)
          umma_f16(tmem_base, umma_desc_sw128(a_addr + k * 32, 0, 1024), umma_desc_sw128(b_addr + k * 32, 0, 1024),
                   idesc, (it > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty[st]);
      }
      if (ok) umma_commit(done);
    }
  } else {
    // ---------------- dequant producers, then epilogue
    const int r = (warp & 3) * 32 + lane;
    const long long row = (long long)n0 + r;
    const bool row_ok = row < w.N;
    bool ok = true;
    constexpr int CBSZ = (FMT == QFMT_OIL4) ? 16 : 256;
    unsigned short* warp_cb =
        reinterpret_cast<unsigned short*>(smem + S::CB_OFFSET) + (warp & 3) * (S::CB_SLOTS * 256);
    const unsigned short* cb_global = reinterpret_cast<const unsigned short*>(w.codebooks);
    int cached_lo = 0, cached_hi = -1;   // codebooks [cached_lo, cached_hi] are in warp_cb
    for (int kb = kb0, it = 0; kb < kb1; ++kb, ++it) {
      const int st = it % DQ_STAGES;
      const uint32_t ph = (it / DQ_STAGES) & 1;
      uint4 vals[8];
      if (FMT == QFMT_I2S) {
        if (row_ok) dequant_row64<FMT, false>(w, row, kb * DQ_BK, nullptr, vals);
      } else {
        // Codebook of this row for this k-block. The 32 rows of a warp usually use a short run of
        // consecutive codebooks: keep up to CB_SLOTS of them in a per-warp shared-memory table so
        // the 64 look-ups per row are shared-memory reads; wider spreads gather from global memory.
        int cbi = -1;
        if (row_ok) {
          const long long blk = (row * w.K + (long long)kb * DQ_BK) / w.block_size;
          cbi = w.cb_map ? w.cb_map[blk] : (int)blk;
        }
        const int hi = __reduce_max_sync(0xffffffffu, cbi);
        const int lo = __reduce_min_sync(0xffffffffu, row_ok ? cbi : 0x7fffffff);
        if (hi >= 0 && hi - lo < S::CB_SLOTS) {
          if (lo < cached_lo || hi > cached_hi) {
            __syncwarp();
            const int last = min(lo + S::CB_SLOTS, w.n_codebooks) - 1;
            const int n_vec = (last - lo + 1) * CBSZ / 8;   // codebooks are 32- or 512-byte records
            const uint4* src = reinterpret_cast<const uint4*>(cb_global + (long long)lo * CBSZ);
            for (int i = lane; i < n_vec; i += 32) reinterpret_cast<uint4*>(warp_cb)[i] = __ldg(src + i);
            cached_lo = lo;
            cached_hi = last;
            __syncwarp();
          }
          if (row_ok) dequant_row64<FMT, true>(w, row, kb * DQ_BK, warp_cb + (cbi - cached_lo) * CBSZ, vals);
        } else if (row_ok) {
          dequant_row64<FMT, false>(w, row, kb * DQ_BK, cb_global + (long long)cbi * CBSZ, vals);
        }
      }
      if (!row_ok) {
#pragma unroll
        for (int c = 0; c < 8; ++c) vals[c] = make_uint4(0, 0, 0, 0);
      }
      ok = mbar_wait(&empty[st], ph ^ 1, abort_flag, status, 64);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      uint8_t* a_tile = smem + st * S::STAGE_BYTES;
#pragma unroll
      for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(a_tile + sw128_offset(r, c)) = vals[c];
      fence_proxy_async_smem();
      mbar_arrive(&full_a[st]);
    }
    if (ok) {
      ok = mbar_wait(done, 0, abort_flag, status, 65);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
      for (int c = 0; c < mt; c += 16) {
        uint32_t v[16];
        tmem_ld16(t_row + c, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c + j;
            if (m < M) {
              const float val = __uint_as_float(v[j]);
              const long long off = (long long)m * ld_out + row;
              if (out_f32 || n_peers > 0) {
                if (n_peers > 0) {
                  for (int p = 0; p < n_peers; ++p) atomicAdd(reinterpret_cast<float*>(peers.p[p]) + off, val);
                } else {
                  atomicAdd(out_f32 + off, val);
                }
              } else {
                out_bf16[off] = __float2bfloat16(val);
              }
            }
          }
        }
      }
    }
  }

  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 10000000LL) {}
    __syncthreads();
  }
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// out_bf16[m, n] = bf16(acc[m, n] (+ residual[m, n])); acc is zeroed for its next use.
__global__ void finalize_acc_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ residual,
                                    __nv_bfloat16* __restrict__ out, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = acc[i];
    if (residual) v += __bfloat162float(residual[i]);
    out[i] = __float2bfloat16(v);
    acc[i] = 0.f;
  }
}

// Full dequantisation to bf16 (prefill path: dequantise once into scratch, then the dense GEMM).
template <int FMT>
__global__ void dequant_full_kernel(DequantWeights w, __nv_bfloat16* __restrict__ out) {
  const long long chunks = (long long)w.N * (w.K / 64);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / (w.K / 64);
    const int k0 = (int)(i % (w.K / 64)) * 64;
    uint4 vals[8];
    const unsigned short* cb = nullptr;
    if (FMT != QFMT_I2S) {
      const long long blk = (row * w.K + k0) / w.block_size;
      const int cbi = w.cb_map ? w.cb_map[blk] : (int)blk;
      cb = reinterpret_cast<const unsigned short*>(w.codebooks) + (long long)cbi * ((FMT == QFMT_OIL4) ? 16 : 256);
    }
    dequant_row64<FMT, false>(w, row, k0, cb, vals);
    uint4* dst = reinterpret_cast<uint4*>(out + row * w.K + k0);
#pragma unroll
    for (int c = 0; c < 8; ++c) dst[c] = vals[c];
  }
}

}  // namespace

void dequant_gemm(const void* x, long long ldx, int M, const DequantWeights& w, void* out_bf16, float* out_f32,
                  const PeerPtrs* peers, int n_peers, long long ld_out, int k_splits, int* status, cudaStream_t stream) {
  MB_REQUIRE(w.K % 64 == 0, "dequant_gemm: K must be a multiple of 64");
  MB_REQUIRE(w.block_size % 64 == 0 && w.K % w.block_size == 0,
             "dequant_gemm: quantisation blocks must be multiples of 64 weights and tile the rows");
  MB_REQUIRE(ldx % 8 == 0, "dequant_gemm: activation row stride must be a multiple of 8 elements");
  MB_REQUIRE(M > 0, "dequant_gemm: no tokens");
  MB_REQUIRE((out_bf16 != nullptr) != (out_f32 != nullptr || n_peers > 0), "dequant_gemm: exactly one output kind");
  int mt = ((M + 15) / 16) * 16;
  if (mt > 256) mt = 256;
  const int m_tiles = (M + mt - 1) / mt;
  const int n_tiles = (w.N + DQ_BM - 1) / DQ_BM;
  const int kblocks = w.K / DQ_BK;
  if (k_splits <= 0) {
    k_splits = 1;
    if (out_bf16 == nullptr) {
      const int want = (sm_count() + n_tiles * m_tiles - 1) / (n_tiles * m_tiles);
      k_splits = want < 1 ? 1 : want;
      if (k_splits > kblocks / 2) k_splits = kblocks / 2 > 0 ? kblocks / 2 : 1;
    }
  }
  MB_REQUIRE(out_bf16 == nullptr || k_splits == 1, "dequant_gemm: split-K needs the fp32 accumulate output");
  uint64_t dims[2] = {(uint64_t)w.K, (uint64_t)M};
  uint64_t strides[1] = {(uint64_t)ldx * 2};
  uint32_t box[2] = {64, (uint32_t)mt};
  const CUtensorMap tx = make_tensor_map(x, TmaDType::BF16, 2, dims, strides, box, true);
  PeerPtrs pp{};
  if (peers) pp = *peers;
  const dim3 grid(n_tiles, k_splits, m_tiles);
#define MB_DQ_LAUNCH(F)                                                                                             \
  do {                                                                                                              \
    static bool configured = false;                                                                                 \
    if (!configured) {                                                                                              \
      MB_CUDA_CHECK(cudaFuncSetAttribute(dequant_gemm_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                         DqSmem::SMEM_BYTES));                                                      \
      configured = true;                                                                                            \
    }                                                                                                               \
    dequant_gemm_kernel<F><<<grid, DQ_THREADS, DqSmem::SMEM_BYTES, stream>>>(                                        \
        tx, w, M, mt, k_splits, (__nv_bfloat16*)out_bf16, out_f32, pp, n_peers, ld_out, status);                    \
  } while (0)
  if (w.fmt == QFMT_OIL8) MB_DQ_LAUNCH(QFMT_OIL8);
  else if (w.fmt == QFMT_OIL4) MB_DQ_LAUNCH(QFMT_OIL4);
  else if (w.fmt == QFMT_I2S) MB_DQ_LAUNCH(QFMT_I2S);
  else MB_REQUIRE(false, "dequant_gemm: unknown weight format");
#undef MB_DQ_LAUNCH
  count_launch();
  check_launch();
}

void finalize_acc(float* acc, const void* residual, void* out, long long n, cudaStream_t stream) {
  if (n == 0) return;
  long long g = (n + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  finalize_acc_kernel<<<(int)g, 256, 0, stream>>>(acc, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, n);
  count_launch();
  check_launch();
}

void dequant_to_bf16(const DequantWeights& w, void* out, cudaStream_t stream) {
  MB_REQUIRE(w.K % 64 == 0 && w.block_size % 64 == 0, "dequant_to_bf16: K and block size must be multiples of 64");
  const long long chunks = (long long)w.N * (w.K / 64);
  if (chunks == 0) return;
  long long g = (chunks + 127) / 128;
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  if (w.fmt == QFMT_OIL8) dequant_full_kernel<QFMT_OIL8><<<(int)g, 128, 0, stream>>>(w, (__nv_bfloat16*)out);
  else if (w.fmt == QFMT_OIL4) dequant_full_kernel<QFMT_OIL4><<<(int)g, 128, 0, stream>>>(w, (__nv_bfloat16*)out);
  else if (w.fmt == QFMT_I2S) dequant_full_kernel<QFMT_I2S><<<(int)g, 128, 0, stream>>>(w, (__nv_bfloat16*)out);
  else MB_REQUIRE(false, "dequant_to_bf16: unknown weight format");
  count_launch();
  check_launch();
}

}  // namespace mb
