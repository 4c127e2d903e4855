// Codebook-dequant GEMM for inference: y[M,N] = x[M,K] * dequant(W)[N,K]^T with W stored in an
// OIL format (OIL8 byte indices, OIL4 nibble indices, I2_S 2-bit trits + per-block scale).
//
// The weight matrix is the A operand of tcgen05.mma (128 weight rows per CTA), the activations
// are the B operand (up to 256 tokens), so the accumulator in TMEM is y^T: lane = output feature,
// column = token. Data flow per 64-wide k-block:
//   TMA  : packed indices [128 rows x 64/32/16 B] -> raw ring (up to 16 stages, deep enough to
//          cover HBM latency at full bandwidth); activations [tokens x 64] -> B tile (128B swizzle)
//   8 producer warps: raw bytes -> codebook look-up -> bf16 -> 128B-swizzled A tile. A thread owns
//          16 weights of a row per pass, 4 lanes cover a row's k-block and a warp covers 8 rows, so
//          raw reads and tile writes are bank-conflict free.
//   1 thread: tcgen05.mma A(smem) x B(smem) -> TMEM, commit frees the A/B stage.
// The packed weights are read from HBM exactly once, which is what a decode step is bound by.
// Look-up tables live in shared memory: OIL8 keeps up to 8 consecutive 256-entry codebooks per warp (its 16 rows rarely span more; wider spreads gather
// from global memory); OIL4 and I2_S
// keep a private 16-entry table per thread and row, interleaved so that every lane reads its own
// bank (OIL4: the row's codebook; I2_S: nibble -> two scaled trits).
// Split-K CTAs fill the machine when N is small (tensor-parallel shards) and combine with fp32
// reductions.
//
// Fused collective: with `peers` set, the epilogue writes over NVLink instead of to local memory.
// Either every CTA adds its fp32 partial tile into the accumulation buffer of EVERY rank (peer
// red.add), or (peer_bf16_offset >= 0, single K split) it stores the bf16 tile into this rank's
// slot of every rank's staging buffer, the first half of a one-shot all-reduce whose second half
// is a local sum over the slots after one barrier.
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
constexpr int DQ_PRODUCERS = 256;             // 8 warps
constexpr int DQ_THREADS = 96 + DQ_PRODUCERS;  // raw loader, MMA issuer, activation loader, producers
constexpr int DQ_MAX_RAW = 16;
constexpr int DQ_MAX_AB = 4;
constexpr int DQ_SMEM_LIMIT = 232448;          // per CTA
constexpr int DQ_SMEM_HALF = 113 * 1024;       // two CTAs per SM fit below this

__host__ __device__ constexpr int dq_raw_row_bytes(int fmt) {
  return fmt == QFMT_OIL8 ? 64 : (fmt == QFMT_OIL4 ? 32 : 16);
}

// Shared-memory plan, computed on the host and passed to the kernel.
struct DqPlan {
  int raw_stages, ab_stages;
  int raw_stage_bytes, ab_stage_bytes;  // ab stage = 16 KB A tile + mt*128 B activation tile
  int cb_slots;                         // OIL8: codebooks cached per producer warp
  int off_ab, off_lut, off_bar, total;  // raw ring starts at 0
};

// Decode-sized token tiles (<= 64) get a plan small enough for two CTAs per SM: twice the warps
// to hide look-up latency and no idle half-wave when the tile count is not a multiple of the SMs.
DqPlan dq_plan(int fmt, int mt) {
  DqPlan p;
  const bool two = mt <= 64;
  p.raw_stage_bytes = DQ_BM * dq_raw_row_bytes(fmt);
  p.ab_stage_bytes = DQ_BM * DQ_BK * 2 + mt * DQ_BK * 2;
  p.ab_stages = two ? 2 : (mt > 128 ? 3 : DQ_MAX_AB);
  p.cb_slots = 8;
  // look-up tables: OIL8 8 warps x slots x 512 B; OIL4 2 rows x 16 x 256 halfwords; I2_S 2 x 16 x 256 words
  const int lut = fmt == QFMT_OIL8 ? 8 * p.cb_slots * 512 : (fmt == QFMT_OIL4 ? 16384 : 32768);
  const int fixed = p.ab_stages * p.ab_stage_bytes + lut + 1024 /*barriers*/ + 1024 /*alignment*/;
  int rs = ((two ? DQ_SMEM_HALF : DQ_SMEM_LIMIT) - fixed) / p.raw_stage_bytes;
  p.raw_stages = rs > DQ_MAX_RAW ? DQ_MAX_RAW : rs;
  p.off_ab = p.raw_stages * p.raw_stage_bytes;          // multiples of 2 KB: 1024-aligned tiles
  p.off_lut = p.off_ab + p.ab_stages * p.ab_stage_bytes;
  p.off_bar = p.off_lut + lut;
  p.total = p.off_bar + 1024 + 1024;
  return p;
}

__device__ __forceinline__ uint32_t lds_u16(uint32_t saddr) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(saddr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t saddr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t bf16_bits(float v) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16(v));
}

// 16 OIL8 indices (one uint4) -> 16 bf16 through a 256-entry table: in shared memory at the 32-bit
// shared address `cb_saddr` (SMEM), or in global memory at `cb`.
template <bool SMEM>
__device__ __forceinline__ void oil8_expand16(const uint4 v, const unsigned short* cb, uint32_t cb_saddr,
                                              uint4 (&out)[2]) {
  const uint32_t words[4] = {v.x, v.y, v.z, v.w};
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t x = words[j];
    uint32_t e[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t idx = __byte_perm(x, 0, 0x4440 + b);   // byte b, zero-extended
      e[b] = SMEM ? lds_u16(cb_saddr + 2 * idx) : (uint32_t)__ldg(cb + idx);
    }
    o[2 * j] = __byte_perm(e[0], e[1], 0x5410);
    o[2 * j + 1] = __byte_perm(e[2], e[3], 0x5410);
  }
  out[0] = make_uint4(o[0], o[1], o[2], o[3]);
  out[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

template <int FMT>
__global__ void __launch_bounds__(DQ_THREADS, 2)
dequant_gemm_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
                    DequantWeights w, DqPlan plan, int M, int mt, int k_splits,
                    __nv_bfloat16* __restrict__ out_bf16, float* __restrict__ out_f32, PeerPtrs peers, int n_peers,
                    long long peer_bf16_offset, long long ld_out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem + plan.off_bar);
  uint64_t* raw_empty = raw_full + DQ_MAX_RAW;
  uint64_t* a_full = raw_empty + DQ_MAX_RAW;
  uint64_t* b_full = a_full + DQ_MAX_AB;
  uint64_t* ab_empty = b_full + DQ_MAX_AB;
  uint64_t* done = ab_empty + DQ_MAX_AB;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * DQ_BM;
  const int split = blockIdx.y;
  const int m0 = blockIdx.z * mt;
  const int kblocks = w.K / DQ_BK;
  const int kbase = kblocks / k_splits, krem = kblocks % k_splits;
  const int kb0 = split * kbase + min(split, krem);
  const int kb1 = kb0 + kbase + (split < krem ? 1 : 0);
  const uint32_t tmem_cols = mt <= 32 ? 32 : (mt <= 64 ? 64 : (mt <= 128 ? 128 : 256));
  constexpr int RB = dq_raw_row_bytes(FMT);

  if (threadIdx.x == 0) {
    for (int s = 0; s < DQ_MAX_RAW; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], DQ_PRODUCERS);
    }
    for (int s = 0; s < DQ_MAX_AB; ++s) {
      mbar_init(&a_full[s], DQ_PRODUCERS);
      mbar_init(&b_full[s], 1);
      mbar_init(&ab_empty[s], 1);
    }
    mbar_init(done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_x);
    tma_prefetch_desc(&tma_w);
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
    // ---------------- packed-weight loader
    if (lane == 0) {
      int st = 0;
      uint32_t ph = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&raw_empty[st], ph ^ 1, abort_flag, status, 60)) break;
        mbar_arrive_expect_tx(&raw_full[st], (uint32_t)plan.raw_stage_bytes);
        tma_load_2d(smem + st * plan.raw_stage_bytes, &tma_w, &raw_full[st], kb * RB, n0);
        if (++st == plan.raw_stages) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 2) {
    // ---------------- activation loader
    if (lane == 0) {
      int st = 0;
      uint32_t ph = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&ab_empty[st], ph ^ 1, abort_flag, status, 61)) break;
        mbar_arrive_expect_tx(&b_full[st], (uint32_t)mt * 128u);
        tma_load_2d(smem + plan.off_ab + st * plan.ab_stage_bytes + DQ_BM * DQ_BK * 2, &tma_x, &b_full[st],
                    kb * DQ_BK, m0);
        if (++st == plan.ab_stages) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(DQ_BM, mt, false, false);
      bool ok = true;
      int st = 0;
      uint32_t ph = 0;
      for (int kb = kb0, it = 0; kb < kb1 && ok; ++kb, ++it) {
        if (!mbar_wait(&a_full[st], ph, abort_flag, status, 62)) { ok = false; break; }
        if (!mbar_wait(&b_full[st], ph, abort_flag, status, 63)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + plan.off_ab + st * plan.ab_stage_bytes);
        const uint32_t b_addr = a_addr + DQ_BM * DQ_BK * 2;
#pragma unroll
        for (int k = 0; k < DQ_BK / 16; ++k)
          umma_f16(tmem_base, umma_desc_sw128(a_addr + k * 32, 0, 1024), umma_desc_sw128(b_addr + k * 32, 0, 1024),
                   idesc, (it > 0 || k > 0) ? 1u : 0u);
        umma_commit(&ab_empty[st]);
        if (++st == plan.ab_stages) { st = 0; ph ^= 1; }
      }
      if (ok) umma_commit(done);
    }
  } else {
    // ---------------- dequant producers, then epilogue
    const int pw = warp - 3;             // producer warp 0..7, owns tile rows [16 pw, 16 pw + 16)
    const int pt = threadIdx.x - 96;     // 0..255
    const int q = lane & 3;              // which 16-weight quarter of the row's k-block
    int trow[2];                         // tile rows of this thread's two passes
    bool row_ok[2];
    long long blk0[2];                   // first quantisation block of the row
    trow[0] = 16 * pw + (lane >> 2);
    trow[1] = trow[0] + 8;
    const int bpr = w.K / w.block_size;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      row_ok[j] = n0 + trow[j] < w.N;
      blk0[j] = (long long)(n0 + trow[j]) * bpr;
    }
    const int kb_per_block = w.block_size / DQ_BK;
    uint8_t* lut_mem = smem + plan.off_lut;
    // OIL8: per-warp cache of codebooks [cached_lo, cached_hi]
    unsigned short* warp_cb = reinterpret_cast<unsigned short*>(lut_mem) + pw * (plan.cb_slots * 256);
    const uint32_t warp_cb_saddr = smem_u32(warp_cb);
    const unsigned short* cb_global = reinterpret_cast<const unsigned short*>(w.codebooks);
    int cached_lo = 0, cached_hi = -1;
    int cbi[2] = {-1, -1};
    bool use_cache = false;
    // OIL4: halfword (j*16 + e) * 256 + pt, I2_S: word (j*16 + e) * 256 + pt holds entry e of this
    // thread's row j: a lane always reads its own bank
    unsigned short* lut_h = reinterpret_cast<unsigned short*>(lut_mem) + pt;
    uint32_t* lut_w = reinterpret_cast<uint32_t*>(lut_mem) + pt;
    const uint32_t lut_h_saddr = smem_u32(lut_h), lut_w_saddr = smem_u32(lut_w);
    bool ok = true;
    int kblk = kb0 / kb_per_block;            // quantisation block (along K) of the current k-block
    int kb_in_blk = kb0 - kblk * kb_per_block;
    int rs = 0, st = 0;                        // raw / tile ring positions and phases
    uint32_t rph = 0, sph = 0;

    for (int kb = kb0, it = 0; kb < kb1; ++kb, ++it) {
      // ---- refresh look-up tables when the k-block enters a new quantisation block
      if (it == 0 || kb_in_blk == 0) {
        if (FMT == QFMT_OIL8) {
#pragma unroll
          for (int j = 0; j < 2; ++j)
            cbi[j] = row_ok[j] ? (w.cb_map ? w.cb_map[blk0[j] + kblk] : (int)(blk0[j] + kblk)) : -1;
          const int hi = __reduce_max_sync(0xffffffffu, max(cbi[0], cbi[1]));
          const int lo = __reduce_min_sync(0xffffffffu, min(row_ok[0] ? cbi[0] : 0x7fffffff,
                                                            row_ok[1] ? cbi[1] : 0x7fffffff));
          use_cache = hi >= 0 && hi - lo < plan.cb_slots;
          if (use_cache && (lo < cached_lo || hi > cached_hi)) {
            __syncwarp();
            const int last = min(lo + plan.cb_slots, w.n_codebooks) - 1;
            const int n_vec = (last - lo + 1) * 32;   // 512-byte codebooks as uint4
            const uint4* src = reinterpret_cast<const uint4*>(cb_global + (long long)lo * 256);
            for (int i = lane; i < n_vec; i += 32) reinterpret_cast<uint4*>(warp_cb)[i] = __ldg(src + i);
            cached_lo = lo;
            cached_hi = last;
            __syncwarp();
          }
        } else if (FMT == QFMT_OIL4) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            if (!row_ok[j]) continue;
            const int c = w.cb_map ? w.cb_map[blk0[j] + kblk] : (int)(blk0[j] + kblk);
            if (c == cbi[j]) continue;
            cbi[j] = c;
            const uint4* src = reinterpret_cast<const uint4*>(cb_global + (long long)c * 16);
            const uint4 a = __ldg(src), b = __ldg(src + 1);
            const uint32_t e[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              lut_h[(j * 16 + 2 * i) * 256] = (unsigned short)(e[i] & 0xFFFFu);
              lut_h[(j * 16 + 2 * i + 1) * 256] = (unsigned short)(e[i] >> 16);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            if (!row_ok[j]) continue;
            const float scale = w.scales[blk0[j] + kblk];
            const uint32_t v[4] = {bf16_bits(-scale), 0u, bf16_bits(scale), 0u};   // code = trit + 1
#pragma unroll
            for (int e = 0; e < 16; ++e) lut_w[(j * 16 + e) * 256] = v[e & 3] | (v[e >> 2] << 16);
          }
        }
      }

      if (++kb_in_blk == kb_per_block) { kb_in_blk = 0; ++kblk; }

      // ---- raw indices of this k-block
      ok = mbar_wait(&raw_full[rs], rph, abort_flag, status, 64);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint8_t* raw = smem + rs * plan.raw_stage_bytes;
      uint4 vals[2][2];
      if (FMT == QFMT_OIL8) {
        uint4 r[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) r[j] = *reinterpret_cast<const uint4*>(raw + trow[j] * RB + q * 16);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (!row_ok[j]) {
            vals[j][0] = vals[j][1] = make_uint4(0, 0, 0, 0);
          } else if (use_cache) {
            oil8_expand16<true>(r[j], nullptr, warp_cb_saddr + (uint32_t)(cbi[j] - cached_lo) * 512u, vals[j]);
          } else {
            oil8_expand16<false>(r[j], cb_global + (long long)cbi[j] * 256, 0u, vals[j]);
          }
        }
      } else if (FMT == QFMT_OIL4) {
        uint2 r[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) r[j] = *reinterpret_cast<const uint2*>(raw + trow[j] * RB + q * 8);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint32_t words[2] = {r[j].x, r[j].y};
          uint32_t o[8];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {   // byte b of word h: weights 8h+2b (low nibble), 8h+2b+1
              const uint32_t lo4 = (words[h] >> (8 * b)) & 0xF, hi4 = (words[h] >> (8 * b + 4)) & 0xF;
              o[4 * h + b] = __byte_perm(lds_u16(lut_h_saddr + (j * 16 + lo4) * 512),
                                         lds_u16(lut_h_saddr + (j * 16 + hi4) * 512), 0x5410);
            }
          }
          if (!row_ok[j]) {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = 0;
          }
          vals[j][0] = make_uint4(o[0], o[1], o[2], o[3]);
          vals[j][1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
      } else {
        uint32_t r[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) r[j] = *reinterpret_cast<const uint32_t*>(raw + trow[j] * RB + q * 4);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = lds_u32(lut_w_saddr + (j * 16 + ((r[j] >> (4 * i)) & 0xF)) * 1024);
          if (!row_ok[j]) {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = 0;
          }
          vals[j][0] = make_uint4(o[0], o[1], o[2], o[3]);
          vals[j][1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }

      // The raw stage is released only here, after the look-ups consumed the index registers: an
      // arrive issued right behind the shared loads does not wait for them, and the refill of the
      // stage by TMA could overtake the tail of a wide load.
      mbar_arrive_after(&raw_empty[rs], vals[0][0].x ^ vals[0][1].w ^ vals[1][0].x ^ vals[1][1].w);

      // ---- publish the bf16 tile
      ok = mbar_wait(&ab_empty[st], sph ^ 1, abort_flag, status, 65);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      uint8_t* a_tile = smem + plan.off_ab + st * plan.ab_stage_bytes;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        *reinterpret_cast<uint4*>(a_tile + sw128_offset(trow[j], 2 * q)) = vals[j][0];
        *reinterpret_cast<uint4*>(a_tile + sw128_offset(trow[j], 2 * q + 1)) = vals[j][1];
      }
      fence_proxy_async_smem();
      mbar_arrive(&a_full[st]);
      if (++rs == plan.raw_stages) { rs = 0; rph ^= 1; }
      if (++st == plan.ab_stages) { st = 0; sph ^= 1; }
    }

    // ---------------- epilogue: warp quarter = TMEM lane group, the two warps of a quarter
    // alternate over 16-token column chunks
    if (ok) {
      ok = mbar_wait(done, 0, abort_flag, status, 66);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const int quarter = warp & 3;
      const int half = pw >> 2;
      const long long row = (long long)n0 + quarter * 32 + lane;
      const bool r_ok = row < w.N;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
      for (int c = half * 16; c < mt; c += 32) {
        uint32_t v[16];
        tmem_ld16(t_row + c, v);
        tmem_ld_wait();
        if (r_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c + j;
            if (m < M) {
              const float val = __uint_as_float(v[j]);
              const long long off = (long long)m * ld_out + row;
              if (n_peers > 0 && peer_bf16_offset >= 0) {
                const __nv_bfloat16 b = __float2bfloat16(val);   // this rank's slot in every peer's staging buffer
                for (int p = 0; p < n_peers; ++p)
                  reinterpret_cast<__nv_bfloat16*>(peers.p[p])[peer_bf16_offset + off] = b;
              } else if (n_peers > 0) {
                for (int p = 0; p < n_peers; ++p) atomicAdd(reinterpret_cast<float*>(peers.p[p]) + off, val);
              } else if (out_f32) {
                atomicAdd(out_f32 + off, val);
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

// The 16 weights that start at flat element ``elem`` (a multiple of 16), as two 16-byte bf16 words.
template <int FMT>
__device__ __forceinline__ void expand_unit(const DequantWeights& w, long long elem, uint4 (&vals)[2]) {
  const long long blk = elem / w.block_size;
  if (FMT == QFMT_OIL8) {
    const int cbi = w.cb_map ? w.cb_map[blk] : (int)blk;
    oil8_expand16<false>(__ldg(reinterpret_cast<const uint4*>(w.packed + elem)),
                         reinterpret_cast<const unsigned short*>(w.codebooks) + (long long)cbi * 256, 0u, vals);
  } else if (FMT == QFMT_OIL4) {
    const int cbi = w.cb_map ? w.cb_map[blk] : (int)blk;
    const unsigned short* cb = reinterpret_cast<const unsigned short*>(w.codebooks) + (long long)cbi * 16;
    const uint2 r = __ldg(reinterpret_cast<const uint2*>(w.packed + elem / 2));
    const uint32_t words[2] = {r.x, r.y};
    uint32_t o[8];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int b = 0; b < 4; ++b)
        o[4 * h + b] = (uint32_t)__ldg(cb + ((words[h] >> (8 * b)) & 0xF)) |
                       ((uint32_t)__ldg(cb + ((words[h] >> (8 * b + 4)) & 0xF)) << 16);
    vals[0] = make_uint4(o[0], o[1], o[2], o[3]);
    vals[1] = make_uint4(o[4], o[5], o[6], o[7]);
  } else {
    const float scale = w.scales[blk];
    const uint32_t neg = bf16_bits(-scale), pos = bf16_bits(scale);
    const uint32_t r = __ldg(reinterpret_cast<const uint32_t*>(w.packed + elem / 4));
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t c0 = (r >> (4 * i)) & 3, c1 = (r >> (4 * i + 2)) & 3;
      const uint32_t v0 = c0 == 0 ? neg : (c0 == 2 ? pos : 0u), v1 = c1 == 0 ? neg : (c1 == 2 ? pos : 0u);
      o[i] = v0 | (v1 << 16);
    }
    vals[0] = make_uint4(o[0], o[1], o[2], o[3]);
    vals[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// Full dequantisation to bf16 (prefill path: dequantise once into scratch, then the dense GEMM).
// One thread expands 16 weights.
template <int FMT>
__global__ void dequant_full_kernel(DequantWeights w, __nv_bfloat16* __restrict__ out) {
  const long long units = (long long)w.N * w.K / 16;
  for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += (long long)gridDim.x * blockDim.x) {
    const long long elem = u * 16;
    uint4 vals[2];
    expand_unit<FMT>(w, elem, vals);
    uint4* dst = reinterpret_cast<uint4*>(out + elem);
    dst[0] = vals[0];
    dst[1] = vals[1];
  }
}

// Row gather through the quantised table: out[t, :] = dequant(W[ids[t], :]); ids are clamped to
// [0, N-1]. One thread per 16 weights, 32 bytes stored per thread.
template <int FMT>
__global__ void dequant_rows_kernel(DequantWeights w, const int* __restrict__ ids, int tokens,
                                    __nv_bfloat16* __restrict__ out, long long ld_out) {
  const int upr = w.K / 16;
  const long long units = (long long)tokens * upr;
  for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(u / upr), c = (int)(u % upr);
    int id = __ldg(ids + t);
    id = id < 0 ? 0 : (id >= w.N ? w.N - 1 : id);
    uint4 vals[2];
    expand_unit<FMT>(w, (long long)id * w.K + (long long)c * 16, vals);
    uint4* dst = reinterpret_cast<uint4*>(out + (long long)t * ld_out + (long long)c * 16);
    dst[0] = vals[0];
    dst[1] = vals[1];
  }
}

}  // namespace

void dequant_gemm(const void* x, long long ldx, int M, const DequantWeights& w, void* out_bf16, float* out_f32,
                  const PeerPtrs* peers, int n_peers, long long ld_out, int k_splits, int* status, cudaStream_t stream,
                  long long peer_bf16_offset) {
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
    if (out_bf16 == nullptr && peer_bf16_offset < 0) {
      const int want = (sm_count() + n_tiles * m_tiles - 1) / (n_tiles * m_tiles);
      k_splits = want < 1 ? 1 : want;
      if (k_splits > kblocks / 4) k_splits = kblocks / 4 > 0 ? kblocks / 4 : 1;
    }
  }
  if (k_splits > kblocks) k_splits = kblocks;
  MB_REQUIRE(out_bf16 == nullptr || k_splits == 1, "dequant_gemm: split-K needs the fp32 accumulate output");
  MB_REQUIRE(peer_bf16_offset < 0 || (n_peers > 0 && k_splits == 1),
             "dequant_gemm: bf16 peer stores need peers and a single K split");
  const DqPlan plan = dq_plan(w.fmt, mt);
  MB_REQUIRE(plan.raw_stages >= 2, "dequant_gemm: shared-memory plan has no room for the index ring");
  CUtensorMap tx, tw;
  {
    uint64_t dims[2] = {(uint64_t)w.K, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)ldx * 2};
    uint32_t box[2] = {64, (uint32_t)mt};
    tx = make_tensor_map(x, TmaDType::BF16, 2, dims, strides, box, true);
  }
  {
    // packed indices as bytes: row pitch K*bits/8, one k-block of a row = 64/32/16 bytes
    const int rb = dq_raw_row_bytes(w.fmt);
    const uint64_t pitch = (uint64_t)w.K / 64 * rb;
    uint64_t dims[2] = {pitch, (uint64_t)w.N};
    uint64_t strides[1] = {pitch};
    uint32_t box[2] = {(uint32_t)rb, (uint32_t)DQ_BM};
    tw = make_tensor_map(w.packed, TmaDType::U8, 2, dims, strides, box, false);
  }
  PeerPtrs pp{};
  if (peers) pp = *peers;
  const dim3 grid(n_tiles, k_splits, m_tiles);
#define MB_DQ_LAUNCH(F)                                                                                             \
  do {                                                                                                              \
    static bool configured = false;                                                                                 \
    if (!configured) {                                                                                              \
      MB_CUDA_CHECK(cudaFuncSetAttribute(dequant_gemm_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                         DQ_SMEM_LIMIT));                                                           \
      configured = true;                                                                                            \
    }                                                                                                               \
    dequant_gemm_kernel<F><<<grid, DQ_THREADS, plan.total, stream>>>(                                                \
        tx, tw, w, plan, M, mt, k_splits, (__nv_bfloat16*)out_bf16, out_f32, pp, n_peers, peer_bf16_offset, ld_out,    \
        status);          \
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
  const long long units = (long long)w.N * w.K / 16;
  if (units == 0) return;
  long long g = (units + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  if (w.fmt == QFMT_OIL8) dequant_full_kernel<QFMT_OIL8><<<(int)g, 256, 0, stream>>>(w, (__nv_bfloat16*)out);
  else if (w.fmt == QFMT_OIL4) dequant_full_kernel<QFMT_OIL4><<<(int)g, 256, 0, stream>>>(w, (__nv_bfloat16*)out);
  else if (w.fmt == QFMT_I2S) dequant_full_kernel<QFMT_I2S><<<(int)g, 256, 0, stream>>>(w, (__nv_bfloat16*)out);
  else MB_REQUIRE(false, "dequant_to_bf16: unknown weight format");
  count_launch();
  check_launch();
}

void dequant_gather_rows(const DequantWeights& w, const int* ids, int tokens, void* out, long long ld_out,
                         cudaStream_t stream) {
  MB_REQUIRE(w.K % 64 == 0 && w.block_size % 64 == 0, "dequant_gather_rows: K and block size must be multiples of 64");
  MB_REQUIRE(ld_out % 8 == 0 && ld_out >= w.K, "dequant_gather_rows: output row stride must be >= K and a multiple of 8");
  const long long units = (long long)tokens * (w.K / 16);
  if (units == 0) return;
  long long g = (units + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  __nv_bfloat16* o = (__nv_bfloat16*)out;
  if (w.fmt == QFMT_OIL8) dequant_rows_kernel<QFMT_OIL8><<<(int)g, 256, 0, stream>>>(w, ids, tokens, o, ld_out);
  else if (w.fmt == QFMT_OIL4) dequant_rows_kernel<QFMT_OIL4><<<(int)g, 256, 0, stream>>>(w, ids, tokens, o, ld_out);
  else if (w.fmt == QFMT_I2S) dequant_rows_kernel<QFMT_I2S><<<(int)g, 256, 0, stream>>>(w, ids, tokens, o, ld_out);
  else MB_REQUIRE(false, "dequant_gather_rows: unknown weight format");
  count_launch();
  check_launch();
}

}  // namespace mb
