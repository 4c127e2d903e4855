// Flash attention backward on tcgen05 tensor cores (head_dim 128).
//
// One CTA owns a 128-row K/V tile of one (batch, kv head) and walks the 64-row query tiles that
// can see it (all query heads of the GQA group). Everything is computed transposed so that one
// thread owns one kv row:
//     S^T  = K Q^T            dP^T = V dO^T                       (TMEM, 64 columns each)
//     P^T  = exp2(S^T*c - lse)        dS^T = P^T o (dP^T - delta) * scale   (registers -> TMEM as bf16 pairs;
//                                                                  dS^T also -> smem)
//     dV  += P^T dO           dK  += dS^T Q                        (A operand from TMEM; 128 columns each)
//     dQ^T = K^T dS^T                                              (TMEM, 64 columns) -> fp32 bulk reductions
// P^T and dS^T are the A operands of the dV / dK products and stay in tensor memory (32 columns each):
// the five products of a step and the compute warps' stores together asked for more than the 128 bytes
// per clock that shared memory delivers, and taking P^T (store + operand read) and the dS^T operand read
// of dK out of shared memory made the whole backward 5-8 % faster.
// The same shared tiles serve as K-major operands in one product and MN-major in another, so
// nothing is transposed in memory. Two compute warpgroups split the 64 query columns of a step
// (32 each), so every SM sub-partition has two warps to hide TMEM-load and exp latency behind one
// another. Q / dO tiles go through a three-stage ring so the load of step n+2 is issued while
// step n computes (with two stages its latency sat on the critical path), and the MMA thread polls
// "scores of the next step can be issued" and "dV/dK/dQ of this step can be issued" independently
// instead of waiting for them in a fixed order. dQ is accumulated in an fp32 scratch buffer with bulk tensor reductions and converted
// to bf16 by a second kernel. Replaces the reference's four O(S^2 D) scalar loops
// (src/autograd.cpp:463-584).
#include "api.h"
#include "common.cuh"
#include "host_util.h"
#include "tc.cuh"

#include <type_traits>

namespace mb {

CUtensorMap make_bshd_map(const void* base, int batch, int seq, int nheads, int head_dim, long long tok_stride,
                          int box_rows);

namespace {

constexpr int BW_THREADS = 320;  // loader warp, MMA warp, two compute warpgroups
constexpr int BW_QH = 32;        // query columns per compute warpgroup
constexpr int BW_KV = 128;  // kv rows per CTA
constexpr int BW_Q = 64;    // query rows per step
constexpr int BW_D = 128;

struct BwCfg {
  static constexpr int KV_BYTES = BW_KV * BW_D * 2;      // 32 KB, two 64-wide chunks of [128 x 128 B]
  static constexpr int QT_BYTES = BW_Q * BW_D * 2;       // 16 KB, two chunks of [64 x 128 B]
  static constexpr int STAGE_BYTES = 2 * QT_BYTES;       // Q + dO
  static constexpr int STAGES = 3;
  static constexpr int PT_BYTES = BW_KV * BW_Q * 2;      // 16 KB
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = KV_BYTES;
  static constexpr int OFF_ST = 2 * KV_BYTES;
  static constexpr int OFF_DST = OFF_ST + STAGES * STAGE_BYTES;   // dS^T, B operand of the dQ^T product
  static constexpr int OFF_DQ = OFF_DST + PT_BYTES;      // [8 warps][32 q][32 d] fp32 staging for the dQ reduce
  static constexpr int OFF_BAR = OFF_DQ + BW_Q * BW_D * 4;
  static constexpr int NUM_BARS = 12;
  static constexpr int SMEM_BYTES = OFF_BAR + NUM_BARS * 8 + 16 + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_ST = 0, COL_DPT = 64, COL_DV = 128, COL_DK = 256, COL_DQT = 384;
  static constexpr int COL_PT = 448, COL_DST = 480;   // P^T and dS^T as bf16 pairs: A operands of the dV / dK products
};

__global__ void __launch_bounds__(BW_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
              const __grid_constant__ CUtensorMap tm_dq, const float* __restrict__ lse,
              const float* __restrict__ delta,
              __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, long long dkv_tok_stride, int seq,
              int heads, int kv_heads, int causal, float scale, float scale_log2, const int* __restrict__ rope_pos,
              const float2* __restrict__ rope_cs, int rope_max_pos, int* status) {
  using Cfg = BwCfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars;         // K and V landed
  uint64_t* q_full = bars + 1;      // [3] Q and dO of a step landed
  uint64_t* q_empty = bars + 4;     // [3] the MMAs reading that stage completed
  uint64_t* s_full = bars + 7;      // S^T and dP^T of a step computed
  uint64_t* sp_free = bars + 8;     // compute threads hold S^T/dP^T in registers
  uint64_t* pds_full = bars + 9;    // P^T and dS^T written to shared memory
  uint64_t* mma_done = bars + 10;   // dV, dK, dQ^T products of a step completed
  uint64_t* dq_free = bars + 11;    // compute threads drained dQ^T
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + Cfg::NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvt = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int group = heads / kv_heads;
  const int kv0 = kvt * BW_KV;
  const int n_qt = (seq + BW_Q - 1) / BW_Q;
  const int i_start = causal ? kv0 / BW_Q : 0;
  const int per_head = n_qt - i_start;
  const int N = group * per_head;  // steps of this CTA

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(sp_free, 256);
    mbar_init(pds_full, 256);
    mbar_init(mma_done, 1);
    mbar_init(dq_free, 256);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do);
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
    // ------------------------------------------------------------------ loader
    if (lane == 0 && N > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * Cfg::KV_BYTES);
      for (int c = 0; c < 2; ++c) {
        tma_load_4d(smem + Cfg::OFF_K + c * (BW_KV * 128), &tm_k, kv_full, c * 64, hkv, kv0, b);
        tma_load_4d(smem + Cfg::OFF_V + c * (BW_KV * 128), &tm_v, kv_full, c * 64, hkv, kv0, b);
      }
      for (int n = 0; n < N; ++n) {
        const int st = n % Cfg::STAGES;
        const uint32_t ph = (n / Cfg::STAGES) & 1;
        if (!mbar_wait(&q_empty[st], ph ^ 1, abort_flag, status, 21)) break;
        const int h = hkv * group + n / per_head;
        const int q0 = (i_start + n % per_head) * BW_Q;
        mbar_arrive_expect_tx(&q_full[st], Cfg::STAGE_BYTES);
        uint8_t* sq = smem + Cfg::OFF_ST + st * Cfg::STAGE_BYTES;
        uint8_t* sdo = sq + Cfg::QT_BYTES;
        for (int c = 0; c < 2; ++c) {
          tma_load_4d(sq + c * (BW_Q * 128), &tm_q, &q_full[st], c * 64, h, q0, b);
          tma_load_4d(sdo + c * (BW_Q * 128), &tm_do, &q_full[st], c * 64, h, q0, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && N > 0) {
      constexpr uint32_t IDESC_ST = umma_idesc_bf16(BW_KV, BW_Q, false, false);   // S^T, dP^T
      constexpr uint32_t IDESC_ACC = umma_idesc_bf16(BW_KV, BW_D, false, true);   // dV, dK
      constexpr uint32_t IDESC_DQT = umma_idesc_bf16(BW_D, BW_Q, true, true);     // dQ^T
      const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K);
      const uint32_t v_addr = smem_u32(smem + Cfg::OFF_V);
      const uint32_t st_addr = smem_u32(smem + Cfg::OFF_ST);
      const uint32_t dst_addr = smem_u32(smem + Cfg::OFF_DST);
      auto issue_scores = [&](int n) {
        const uint32_t qa = st_addr + (n % Cfg::STAGES) * Cfg::STAGE_BYTES;
        const uint32_t doa = qa + Cfg::QT_BYTES;
#pragma unroll
        for (int k = 0; k < BW_D / 16; ++k) {
          const int c = k >> 2, kk = k & 3;
          umma_f16(tmem_base + Cfg::COL_ST, umma_desc_sw128(k_addr + c * (BW_KV * 128) + kk * 32, 0, 1024),
                   umma_desc_sw128(qa + c * (BW_Q * 128) + kk * 32, 0, 1024), IDESC_ST, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BW_D / 16; ++k) {
          const int c = k >> 2, kk = k & 3;
          umma_f16(tmem_base + Cfg::COL_DPT, umma_desc_sw128(v_addr + c * (BW_KV * 128) + kk * 32, 0, 1024),
                   umma_desc_sw128(doa + c * (BW_Q * 128) + kk * 32, 0, 1024), IDESC_ST, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, status, 22);
      if (ok) ok = mbar_wait(&q_full[0], 0, abort_flag, status, 23);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      // Two independent streams of work share this thread: the scores of step ns (need Q/dO of
      // that step and the S/dP accumulators, which the compute threads release once per step) and
      // the dV/dK/dQ products of step nm (need P/dS in shared memory and the drained dQ
      // accumulator). Each is issued the moment its inputs are ready.
      int ns = 1, nm = 0;
      long long t_idle = clock64();
      while (ok && nm < N) {
        bool progressed = false;
        if (ns < N && mbar_test_wait(&q_full[ns % Cfg::STAGES], (ns / Cfg::STAGES) & 1) &&
            mbar_test_wait(sp_free, (ns - 1) & 1)) {
          tc_fence_after();
          issue_scores(ns);
          ++ns;
          progressed = true;
        }
        if (mbar_test_wait(pds_full, nm & 1) && (nm == 0 || mbar_test_wait(dq_free, (nm - 1) & 1))) {
          tc_fence_after();
          const uint32_t qa = st_addr + (nm % Cfg::STAGES) * Cfg::STAGE_BYTES;
          const uint32_t doa = qa + Cfg::QT_BYTES;
#pragma unroll
          for (int k = 0; k < BW_Q / 16; ++k)  // dV += P^T dO, P^T from tensor memory
            umma_f16_ts(tmem_base + Cfg::COL_DV, tmem_base + Cfg::COL_PT + k * 8,
                        umma_desc_sw128(doa + k * 2048, BW_Q * 128, 1024), IDESC_ACC, (nm > 0 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < BW_Q / 16; ++k)  // dK += dS^T Q, dS^T from tensor memory
            umma_f16_ts(tmem_base + Cfg::COL_DK, tmem_base + Cfg::COL_DST + k * 8,
                        umma_desc_sw128(qa + k * 2048, BW_Q * 128, 1024), IDESC_ACC, (nm > 0 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < BW_KV / 16; ++k)  // dQ^T = K^T dS^T
            umma_f16(tmem_base + Cfg::COL_DQT, umma_desc_sw128(k_addr + k * 2048, BW_KV * 128, 1024),
                     umma_desc_sw128(dst_addr + k * 2048, BW_KV * 128, 1024), IDESC_DQT, k > 0 ? 1u : 0u);
          umma_commit(mma_done);
          umma_commit(&q_empty[nm % Cfg::STAGES]);
          ++nm;
          progressed = true;
        }
        if (progressed) {
          t_idle = clock64();
        } else if (*abort_flag) {
          ok = false;
        } else if (clock64() - t_idle > MB_WAIT_LIMIT_CYCLES) {
          *abort_flag = 1;
          if (status) atomicCAS(status, 0, ST_TIMEOUT | (24 << 16));
          ok = false;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    const int quarter = warp & 3;        // TMEM lane quarter this warp may read
    const int wg = (warp - 2) >> 2;      // 0/1: query columns [32 wg, 32 wg + 32) of every step
    const int cw = warp - 2;             // 0..7
    const int r = quarter * 32 + lane;   // kv row of this thread; also the d row of dQ^T
    const int kv_row = kv0 + r;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;

    float* dq_stage = reinterpret_cast<float*>(smem + Cfg::OFF_DQ) + cw * (BW_QH * 32);
    // dQ^T of step n is in TMEM: lane = d, column = q. Draining it has two halves. fetch_dq copies this
    // warp's 32 d-rows x 32 q-columns into registers and frees the accumulator (the MMA thread waits for
    // that before the next dQ product); store_dq transposes them into a [32 q][32 d] fp32 tile in shared
    // memory and adds it to the fp32 dQ buffer with one bulk tensor reduction (no per-element atomics).
    // Only the first half sits between a step's arithmetic and its P / dS stores; the second runs after
    // the stores, while the tensor pipe works on the step's products.
    uint32_t dq_regs[32];
    auto fetch_dq = [&]() {
      tmem_ld32(tmem_base + Cfg::COL_DQT + wg * BW_QH + lane_sel, dq_regs);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dq_free);
    };
    auto store_dq = [&](int n) {
      const int h = hkv * group + n / per_head;
      const int q0 = (i_start + n % per_head) * BW_Q;
      if (lane == 0) tma_store_wait_read0();  // the previous reduction has finished reading the staging tile
      __syncwarp();
#pragma unroll
      for (int q = 0; q < BW_QH; ++q) dq_stage[q * 32 + lane] = __uint_as_float(dq_regs[q]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && q0 + wg * BW_QH < seq) {   // a box wholly past the sequence end is not issued
        tma_reduce_add_4d(&tm_dq, dq_stage, quarter * 32, h, q0 + wg * BW_QH, b);
        tma_store_commit();
      }
    };

    // lse and delta of a step's 32 query columns are the same for every thread of the warp: each thread
    // reads them itself with eight uniform 16-byte loads per array (one L1 transaction per load, issued
    // before the wait for the scores) instead of receiving them through 64 shuffles per step, which kept
    // the shuffle unit busy for 512 cycles of a 1280-cycle step. delta arrives as -delta * scale.
    const bool vec_rows = (seq & 3) == 0 && (reinterpret_cast<uintptr_t>(lse) & 15) == 0 &&
                          (reinterpret_cast<uintptr_t>(delta) & 15) == 0;
    const uint64_t sc2 = f32x2(scale_log2, scale_log2), s2 = f32x2(scale, scale);
    const uint64_t nlog2 = f32x2(-LOG2E, -LOG2E);
    for (int n = 0; n < N && ok; ++n) {
      const int h = hkv * group + n / per_head;
      const int q0 = (i_start + n % per_head) * BW_Q;
      const int qc0 = q0 + wg * BW_QH;   // first query row of this warpgroup's columns
      const long long off = ((long long)b * heads + h) * seq + qc0;
      const bool tail = qc0 + BW_QH > seq;
      float nl[BW_QH], nd[BW_QH];        // -lse * log2(e) and -delta * scale of the 32 query columns
      if (vec_rows && !tail) {
#pragma unroll
        for (int c = 0; c < BW_QH / 4; ++c) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(lse + off) + c);
          const float4 g = __ldg(reinterpret_cast<const float4*>(delta + off) + c);
          nl[4 * c] = a.x; nl[4 * c + 1] = a.y; nl[4 * c + 2] = a.z; nl[4 * c + 3] = a.w;
          nd[4 * c] = g.x; nd[4 * c + 1] = g.y; nd[4 * c + 2] = g.z; nd[4 * c + 3] = g.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < BW_QH; ++i) {
          const bool in = qc0 + i < seq;
          nl[i] = in ? __ldg(lse + off + i) : 0.f;
          nd[i] = in ? __ldg(delta + off + i) : 0.f;
        }
      }

      ok = mbar_wait(s_full, n & 1, abort_flag, status, 28);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[32], dr[32];
      tmem_ld32(tmem_base + Cfg::COL_ST + wg * BW_QH + lane_sel, sr);
      tmem_ld32(tmem_base + Cfg::COL_DPT + wg * BW_QH + lane_sel, dr);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(sp_free);
      float* s = reinterpret_cast<float*>(&sr[0]);
      float* d = reinterpret_cast<float*>(&dr[0]);
      // P = exp2(S c - lse log2 e), dS = P (dP scale - delta scale), on packed fp32 pairs.
      const bool masked = tail || (causal && (qc0 < kv0 + BW_KV));
      auto body = [&](auto mask_tag) {
        constexpr bool MASK = decltype(mask_tag)::value;
#pragma unroll
        for (int i = 0; i < BW_QH; i += 2) {
          float e0, e1;
          f32x2_unpack(fma_f32x2(f32x2(s[i], s[i + 1]), sc2, mul_f32x2(f32x2(nl[i], nl[i + 1]), nlog2)), e0, e1);
          float p0 = fast_exp2(e0), p1 = fast_exp2(e1);
          if (MASK) {
            if ((causal && kv_row > qc0 + i) || qc0 + i >= seq) p0 = 0.f;
            if ((causal && kv_row > qc0 + i + 1) || qc0 + i + 1 >= seq) p1 = 0.f;
          }
          const uint64_t dd = fma_f32x2(f32x2(d[i], d[i + 1]), s2, f32x2(nd[i], nd[i + 1]));
          f32x2_unpack(mul_f32x2(f32x2(p0, p1), dd), d[i], d[i + 1]);
          s[i] = p0;
          s[i + 1] = p1;
        }
      };
      if (masked) body(std::true_type{}); else body(std::false_type{});
      if (n > 0) {
        ok = mbar_wait(mma_done, (n - 1) & 1, abort_flag, status, 29);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        fetch_dq();
      }
      // P^T and dS^T go back to tensor memory as bf16 pairs (A operands of the dV and dK products, which
      // then read only dO / Q from shared memory); dS^T is also the B operand of the dQ^T product and
      // is stored to shared memory for that.
      uint32_t pp[16], dd[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        pp[c] = pack_bf16x2(s[2 * c], s[2 * c + 1]);
        dd[c] = pack_bf16x2(d[2 * c], d[2 * c + 1]);
      }
      tmem_st16(tmem_base + Cfg::COL_PT + wg * (BW_QH / 2) + lane_sel, pp);
      tmem_st16(tmem_base + Cfg::COL_DST + wg * (BW_QH / 2) + lane_sel, dd);
      uint8_t* dst = smem + Cfg::OFF_DST;
#pragma unroll
      for (int c = 0; c < BW_QH / 8; ++c)
        *reinterpret_cast<uint4*>(dst + sw128_offset(r, wg * (BW_QH / 8) + c)) =
            make_uint4(dd[4 * c], dd[4 * c + 1], dd[4 * c + 2], dd[4 * c + 3]);
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_full);
      if (n > 0) store_dq(n - 1);
    }
    if (ok && N > 0) {
      ok = mbar_wait(mma_done, (N - 1) & 1, abort_flag, status, 30);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        fetch_dq();
        store_dq(N - 1);
        if (lane == 0) tma_store_wait0();  // all dQ reductions of this warp have landed
        // this thread's kv row of dV (warpgroup 0) or dK (warpgroup 1)
        const long long row_off = ((long long)b * seq + kv_row) * dkv_tok_stride + (long long)hkv * BW_D;
        const int which = wg;
        __nv_bfloat16* out = (which == 0 ? dv : dk) + row_off;
        const uint32_t col = which == 0 ? Cfg::COL_DV : Cfg::COL_DK;
        if (which == 1 && rope_cs != nullptr) {
          // dK leaves rotated back by the row's position (the gradient of the un-rotated projection):
          // dx1 = dy1 cos + dy2 sin, dx2 = dy2 cos - dy1 sin for the pair (d, d + 64).
          int p = kv_row < seq ? __ldg(rope_pos + (long long)b * seq + kv_row) : 0;
          p = min(max(p, 0), rope_max_pos - 1);
          const float4* cs_row = reinterpret_cast<const float4*>(rope_cs + (long long)p * 64);
#pragma unroll 1
          for (int cc = 0; cc < 2; ++cc) {
            uint32_t lo[32], hi[32];
            tmem_ld32(tmem_base + col + cc * 32 + lane_sel, lo);
            tmem_ld32(tmem_base + col + 64 + cc * 32 + lane_sel, hi);
            tmem_ld_wait();
            if (kv_row < seq) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t a[4], c2[4];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                  const float4 t = __ldg(cs_row + ((cc * 32 + 8 * j + i) >> 1));  // (cos, sin) of two pairs
                  const float x0 = __uint_as_float(lo[8 * j + i]), x1 = __uint_as_float(lo[8 * j + i + 1]);
                  const float y0 = __uint_as_float(hi[8 * j + i]), y1 = __uint_as_float(hi[8 * j + i + 1]);
                  a[i >> 1] = pack_bf16x2(x0 * t.x + y0 * t.y, x1 * t.z + y1 * t.w);
                  c2[i >> 1] = pack_bf16x2(y0 * t.x - x0 * t.y, y1 * t.z - x1 * t.w);
                }
                *reinterpret_cast<uint4*>(out + cc * 32 + 8 * j) = make_uint4(a[0], a[1], a[2], a[3]);
                *reinterpret_cast<uint4*>(out + 64 + cc * 32 + 8 * j) = make_uint4(c2[0], c2[1], c2[2], c2[3]);
              }
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < BW_D / 32; ++c) {
            uint32_t a[32];
            tmem_ld32(tmem_base + col + c * 32 + lane_sel, a);
            tmem_ld_wait();
            if (kv_row < seq) {
              uint4* p4 = reinterpret_cast<uint4*>(out + c * 32);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(a[8 * i + 0]), __uint_as_float(a[8 * i + 1]));
                v.y = pack_bf16x2(__uint_as_float(a[8 * i + 2]), __uint_as_float(a[8 * i + 3]));
                v.z = pack_bf16x2(__uint_as_float(a[8 * i + 4]), __uint_as_float(a[8 * i + 5]));
                v.w = pack_bf16x2(__uint_as_float(a[8 * i + 6]), __uint_as_float(a[8 * i + 7]));
                p4[i] = v;
              }
            }
          }
        }
      }
    } else if (N == 0 && kv_row < seq && wg == 0) {
      // no query can see this tile (cannot happen with causal self-attention, kept for safety)
      const long long row_off = ((long long)b * seq + kv_row) * dkv_tok_stride + (long long)hkv * BW_D;
      for (int i = 0; i < BW_D; ++i) {
        dv[row_off + i] = __float2bfloat16(0.f);
        dk[row_off + i] = __float2bfloat16(0.f);
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
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// Prologue of the backward pass, one pass over O and dO: delta[b,h,s] = -scale * sum_d dO[b,s,h,d] *
// O[b,s,h,d] (the form the main kernel adds to dP * scale), and the fp32 dQ accumulator row of the same
// (b,s,h) is zeroed (it used to be a separate memset). Sixteen lanes own one row of 128 columns, eight
// columns each; every thread works on two rows so that four 16-byte loads are in flight.
__global__ void __launch_bounds__(256)
fa_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                   float* __restrict__ dq_accum, long long rows, int seq, int heads, float scale) {
  const int sub = threadIdx.x & 15;
  const long long r0 = ((long long)blockIdx.x * 16 + (threadIdx.x >> 4)) * 2;
  float acc[2] = {0.f, 0.f};
  bf16x8 ov[2], gv[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const long long row = r0 + k;
    if (row < rows) {
      ov[k] = ldg8(o, row * BW_D + sub * 8);
      gv[k] = ldg8(dout, row * BW_D + sub * 8);
    } else {
      ov[k] = bf16x8{};
      gv[k] = bf16x8{};
    }
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const long long row = r0 + k;
    float a[8], g[8];
    unpack8(ov[k], a);
    unpack8(gv[k], g);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[k] += a[i] * g[i];
#pragma unroll
    for (int m = 8; m >= 1; m >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], m);
    if (row < rows) {
      float4* z = reinterpret_cast<float4*>(dq_accum + row * BW_D + sub * 8);
      z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (sub == 0) {
        const long long bs = row / heads;  // b*seq + s
        const int h = (int)(row % heads);
        const long long bb = bs / seq, ss = bs % seq;
        delta[(bb * heads + h) * seq + ss] = -scale * acc[k];
      }
    }
  }
}

// dst[r, 0:cols] (row stride dst_stride) = bf16(src[r, 0:cols]); cols is a multiple of 4.
__global__ void cast_rows_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows,
                                 int cols, long long dst_stride) {
  const int per_row = cols >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c = (int)(i % per_row) * 4;
    const float4 v = *reinterpret_cast<const float4*>(src + r * cols + c);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dst + r * dst_stride + c) = o;
  }
}

// The same conversion with the rotary embedding undone on the way (heads of 128, pairs (d, d + 64)):
// dst = bf16(R(-pos[r]) src). One thread owns four pairs of one head.
__global__ void cast_rows_rope_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows,
                                      int heads, long long dst_stride, const int* __restrict__ pos,
                                      const float2* __restrict__ cs, int max_pos) {
  const int per_row = heads * 16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int w = (int)(i % per_row);
    const int h = w >> 4, c = (w & 15) * 4;
    const int p = min(max(__ldg(pos + r), 0), max_pos - 1);
    const float4* t4 = reinterpret_cast<const float4*>(cs + (long long)p * 64 + c);
    const float4 t0 = __ldg(t4), t1 = __ldg(t4 + 1);   // (cos, sin) of pairs c, c+1 | c+2, c+3
    const float* s = src + (r * heads + h) * BW_D;
    const float4 x = *reinterpret_cast<const float4*>(s + c);
    const float4 y = *reinterpret_cast<const float4*>(s + 64 + c);
    __nv_bfloat16* d = dst + r * dst_stride + h * BW_D;
    uint2 lo, hi;
    lo.x = pack_bf16x2(x.x * t0.x + y.x * t0.y, x.y * t0.z + y.y * t0.w);
    lo.y = pack_bf16x2(x.z * t1.x + y.z * t1.y, x.w * t1.z + y.w * t1.w);
    hi.x = pack_bf16x2(y.x * t0.x - x.x * t0.y, y.y * t0.z - x.y * t0.w);
    hi.y = pack_bf16x2(y.z * t1.x - x.z * t1.y, y.w * t1.z - x.w * t1.w);
    *reinterpret_cast<uint2*>(d + c) = lo;
    *reinterpret_cast<uint2*>(d + 64 + c) = hi;
  }
}

}  // namespace

void flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                    void* dq, void* dk, void* dv, float* dq_accum, float* delta, int batch, int seq, int heads,
                    int kv_heads, int head_dim, bool causal, float scale, int* status, cudaStream_t stream) {
  flash_attn_bwd_strided(q, k, v, o, dout, lse, dq, dk, dv, dq_accum, delta, batch, seq, heads, kv_heads, head_dim,
                         (long long)heads * head_dim, (long long)kv_heads * head_dim, (long long)heads * head_dim,
                         (long long)kv_heads * head_dim, causal, scale, status, stream, nullptr, nullptr, 0);
}

void flash_attn_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* dout,
                            const float* lse, void* dq, void* dk, void* dv, float* dq_accum, float* delta, int batch,
                            int seq, int heads, int kv_heads, int head_dim, long long q_tok_stride,
                            long long kv_tok_stride, long long dq_tok_stride, long long dkv_tok_stride, bool causal,
                            float scale, int* status, cudaStream_t stream, const int* rope_pos, const float* rope_cs,
                            int rope_max_pos) {
  MB_REQUIRE(head_dim == 128, "flash_attn_bwd: head_dim must be 128");
  MB_REQUIRE(heads % kv_heads == 0, "flash_attn_bwd: heads must be a multiple of kv_heads");
  if (batch == 0 || seq == 0) return;
  const long long rows = (long long)batch * seq * heads;
  MB_REQUIRE(rope_cs == nullptr || (rope_pos != nullptr && rope_max_pos > 0), "flash_attn_bwd: rope table without positions");
  fa_bwd_prep_kernel<<<(unsigned)ceil_div(rows, 32), 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout,
                                                                     delta, dq_accum, rows, seq, heads, scale);
  count_launch();
  check_launch();
  const CUtensorMap tq = make_bshd_map(q, batch, seq, heads, head_dim, q_tok_stride, BW_Q);
  const CUtensorMap tdo = make_bshd_map(dout, batch, seq, heads, head_dim, (long long)heads * head_dim, BW_Q);
  const CUtensorMap tk = make_bshd_map(k, batch, seq, kv_heads, head_dim, kv_tok_stride, BW_KV);
  const CUtensorMap tv = make_bshd_map(v, batch, seq, kv_heads, head_dim, kv_tok_stride, BW_KV);
  CUtensorMap tdq;
  {
    uint64_t dims[4] = {(uint64_t)head_dim, (uint64_t)heads, (uint64_t)seq, (uint64_t)batch};
    uint64_t strides[3] = {(uint64_t)head_dim * 4, (uint64_t)heads * head_dim * 4,
                           (uint64_t)seq * heads * head_dim * 4};
    uint32_t box[4] = {32, 1, BW_QH, 1};
    tdq = make_tensor_map(dq_accum, TmaDType::F32, 4, dims, strides, box, false);
  }
  static bool configured = false;
  if (!configured) {
    MB_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwCfg::SMEM_BYTES));
    configured = true;
  }
  const dim3 grid((seq + BW_KV - 1) / BW_KV, kv_heads, batch);
  fa_bwd_kernel<<<grid, BW_THREADS, BwCfg::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, tdq, lse, delta,
                                                                 (__nv_bfloat16*)dk, (__nv_bfloat16*)dv,
                                                                 dkv_tok_stride, seq, heads, kv_heads, causal ? 1 : 0, scale,
                                                                 scale * 1.4426950408889634f, rope_pos,
                                                                 reinterpret_cast<const float2*>(rope_cs), rope_max_pos, status);
  count_launch();
  check_launch();
  {
    const long long tok = (long long)batch * seq;
    const int cols = heads * head_dim;
    long long g = (tok * (cols / 4) + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    if (g > cap) g = cap;
    if (rope_cs != nullptr)
      cast_rows_rope_kernel<<<(int)g, 256, 0, stream>>>(dq_accum, (__nv_bfloat16*)dq, tok, heads, dq_tok_stride, rope_pos,
                                                        reinterpret_cast<const float2*>(rope_cs), rope_max_pos);
    else
      cast_rows_kernel<<<(int)g, 256, 0, stream>>>(dq_accum, (__nv_bfloat16*)dq, tok, cols, dq_tok_stride);
    count_launch();
    check_launch();
  }
}

}  // namespace mb
