// Flash attention forward, head_dim 128, second generation: persistent CTAs, 128 x 128 score tiles,
// P kept in tensor memory.
//
// Differences from fa_fwd_kernel (attention_fwd.cu), each aimed at the idle tensor pipe that kernel
// shows (SM busy ~30-40 %):
//   * kv tiles of 128 rows instead of 64: every S = Q K^T product is a 128 x 128 x 128 MMA chain whose
//     shared-memory operand traffic matches the tensor rate (a 64-wide B operand re-reads the A tile
//     twice as often), and the fixed costs per step (barrier round trips, TMEM loads, fences) are paid
//     half as often;
//   * the probabilities never touch shared memory: the softmax warpgroup converts its row of S to bf16
//     and stores it back into the first half of S's own TMEM columns; the PV product takes its A
//     operand from TMEM (tcgen05.mma with a tensor-memory A). No proxy fence, no swizzled stores, and
//     the PV product reads only V from shared memory;
//   * the CTA is persistent over (batch, head, 256-row query block) work items, heaviest causal blocks
//     first: the epilogue of one item overlaps the first score products of the next, and barrier /
//     TMEM set-up is paid once per SM instead of once per 256 query rows;
//   * K and V travel in separate rings (2 and 3 stages of 32 KB), so a K tile is released as soon as
//     both score products that read it were issued, one full step before its V tile.
// Warps: 0 = K/V loader, 1 = MMA issuer + TMEM owner, 2 = Q loader, 3 idle, 4-7 = softmax of query
// tile 0, 8-11 = softmax of tile 1. Two 128-row query tiles per work item ping-pong as before: while one
// tile's warpgroup does its softmax the tensor pipe works for the other tile. (Splitting every row over
// two threads, 16 softmax warps with a named barrier per step, measured slower: 415 against
// 625 TFLOP/s at batch 8, sequence 2048.)
// TMEM (512 columns): S0 | S1 (128 fp32 columns each, P aliased on their first 64) | O0 | O1 (128 each).
#include "api.h"
#include "host_util.h"
#include "tc.cuh"

namespace mb {

CUtensorMap make_bshd_map(const void* base, int batch, int seq, int nheads, int head_dim, long long tok_stride,
                          int box_rows);

namespace {

constexpr int F2_THREADS = 384;   // three warpgroups: service warps, softmax of tile 0, softmax of tile 1
constexpr int F2_BM = 128;
constexpr int F2_BN = 128;
constexpr int F2_D = 128;
constexpr int F2_KS = 2;   // K stages
constexpr int F2_VS = 3;   // V stages

struct F2Cfg {
  static constexpr int TILE_BYTES = 128 * F2_D * 2;        // 32 KB: two 64-column chunks of [128 rows x 128 B]
  static constexpr int OFF_Q = 0;                          // two query tiles
  static constexpr int OFF_K = 2 * TILE_BYTES;
  static constexpr int OFF_V = OFF_K + F2_KS * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_V + F2_VS * TILE_BYTES;
  static constexpr int NUM_BARS = 4 + 2 * F2_KS + 2 * F2_VS + 6;
  static constexpr int SMEM_BYTES = OFF_BAR + NUM_BARS * 8 + 16 + 1024;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");
  static constexpr int COL_S = 0;     // S_t at t * 128
  static constexpr int COL_O = 256;   // O_t at 256 + t * 128
};

struct F2Item {
  int b, h, q0, n_qt, J[2], Jmax;
};
// Work item w: items are ordered by query block, last (heaviest under the causal mask) block first.
__device__ __forceinline__ F2Item f2_item(int w, int n_qb, int heads, int batch, int seq, int causal) {
  F2Item it;
  const int bh = w % (heads * batch);
  const int qblk = n_qb - 1 - w / (heads * batch);
  it.h = bh % heads;
  it.b = bh / heads;
  it.q0 = qblk * 2 * F2_BM;
  it.n_qt = (it.q0 + F2_BM < seq) ? 2 : 1;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int hi = causal ? min(seq, it.q0 + (t + 1) * F2_BM) : seq;
    it.J[t] = (t < it.n_qt) ? (hi + F2_BN - 1) / F2_BN : 0;
  }
  it.Jmax = max(it.J[0], it.J[1]);
  return it;
}

__global__ void __launch_bounds__(F2_THREADS, 1)
fa_fwd2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, __nv_bfloat16* __restrict__ o, float* __restrict__ lse, int seq,
               int heads, int kv_heads, long long o_tok_stride, int causal, float scale_log2, int n_items, int n_qb,
               int batch, int* status) {
  using Cfg = F2Cfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;                 // [2]
  uint64_t* q_free = bars + 2;             // [2]
  uint64_t* k_full = bars + 4;             // [KS]
  uint64_t* k_empty = k_full + F2_KS;
  uint64_t* v_full = k_empty + F2_KS;      // [VS]
  uint64_t* v_empty = v_full + F2_VS;
  uint64_t* s_full = v_empty + F2_VS;      // [2]
  uint64_t* p_full = s_full + 2;           // [2]
  uint64_t* o_full = p_full + 2;           // [2]
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(o_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = heads / kv_heads;

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(&q_full[t], 1);
      mbar_init(&q_free[t], 1);
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
      mbar_init(&o_full[t], 1);
    }
    for (int s = 0; s < F2_KS; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < F2_VS; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 2) {
    // ------------------------------------------------------------------ Q loader
    if (lane == 0) {
      uint32_t n_q[2] = {0, 0};   // loads issued per tile (phase of q_free / q_full)
      for (int w = blockIdx.x; w < n_items; w += gridDim.x) {
        const F2Item it = f2_item(w, n_qb, heads, batch, seq, causal);
        bool ok = true;
        for (int t = 0; t < it.n_qt && ok; ++t) {
          if (it.J[t] == 0) continue;
          if (!mbar_wait(&q_free[t], (n_q[t] & 1) ^ 1, abort_flag, status, 81)) { ok = false; break; }
          mbar_arrive_expect_tx(&q_full[t], Cfg::TILE_BYTES);
          for (int c = 0; c < 2; ++c)
            tma_load_4d(smem + Cfg::OFF_Q + t * Cfg::TILE_BYTES + c * (F2_BM * 128), &tm_q, &q_full[t], c * 64, it.h,
                        it.q0 + t * F2_BM, it.b);
          ++n_q[t];
        }
        if (!ok) break;
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ K / V loader
    if (lane == 0) {
      uint32_t kc = 0, vc = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
        const F2Item it = f2_item(w, n_qb, heads, batch, seq, causal);
        const int hkv = it.h / group;
        for (int j = 0; j < it.Jmax; ++j) {
          {
            const int st = kc % F2_KS;
            if (!mbar_wait(&k_empty[st], ((kc / F2_KS) & 1) ^ 1, abort_flag, status, 82)) { ok = false; break; }
            mbar_arrive_expect_tx(&k_full[st], Cfg::TILE_BYTES);
            for (int c = 0; c < 2; ++c)
              tma_load_4d(smem + Cfg::OFF_K + st * Cfg::TILE_BYTES + c * (F2_BN * 128), &tm_k, &k_full[st], c * 64, hkv,
                          j * F2_BN, it.b);
            ++kc;
          }
          {
            const int st = vc % F2_VS;
            if (!mbar_wait(&v_empty[st], ((vc / F2_VS) & 1) ^ 1, abort_flag, status, 83)) { ok = false; break; }
            mbar_arrive_expect_tx(&v_full[st], Cfg::TILE_BYTES);
            for (int c = 0; c < 2; ++c)
              tma_load_4d(smem + Cfg::OFF_V + st * Cfg::TILE_BYTES + c * (F2_BN * 128), &tm_v, &v_full[st], c * 64, hkv,
                          j * F2_BN, it.b);
            ++vc;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_S = umma_idesc_bf16(F2_BM, F2_BN, false, false);
      constexpr uint32_t IDESC_O = umma_idesc_bf16(F2_BM, F2_D, false, true);
      const uint32_t q_addr = smem_u32(smem + Cfg::OFF_Q);
      const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K);
      const uint32_t v_addr = smem_u32(smem + Cfg::OFF_V);
      uint32_t kc = 0, vc = 0;              // K / V tiles consumed so far (ring position and phase)
      uint32_t n_q[2] = {0, 0}, n_p[2] = {0, 0};
      bool ok = true;
      auto issue_s = [&](int t, uint32_t kpos) {
        const uint32_t qa = q_addr + t * Cfg::TILE_BYTES;
        const uint32_t ka = k_addr + (kpos % F2_KS) * Cfg::TILE_BYTES;
#pragma unroll
        for (int k = 0; k < F2_D / 16; ++k) {
          const int c = k >> 2, kk = k & 3;
          umma_f16(tmem_base + Cfg::COL_S + t * 128, umma_desc_sw128(qa + c * (F2_BM * 128) + kk * 32, 0, 1024),
                   umma_desc_sw128(ka + c * (F2_BN * 128) + kk * 32, 0, 1024), IDESC_S, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
        const F2Item it = f2_item(w, n_qb, heads, batch, seq, causal);
        if (it.Jmax == 0) continue;
        // scores of step 0 for both tiles
        if (!mbar_wait(&k_full[kc % F2_KS], (kc / F2_KS) & 1, abort_flag, status, 84)) { ok = false; break; }
        for (int t = 0; t < 2 && ok; ++t) {
          if (it.J[t] == 0) continue;
          if (!mbar_wait(&q_full[t], n_q[t] & 1, abort_flag, status, 85)) { ok = false; break; }
          tc_fence_after();
          issue_s(t, kc);
          if (it.J[t] == 1) umma_commit(&q_free[t]);
        }
        if (!ok) break;
        umma_commit(&k_empty[kc % F2_KS]);   // every score product of kv tile 0 has been issued
        ++kc;
        for (int j = 0; j < it.Jmax && ok; ++j) {
          bool v_ready = false, k_ready = false;
          const bool have_next = j + 1 < it.Jmax;
          for (int t = 0; t < 2 && ok; ++t) {
            if (j >= it.J[t]) continue;
            if (!mbar_wait(&p_full[t], n_p[t] & 1, abort_flag, status, 86)) { ok = false; break; }
            ++n_p[t];
            if (!v_ready) {
              if (!mbar_wait(&v_full[vc % F2_VS], (vc / F2_VS) & 1, abort_flag, status, 87)) { ok = false; break; }
              v_ready = true;
            }
            tc_fence_after();
            const uint32_t va = v_addr + (vc % F2_VS) * Cfg::TILE_BYTES;
#pragma unroll
            for (int k = 0; k < F2_BN / 16; ++k)   // O_t += P_t(tmem) V
              umma_f16_ts(tmem_base + Cfg::COL_O + t * 128, tmem_base + Cfg::COL_S + t * 128 + k * 8,
                          umma_desc_sw128(va + k * 2048, F2_BN * 128, 1024), IDESC_O, (j > 0 || k > 0) ? 1u : 0u);
            if (j == it.J[t] - 1) umma_commit(&o_full[t]);
            if (j + 1 < it.J[t]) {
              if (!k_ready) {
                if (!mbar_wait(&k_full[kc % F2_KS], (kc / F2_KS) & 1, abort_flag, status, 88)) { ok = false; break; }
                tc_fence_after();
                k_ready = true;
              }
              issue_s(t, kc);               // overwrites S_t / P_t: ordered behind the PV product just issued
              if (j + 2 == it.J[t]) umma_commit(&q_free[t]);   // that was the tile's last score product
            }
          }
          if (!ok) break;
          umma_commit(&v_empty[vc % F2_VS]);
          ++vc;
          if (have_next) {
            umma_commit(&k_empty[kc % F2_KS]);
            ++kc;
          }
        }
        for (int t = 0; t < 2; ++t)
          if (it.J[t] > 0) ++n_q[t];
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax + epilogue
    const int sw = warp - 4;                 // 0..7
    const int t = sw >> 2;                   // query tile
    const int quarter = warp & 3;            // TMEM lane quarter this warp may access
    const int r = quarter * 32 + lane;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + Cfg::COL_S + t * 128 + lane_sel;
    const uint32_t t_o = tmem_base + Cfg::COL_O + t * 128 + lane_sel;
    uint32_t n_s = 0, n_o = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
      const F2Item it = f2_item(w, n_qb, heads, batch, seq, causal);
      const int Jt = it.J[t];
      if (Jt == 0) continue;
      const int q_row = it.q0 + t * F2_BM + r;
      float m_ref = 0.f, l = 0.f;
      for (int j = 0; j < Jt && ok; ++j) {
        ok = mbar_wait(&s_full[t], n_s & 1, abort_flag, status, 89);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++n_s;
        tc_fence_after();
        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, sr[c]);
        tmem_ld_wait();
        float* s = reinterpret_cast<float*>(&sr[0][0]);
        const int kv0 = j * F2_BN;
        const int limit = causal ? min(seq - 1, q_row) : seq - 1;
        if (kv0 + F2_BN - 1 > limit) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (kv0 + i > limit) s[i] = -INFINITY;
        }
        float mx4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
        for (int i = 4; i < 124; i += 8) {
          mx4[0] = fmax3(mx4[0], s[i], s[i + 1]);
          mx4[1] = fmax3(mx4[1], s[i + 2], s[i + 3]);
          mx4[2] = fmax3(mx4[2], s[i + 4], s[i + 5]);
          mx4[3] = fmax3(mx4[3], s[i + 6], s[i + 7]);
        }
        mx4[0] = fmax3(mx4[0], s[124], s[125]);
        mx4[1] = fmax3(mx4[1], s[126], s[127]);
        const float m_new = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
        float alpha = 1.f;
        bool need = false;
        if (j == 0) {
          m_ref = (m_new == -INFINITY) ? 0.f : m_new;
        } else if (m_new - m_ref > 8.f) {
          need = true;
          alpha = fast_exp2(m_ref - m_new);
          m_ref = m_new;
        }
        // S_t(j) complete implies PV_t(j-1) complete (same issuing thread, commit covers earlier MMAs):
        // O_t is quiescent until this warpgroup arrives on p_full, so a rescale can happen right here.
        if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t orr[32];
            tmem_ld32(t_o + c * 32, orr);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
            tmem_st32(t_o + c * 32, orr);
          }
        }
        // Packed fp32 pairs (fma.rn.f32x2 / add.rn.f32x2) halve the issue slots of the scale-and-shift
        // and of the row sum; the exponentials themselves run at the special-function rate of 16 per
        // clock per SM, which for two 128 x 128 tiles equals the tensor time of a step.
        const uint64_t sc2 = f32x2(scale_log2, scale_log2), nm2 = f32x2(-m_ref, -m_ref);
        uint64_t rs2[4] = {0ull, 0ull, 0ull, 0ull};
        uint32_t* pk = &sr[0][0];         // packed in place: pair i lands in word i / 2, behind the read position
#pragma unroll
        for (int i = 0; i < 128; i += 2) {
          float e0, e1;
          f32x2_unpack(fma_f32x2(f32x2(s[i], s[i + 1]), sc2, nm2), e0, e1);
          const float p0 = fast_exp2(e0), p1 = fast_exp2(e1);
          rs2[(i >> 1) & 3] = add_f32x2(rs2[(i >> 1) & 3], f32x2(p0, p1));
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
        float rs[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) f32x2_unpack(rs2[q], rs[2 * q], rs[2 * q + 1]);
        l = l * alpha + (((rs[0] + rs[1]) + (rs[2] + rs[3])) + ((rs[4] + rs[5]) + (rs[6] + rs[7])));
        tmem_st32(t_s, sr[0]);            // P_t: bf16 pairs over the first 64 columns of S_t
        tmem_st32(t_s + 32, sr[1]);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&p_full[t]);
      }
      if (!ok) break;
      ok = mbar_wait(&o_full[t], n_o & 1, abort_flag, status, 90);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++n_o;
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = o + ((long long)it.b * seq + q_row) * o_tok_stride + (long long)it.h * F2_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t orr[32];
        tmem_ld32(t_o + c * 32, orr);
        tmem_ld_wait();
        if (q_row < seq) {
          uint4* p4 = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(orr[8 * i + 0]) * inv_l, __uint_as_float(orr[8 * i + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(orr[8 * i + 2]) * inv_l, __uint_as_float(orr[8 * i + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(orr[8 * i + 4]) * inv_l, __uint_as_float(orr[8 * i + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(orr[8 * i + 6]) * inv_l, __uint_as_float(orr[8 * i + 7]) * inv_l);
            p4[i] = v;
          }
        }
      }
      if (q_row < seq && lse) lse[((long long)it.b * heads + it.h) * seq + q_row] = m_ref * 0.6931471805599453f + logf(l);
      // The TMEM loads above have completed (tmem_ld_wait); the next item's first PV product waits for
      // this warpgroup's next arrives on p_full, so O_t is not overwritten before it was read.
      tc_fence_before();
    }
  }

  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 10000000LL) {}
    __syncthreads();
  }
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

bool flash_attn_fwd2_supported(int head_dim, int seq) { return head_dim == 128 && seq >= 128; }

void flash_attn_fwd2_strided(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq,
                             int heads, int kv_heads, long long q_tok_stride, long long kv_tok_stride,
                             long long o_tok_stride, bool causal, float scale, int* status, cudaStream_t stream) {
  MB_REQUIRE(heads % kv_heads == 0, "flash_attn_fwd2: heads must be a multiple of kv_heads");
  MB_REQUIRE(q_tok_stride % 8 == 0 && kv_tok_stride % 8 == 0 && o_tok_stride % 8 == 0,
             "flash_attn_fwd2: token strides must be multiples of 8 elements");
  MB_REQUIRE((reinterpret_cast<uintptr_t>(o) & 15) == 0, "flash_attn_fwd2: output must be 16-byte aligned");
  if (batch == 0 || seq == 0) return;
  const CUtensorMap tq = make_bshd_map(q, batch, seq, heads, F2_D, q_tok_stride, F2_BM);
  const CUtensorMap tk = make_bshd_map(k, batch, seq, kv_heads, F2_D, kv_tok_stride, F2_BN);
  const CUtensorMap tv = make_bshd_map(v, batch, seq, kv_heads, F2_D, kv_tok_stride, F2_BN);
  const int n_qb = (seq + 2 * F2_BM - 1) / (2 * F2_BM);
  const int n_items = n_qb * heads * batch;
  static bool configured = false;
  if (!configured) {
    MB_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F2Cfg::SMEM_BYTES));
    configured = true;
  }
  const int grid_x = n_items < sm_count() ? n_items : sm_count();
  fa_fwd2_kernel<<<dim3(grid_x, 1, 1), F2_THREADS, F2Cfg::SMEM_BYTES, stream>>>(
      tq, tk, tv, (__nv_bfloat16*)o, lse, seq, heads, kv_heads, o_tok_stride, causal ? 1 : 0,
      scale * 1.4426950408889634f, n_items, n_qb, batch, status);
  count_launch();
  check_launch();
}

}  // namespace mb
