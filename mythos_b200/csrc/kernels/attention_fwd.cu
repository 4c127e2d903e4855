// Causal / full flash attention forward on tcgen05 tensor cores.
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles that ping-pong:
// while the softmax warpgroup of tile 0 works on S0 = Q0 K^T, the tensor core is busy with
// tile 1, and vice versa. S lives in TMEM (one row per thread, so row max / row sum need no
// shuffles), P goes back through a 128-byte-swizzled shared tile, O accumulates in TMEM and
// is rescaled lazily (only when a row maximum grows by more than 2^8).
//
// Warps: 0 = TMA loader, 1 = MMA issuer + TMEM owner, 2..5 = softmax tile 0, 6..9 = softmax tile 1.
// Tensors are token-major [batch, seq, heads, head_dim] with an arbitrary token stride, so Q, K
// and V can be views into one fused QKV projection output and O feeds the output projection
// without a transpose. Replaces the reference's materialised S x S attention
// (src/autograd.cpp:361-461) and its CPU tiled kernel (src/flash_attention.cpp:37-159).
#include "api.h"
#include "host_util.h"
#include "tc.cuh"

namespace mb {
namespace {

constexpr int FA_THREADS = 320;
constexpr int FA_BM = 128;  // query rows per tile (two tiles per CTA)
constexpr int FA_BN = 64;   // kv rows per step
constexpr int FA_STAGES = 3;

template <int D>
struct FaFwdCfg {
  static constexpr int Q_BYTES = FA_BM * D * 2;
  static constexpr int KV_BYTES = FA_BN * D * 2;
  static constexpr int STAGE_BYTES = 2 * KV_BYTES;
  static constexpr int P_BYTES = FA_BM * FA_BN * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = 2 * Q_BYTES;
  static constexpr int OFF_P = OFF_KV + FA_STAGES * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
  static constexpr int NUM_BARS = 1 + 2 * FA_STAGES + 6;
  static constexpr int SMEM_BYTES = OFF_BAR + NUM_BARS * 8 + 16 + 1024;
  static constexpr int TMEM_COLS = (D == 128) ? 512 : 256;
  static constexpr int COL_S = 0;    // S0 at 0, S1 at 64
  static constexpr int COL_O = 128;  // O0 at 128, O1 at 128 + D
};

// PAGED: prefill attention whose K/V live in the paged cache. Queries are the new tokens of each
// sequence, packed one sequence after another ([total_q, heads, D], sequence b = rows cu_q[b] ..
// cu_q[b+1]); keys / values are read page by page (16 tokens each) through the block table, one TMA
// box per page and 64-wide chunk, landing in the same swizzled tiles as the contiguous loads. The
// first query of sequence b sits at position kv_lens[b] - q_len, so the kernel serves a whole prompt
// (offset 0), one chunk of a long prompt, the remainder after a cached prefix, and ragged batches.
struct PagedPrefillArgs {
  const int* block_table;   // [batch, table_stride] page ids
  const int* cu_q;          // [batch + 1] first query row of every sequence
  const int* kv_lens;       // [batch] keys visible to the LAST query of the sequence (prefix + new tokens)
  int table_stride;
};
constexpr int FA_PAGE = 16;

template <int D, bool PAGED>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, __nv_bfloat16* __restrict__ o, float* __restrict__ lse,
              int seq, int heads, int kv_heads, long long o_tok_stride, int causal, float scale_log2, int* status,
              PagedPrefillArgs pa) {
  using Cfg = FaFwdCfg<D>;
  constexpr int DC = D / 64;  // 64-wide chunks of head_dim
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + FA_STAGES;
  uint64_t* s_full = kv_empty + FA_STAGES;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_done = p_full + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblk = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (heads / kv_heads);
  const int q0 = qblk * 2 * FA_BM;
  // q_len queries (rows q_row0 .. of the query tensor) see kv_len keys; query i sits at position q_off + i
  int q_len = seq, kv_len = seq, q_off = 0, q_row0 = 0;
  if constexpr (PAGED) {
    q_row0 = pa.cu_q[b];
    q_len = pa.cu_q[b + 1] - q_row0;
    kv_len = pa.kv_lens[b];
    q_off = kv_len - q_len;
    if (q0 >= q_len) return;                     // uniform over the CTA, before any barrier exists
  }
  const int n_qt = (q0 + FA_BM < q_len) ? 2 : 1;
  int J[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int hi = causal ? min(kv_len, q_off + min(q_len, q0 + (t + 1) * FA_BM)) : kv_len;
    J[t] = (t < n_qt) ? (hi + FA_BN - 1) / FA_BN : 0;
  }
  const int Jmax = max(J[0], J[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
      mbar_init(&o_done[t], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
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
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * Cfg::Q_BYTES);
      for (int t = 0; t < 2; ++t)
        for (int c = 0; c < DC; ++c)
          tma_load_4d(smem + Cfg::OFF_Q + t * Cfg::Q_BYTES + c * (FA_BM * 128), &tm_q, q_full, c * 64, h,
                      q_row0 + q0 + t * FA_BM, PAGED ? 0 : b);
      for (int j = 0; j < Jmax; ++j) {
        const int st = j % FA_STAGES;
        const uint32_t ph = (j / FA_STAGES) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, abort_flag, status, 11)) break;
        mbar_arrive_expect_tx(&kv_full[st], Cfg::STAGE_BYTES);
        uint8_t* sk = smem + Cfg::OFF_KV + st * Cfg::STAGE_BYTES;
        uint8_t* sv = sk + Cfg::KV_BYTES;
        if constexpr (PAGED) {
          // four pages of 16 tokens per kv tile; pages past the sequence's end (never visible: the
          // causal limit masks them) read page 0 so that the transaction count stays fixed
          const int* row = pa.block_table + (long long)b * pa.table_stride;
#pragma unroll
          for (int p = 0; p < FA_BN / FA_PAGE; ++p) {
            const int lp = j * (FA_BN / FA_PAGE) + p;
            int page = (lp * FA_PAGE < kv_len && lp < pa.table_stride) ? row[lp] : 0;
            if (page < 0) page = 0;
            for (int c = 0; c < DC; ++c) {
              tma_load_4d(sk + c * (FA_BN * 128) + p * (FA_PAGE * 128), &tm_k, &kv_full[st], c * 64, hkv, 0, page);
              tma_load_4d(sv + c * (FA_BN * 128) + p * (FA_PAGE * 128), &tm_v, &kv_full[st], c * 64, hkv, 0, page);
            }
          }
        } else {
          for (int c = 0; c < DC; ++c) {
            tma_load_4d(sk + c * (FA_BN * 128), &tm_k, &kv_full[st], c * 64, hkv, j * FA_BN, b);
            tma_load_4d(sv + c * (FA_BN * 128), &tm_v, &kv_full[st], c * 64, hkv, j * FA_BN, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_S = umma_idesc_bf16(FA_BM, FA_BN, false, false);
      constexpr uint32_t IDESC_O = umma_idesc_bf16(FA_BM, D, false, true);
      const uint32_t q_addr = smem_u32(smem + Cfg::OFF_Q);
      const uint32_t kv_addr = smem_u32(smem + Cfg::OFF_KV);
      const uint32_t p_addr = smem_u32(smem + Cfg::OFF_P);
      auto issue_s = [&](int t, int j) {
        const uint32_t qa = q_addr + t * Cfg::Q_BYTES;
        const uint32_t ka = kv_addr + (j % FA_STAGES) * Cfg::STAGE_BYTES;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const int c = k >> 2, kk = k & 3;
          umma_f16(tmem_base + Cfg::COL_S + t * FA_BN, umma_desc_sw128(qa + c * (FA_BM * 128) + kk * 32, 0, 1024),
                   umma_desc_sw128(ka + c * (FA_BN * 128) + kk * 32, 0, 1024), IDESC_S, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int j) {
        const uint32_t pa = p_addr + t * Cfg::P_BYTES;
        const uint32_t va = kv_addr + (j % FA_STAGES) * Cfg::STAGE_BYTES + Cfg::KV_BYTES;
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          umma_f16(tmem_base + Cfg::COL_O + t * D, umma_desc_sw128(pa + k * 32, 0, 1024),
                   umma_desc_sw128(va + k * 2048, FA_BN * 128, 1024), IDESC_O, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&o_done[t]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, status, 12);
      if (ok && Jmax > 0) ok = mbar_wait(&kv_full[0], 0, abort_flag, status, 13);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (J[t] > 0) issue_s(t, 0);
      }
      for (int j = 0; j < Jmax && ok; ++j) {
        const bool have_next = j + 1 < Jmax;
        bool next_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= J[t]) continue;
          if (!mbar_wait(&p_full[t], j & 1, abort_flag, status, 14)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, j);
          const bool last_user = (t == 1) || (j >= J[1]);
          if (last_user) umma_commit(&kv_empty[j % FA_STAGES]);
          if (j + 1 < J[t]) {
            if (have_next && !next_ready) {
              const int st = (j + 1) % FA_STAGES;
              if (!mbar_wait(&kv_full[st], ((j + 1) / FA_STAGES) & 1, abort_flag, status, 15)) { ok = false; break; }
              tc_fence_after();
              next_ready = true;
            }
            issue_s(t, j + 1);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int t = (warp - 2) >> 2;  // tile of this warpgroup
    const int quarter = warp & 3;   // TMEM lane quarter this warp may access
    const int r = quarter * 32 + lane;
    const int q_row = q0 + t * FA_BM + r;      // row within the sequence's queries
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + Cfg::COL_S + t * FA_BN + lane_sel;
    const uint32_t t_o = tmem_base + Cfg::COL_O + t * D + lane_sel;
    uint8_t* p_tile = smem + Cfg::OFF_P + t * Cfg::P_BYTES;
    float m_ref = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < J[t] && ok; ++j) {
      ok = mbar_wait(&s_full[t], j & 1, abort_flag, status, 16);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld32(t_s, sr[0]);
      tmem_ld32(t_s + 32, sr[1]);
      tmem_ld_wait();
      float* s = reinterpret_cast<float*>(&sr[0][0]);
      const int kv0 = j * FA_BN;
      const int limit = causal ? min(kv_len - 1, q_off + q_row) : kv_len - 1;  // last visible kv index
      if (kv0 + FA_BN - 1 > limit) {
#pragma unroll
        for (int i = 0; i < FA_BN; ++i)
          if (kv0 + i > limit) s[i] = -INFINITY;
      }
      float mx4[4] = {s[0], s[1], s[2], s[3]};  // four independent chains instead of one of length 64
#pragma unroll
      for (int i = 4; i < FA_BN; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], s[i]);
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = mx * scale_log2;
      float alpha = 1.f;
      bool need = false;
      if (j == 0) {
        m_ref = (m_new == -INFINITY) ? 0.f : m_new;
      } else if (m_new - m_ref > 8.f) {
        need = true;
        alpha = fast_exp2(m_ref - m_new);
        m_ref = m_new;
      }
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < FA_BN; ++i) {
        // three of four exponentials on the special-function unit, one on the FMA pipe
        const float e = fmaf(s[i], scale_log2, -m_ref);
        s[i] = ((i & 3) == 3) ? poly_exp2(e) : fast_exp2(e);
        rs4[i & 3] += s[i];
      }
      l = l * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
      if (j > 0) {
        ok = mbar_wait(&o_done[t], (j - 1) & 1, abort_flag, status, 17);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, need)) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t orr[32];
            tmem_ld32(t_o + c * 32, orr);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
            tmem_st32(t_o + c * 32, orr);
          }
          tmem_st_wait();
        }
      }
#pragma unroll
      for (int c = 0; c < FA_BN / 8; ++c) {
        uint4 v;
        v.x = pack_bf16x2(s[8 * c + 0], s[8 * c + 1]);
        v.y = pack_bf16x2(s[8 * c + 2], s[8 * c + 3]);
        v.z = pack_bf16x2(s[8 * c + 4], s[8 * c + 5]);
        v.w = pack_bf16x2(s[8 * c + 6], s[8 * c + 7]);
        *reinterpret_cast<uint4*>(p_tile + sw128_offset(r, c)) = v;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full[t]);
    }
    if (ok && J[t] > 0) {
      ok = mbar_wait(&o_done[t], (J[t] - 1) & 1, abort_flag, status, 18);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        const float inv_l = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* orow = o + (PAGED ? (long long)(q_row0 + q_row) : (long long)b * seq + q_row) * o_tok_stride +
                              (long long)h * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld32(t_o + c * 32, orr);
          tmem_ld_wait();
          if (q_row < q_len) {
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
        if (q_row < q_len && lse && !PAGED)
          lse[((long long)b * heads + h) * seq + q_row] = m_ref * 0.6931471805599453f + logf(l);
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

}  // namespace

// Tensor map over a token-major [batch, seq, nheads, head_dim] view with the given token stride.
CUtensorMap make_bshd_map(const void* base, int batch, int seq, int nheads, int head_dim, long long tok_stride,
                          int box_rows) {
  uint64_t dims[4] = {(uint64_t)head_dim, (uint64_t)nheads, (uint64_t)seq, (uint64_t)batch};
  uint64_t strides[3] = {(uint64_t)head_dim * 2, (uint64_t)tok_stride * 2, (uint64_t)seq * tok_stride * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_tensor_map(base, TmaDType::BF16, 4, dims, strides, box, true);
}

namespace { int g_attn_fwd_mode = 1; }   // 1: the persistent 128 x 128 kernel where it applies (head_dim 128)
void set_attn_fwd_mode(int mode) { g_attn_fwd_mode = mode; }
int get_attn_fwd_mode() { return g_attn_fwd_mode; }

void flash_attn_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq,
                            int heads, int kv_heads, int head_dim, long long q_tok_stride, long long kv_tok_stride,
                            long long o_tok_stride, bool causal, float scale, int* status, cudaStream_t stream) {
  MB_REQUIRE(head_dim == 64 || head_dim == 128, "flash_attn_fwd: head_dim must be 64 or 128");
  if (g_attn_fwd_mode == 1 && flash_attn_fwd2_supported(head_dim, seq)) {
    flash_attn_fwd2_strided(q, k, v, o, lse, batch, seq, heads, kv_heads, q_tok_stride, kv_tok_stride, o_tok_stride,
                            causal, scale, status, stream);
    return;
  }
  MB_REQUIRE(heads % kv_heads == 0, "flash_attn_fwd: heads must be a multiple of kv_heads");
  MB_REQUIRE(q_tok_stride % 8 == 0 && kv_tok_stride % 8 == 0 && o_tok_stride % 8 == 0,
             "flash_attn_fwd: token strides must be multiples of 8 elements");
  MB_REQUIRE((reinterpret_cast<uintptr_t>(o) & 15) == 0, "flash_attn_fwd: output must be 16-byte aligned");
  if (batch == 0 || seq == 0) return;
  const CUtensorMap tq = make_bshd_map(q, batch, seq, heads, head_dim, q_tok_stride, FA_BM);
  const CUtensorMap tk = make_bshd_map(k, batch, seq, kv_heads, head_dim, kv_tok_stride, FA_BN);
  const CUtensorMap tv = make_bshd_map(v, batch, seq, kv_heads, head_dim, kv_tok_stride, FA_BN);
  const dim3 grid((seq + 2 * FA_BM - 1) / (2 * FA_BM), heads, batch);
  const float scale_log2 = scale * 1.4426950408889634f;
  if (head_dim == 128) {
    static bool configured = false;
    if (!configured) {
      MB_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FaFwdCfg<128>::SMEM_BYTES));
      configured = true;
    }
    fa_fwd_kernel<128, false><<<grid, FA_THREADS, FaFwdCfg<128>::SMEM_BYTES, stream>>>(
        tq, tk, tv, (__nv_bfloat16*)o, lse, seq, heads, kv_heads, o_tok_stride, causal ? 1 : 0, scale_log2, status,
        PagedPrefillArgs{});
  } else {
    static bool configured = false;
    if (!configured) {
      MB_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FaFwdCfg<64>::SMEM_BYTES));
      configured = true;
    }
    fa_fwd_kernel<64, false><<<grid, FA_THREADS, FaFwdCfg<64>::SMEM_BYTES, stream>>>(
        tq, tk, tv, (__nv_bfloat16*)o, lse, seq, heads, kv_heads, o_tok_stride, causal ? 1 : 0, scale_log2, status,
        PagedPrefillArgs{});
  }
  count_launch();
  check_launch();
}

void flash_attn_paged_prefill(const void* q, long long q_tok_stride, const void* k_cache, const void* v_cache,
                              int n_pages, const int* block_table, int table_stride, const int* cu_q, const int* kv_lens,
                              void* o, long long o_tok_stride, int batch, int total_q, int max_q_len, int heads,
                              int kv_heads, int head_dim, float scale, int* status, cudaStream_t stream) {
  MB_REQUIRE(head_dim == 64 || head_dim == 128, "flash_attn_paged_prefill: head_dim must be 64 or 128");
  MB_REQUIRE(heads % kv_heads == 0, "flash_attn_paged_prefill: heads must be a multiple of kv_heads");
  MB_REQUIRE(q_tok_stride % 8 == 0 && o_tok_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0,
             "flash_attn_paged_prefill: strides / alignment");
  if (batch == 0 || total_q == 0 || max_q_len == 0) return;
  const CUtensorMap tq = make_bshd_map(q, 1, total_q, heads, head_dim, q_tok_stride, FA_BM);
  // pages: [n_pages, 16 tokens, kv_heads, head_dim]; one box = 16 tokens x 64 columns of one head
  auto page_map = [&](const void* base) {
    uint64_t dims[4] = {(uint64_t)head_dim, (uint64_t)kv_heads, (uint64_t)FA_PAGE, (uint64_t)n_pages};
    uint64_t strides[3] = {(uint64_t)head_dim * 2, (uint64_t)kv_heads * head_dim * 2,
                           (uint64_t)FA_PAGE * kv_heads * head_dim * 2};
    uint32_t box[4] = {64, 1, (uint32_t)FA_PAGE, 1};
    return make_tensor_map(base, TmaDType::BF16, 4, dims, strides, box, true);
  };
  const CUtensorMap tk = page_map(k_cache), tv = page_map(v_cache);
  const dim3 grid((max_q_len + 2 * FA_BM - 1) / (2 * FA_BM), heads, batch);
  const float scale_log2 = scale * 1.4426950408889634f;
  PagedPrefillArgs pa{block_table, cu_q, kv_lens, table_stride};
  if (head_dim == 128) {
    static bool configured = false;
    if (!configured) {
      MB_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FaFwdCfg<128>::SMEM_BYTES));
      configured = true;
    }
    fa_fwd_kernel<128, true><<<grid, FA_THREADS, FaFwdCfg<128>::SMEM_BYTES, stream>>>(
        tq, tk, tv, (__nv_bfloat16*)o, nullptr, total_q, heads, kv_heads, o_tok_stride, 1, scale_log2, status, pa);
  } else {
    static bool configured = false;
    if (!configured) {
      MB_CUDA_CHECK(cudaFuncSetAttribute(fa_fwd_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FaFwdCfg<64>::SMEM_BYTES));
      configured = true;
    }
    fa_fwd_kernel<64, true><<<grid, FA_THREADS, FaFwdCfg<64>::SMEM_BYTES, stream>>>(
        tq, tk, tv, (__nv_bfloat16*)o, nullptr, total_q, heads, kv_heads, o_tok_stride, 1, scale_log2, status, pa);
  }
  count_launch();
  check_launch();
}

void flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq, int heads,
                    int kv_heads, int head_dim, bool causal, float scale, int* status, cudaStream_t stream) {
  flash_attn_fwd_strided(q, k, v, o, lse, batch, seq, heads, kv_heads, head_dim, (long long)heads * head_dim,
                         (long long)kv_heads * head_dim, (long long)heads * head_dim, causal, scale, status, stream);
}

}  // namespace mb
