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
  static constexpr int SEG_OFFSET = BAR_OFFSET + 256;             // grouped GEMM: segment starts / rows (2 x 16 ints)
  static constexpr int EPI_STAGE_OFFSET = BAR_OFFSET + 512;       // [up to 8 epilogue warps][32 rows][128 B]
  static constexpr int SMEM_BYTES = EPI_STAGE_OFFSET + 8 * 4096 + 1024;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");
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
  int e = 0;      // grouped GEMM: segment (expert) of this tile
  int kofs = 0;   // grouped GEMM over K: first row of the segment (added to every K coordinate)
};

// Grouped (ragged) GEMM. One launch covers several segments of one row-indexed buffer, e.g. the
// tokens routed to each local expert; segment starts and row counts live in device memory (they come
// from the router kernel, the host never sees them). Segment starts are multiples of 256 rows and the
// rows between a segment's end and the next multiple of 256 hold zeros.
//   GROUP_ROWS  C[rows of segment e, :] = A[rows of segment e, :] * B_e^T   (ragged M; B per segment)
//   GROUP_K     C_e (+)= A[rows of e, :]^T * B[rows of e, :]                (ragged K; C per segment)
constexpr int MAX_GROUPS = 16;
enum : int { GROUP_NONE = 0, GROUP_ROWS = 1, GROUP_K = 2, GROUP_GATHER = 3 };
constexpr int AG_MAX_RANKS = 8;
template <int G>
struct GroupArgsT {};
template <>
struct GroupArgsT<GROUP_ROWS> {
  const int* seg_start;
  const int* seg_rows;
  int n_seg;
  CUtensorMap bmaps[MAX_GROUPS];
};
template <>
struct GroupArgsT<GROUP_K> {
  const int* seg_start;
  const int* seg_rows;
  int n_seg;
  void* cptrs[MAX_GROUPS];
};
// All-gather fused into the GEMM (GROUP_GATHER). A = [M, K] is sharded by rows over the ranks: every rank
// holds a full-size buffer in symmetric memory and has written only its own rows. A few SM pairs of the
// launch do not compute: their CTAs copy the other ranks' rows into this rank's buffer, 128 x 64 pieces
// through a shared-memory ring with non-multicast TMA loads from the peer's buffer and TMA stores into the
// local one, 256-row tile by tile in the order in which the computing SM pairs consume them (own rows
// first, then the rows of rank + 1, rank + 2, ...). When a copier has stored its pieces of a tile it adds
// one to the tile's counter; the TMA producers of the computing CTAs wait (bounded) for the counter to
// reach `target` before they load a tile that is not the rank's own. Every remote byte crosses NVLink
// once, and the copy of the later tiles overlaps the products of the earlier ones.
template <>
struct GroupArgsT<GROUP_GATHER> {
  CUtensorMap peer[AG_MAX_RANKS];  // the gathered operand's buffer on every rank as mapped here; same shape and
                                   // box as the launch's own map of that operand (tma_a or tma_b)
  int* tile_count;                 // [256-row tiles of the gathered operand], monotonic over calls
  int target;                      // copier CTAs x calls so far (this one included)
  int rank, world, tiles_per_rank, copier_clusters;
  int gather_b;                    // 0: A (activations sharded by tokens); 1: B (a weight sharded by output rows).
                                   // With B the tiles are walked column block by column block (own columns first),
                                   // all row tiles of a column block on neighbouring SM pairs, so that a gathered
                                   // 256-row block of B is reused out of L2 while it is current.
};
__device__ __forceinline__ int ld_acquire_gpu_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

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

__device__ __forceinline__ uint4 pack8_bf16(const float* v) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]);
  o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]);
  o.w = pack_bf16x2(v[6], v[7]);
  return o;
}
__device__ __forceinline__ void unpack8_bf16(const uint4& q, float* v) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
// sigmoid(x) = 0.5 * tanh(0.5 x) + 0.5 with the hardware tanh: one special-function op per element
// (exp + reciprocal would be two, and the special-function pipe is what bounds these epilogues).
__device__ __forceinline__ float sigmoid_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}

// FUSE selects work folded into the epilogue (a separate instantiation each, so the plain GEMM's
// code and register allocation are unaffected):
//   FUSE_SWIGLU_FWD  gate/up projection: the pair's B halves are the gate rows [tn*128, +128) and the
//                    up rows [F + tn*128, +128) of the [2F, K] weight, so every thread holds gate and
//                    up of the same output element; writes both pre-activations and silu(g)*u.
//   FUSE_SWIGLU_BWD  down-projection dgrad: the accumulator is dL/dh; the epilogue reads the saved
//                    pre-activations and writes dL/dgate and dL/dup, dL/dh never reaches memory.
//   FUSE_ROPE        QKV projection: columns [0, rope_cols) are heads of 128 that get the half-split
//                    rotation by the row's position (table of cos/sin pairs) before the bf16 store.
// The SwiGLU-backward epilogue waits on global loads (the saved pre-activations); it runs eight
// epilogue warps (two per TMEM lane quarter, four 32-column chunks each) to have twice the loads in flight.
template <int FUSE>
__host__ __device__ constexpr int epi_warps() { return FUSE == FUSE_SWIGLU_BWD ? 8 : 4; }
template <int FUSE>
__host__ __device__ constexpr int cta_threads() { return 64 + 32 * epi_warps<FUSE>(); }
static_assert(cta_threads<FUSE_NONE>() == T_THREADS, "plain kernel: producer + MMA + four epilogue warps");

// Tile list of a grouped launch: segment-major; s_seg = [starts | rows] in shared memory.
template <int GROUP>
__device__ __forceinline__ int group_total(const int* s_seg, int n_seg, int tiles_m, int tiles_n) {
  int total = 0;
  for (int e = 0; e < n_seg; ++e) {
    const int rows = s_seg[MAX_GROUPS + e];
    if (rows > 0) total += (GROUP == GROUP_ROWS ? (rows + T_BM - 1) / T_BM : tiles_m) * tiles_n;
  }
  return total;
}
template <int GROUP>
__device__ __forceinline__ Work2 group_decode(int w, const int* s_seg, int n_seg, int tiles_m, int tiles_n, int kblocks) {
  Work2 wi{0, 0, 0, 0, 0, 0};
  for (int e = 0; e < n_seg; ++e) {
    const int rows = s_seg[MAX_GROUPS + e];
    if (rows <= 0) continue;
    const int tm_e = GROUP == GROUP_ROWS ? (rows + T_BM - 1) / T_BM : tiles_m;
    const int n_e = tm_e * tiles_n;
    if (w < n_e) {
      wi = decode2(w, tm_e, tiles_n, 1, kblocks);
      wi.e = e;
      if (GROUP == GROUP_ROWS) {
        wi.m0 += s_seg[e];
      } else {
        wi.kofs = s_seg[e];
        wi.kb0 = 0;
        wi.kb1 = (rows + T_BK - 1) / T_BK;
      }
      return wi;
    }
    w -= n_e;
  }
  return wi;
}

template <bool A_MN, bool B_MN, int FUSE, int GROUP = GROUP_NONE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(cta_threads<FUSE>(), 1)
gemm_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 void* __restrict__ Cout, int M, int N, int K, long long ldc, int tiles_m, int tiles_n, int k_splits,
                 int epi, int vec_ok, float alpha, int* status, PeerPtrs scatter, int n_scatter,
                 long long rows_per_rank, long long slot_off, EpiFuse fz,
                 const __grid_constant__ GroupArgsT<GROUP> ga) {
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
  const int cluster_id = blockIdx.x >> 1;
  int n_clusters = gridDim.x >> 1;      // SM pairs that compute tiles
  bool is_copier = false;
  if constexpr (GROUP == GROUP_GATHER) {
    n_clusters -= ga.copier_clusters;
    is_copier = cluster_id >= n_clusters;
  }
  int* s_seg = reinterpret_cast<int*>(smem + Cfg::SEG_OFFSET);
  int n_seg = 0;
  if constexpr (GROUP == GROUP_ROWS || GROUP == GROUP_K) {
    n_seg = ga.n_seg;
    if (threadIdx.x < MAX_GROUPS) {
      const bool in = (int)threadIdx.x < n_seg;
      s_seg[threadIdx.x] = in ? ga.seg_start[threadIdx.x] : 0;
      s_seg[MAX_GROUPS + threadIdx.x] = in ? ga.seg_rows[threadIdx.x] : 0;
    }
    __syncthreads();
  }
  constexpr bool SEGMENTED = GROUP == GROUP_ROWS || GROUP == GROUP_K;
  const int total = SEGMENTED ? group_total<GROUP>(s_seg, n_seg, tiles_m, tiles_n) : tiles_m * tiles_n * k_splits;
  auto get_work = [&](int w) -> Work2 {
    if constexpr (SEGMENTED) {
      return group_decode<GROUP>(w, s_seg, n_seg, tiles_m, tiles_n, kblocks);
    } else {
      if constexpr (GROUP == GROUP_GATHER) {   // this rank's own rows first, then the ranks after it
        if (ga.gather_b) {
          const int tn = w / tiles_m, tm = w - tn * tiles_m;
          return Work2{tm * T_BM, ((tn + ga.rank * ga.tiles_per_rank) % tiles_n) * T_BN, 0, kblocks};
        }
        Work2 wi = decode2(w, tiles_m, tiles_n, k_splits, kblocks);
        wi.m0 = ((wi.m0 / T_BM + ga.rank * ga.tiles_per_rank) % tiles_m) * T_BM;
        return wi;
      }
      return decode2(w, tiles_m, tiles_n, k_splits, kblocks);
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < T_STAGES; ++s) {
      mbar_init(&full[s], 1);   // leader: its own arrive.expect_tx (bytes of both CTAs)
      mbar_init(&empty[s], 1);  // one commit from the leader's MMA thread
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 2 * epi_warps<FUSE>());   // leader: the epilogue warps of both CTAs
    mbar_init(&tempty[1], 2 * epi_warps<FUSE>());
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

  if (is_copier) {
    // ------------------------------------------------------------------ all-gather copier CTAs
    if constexpr (GROUP == GROUP_GATHER) {
      constexpr int CS = 12, PIECE = 128 * T_BK * 2;   // twelve 16 KB pieces in flight per CTA
      static_assert(CS * PIECE <= Cfg::BAR_OFFSET, "copier ring must fit into the stage area");
      uint64_t* cfull = reinterpret_cast<uint64_t*>(smem + Cfg::EPI_STAGE_OFFSET);
      uint64_t* cempty = cfull + CS;
      const int ci = (cluster_id - n_clusters) * 2 + (int)cta, n_cop = ga.copier_clusters * 2;
      if (threadIdx.x == 0) {
        for (int i = 0; i < CS; ++i) {
          mbar_init(&cfull[i], 1);
          mbar_init(&cempty[i], 1);
        }
        fence_mbar_init();
      }
      __syncthreads();
      const int tiles_g = ga.gather_b ? tiles_n : tiles_m;   // 256-row tiles of the gathered operand
      const CUtensorMap* store_map = ga.gather_b ? &tma_b : &tma_a;
      const int n_remote = tiles_g - ga.tiles_per_rank;
      const int pieces = 2 * kblocks;                  // two 128-row halves per k-block of a 256-row tile
      if (warp == 0 && lane == 0) {
        // loads: the owner's buffer -> ring
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int j = 0; j < n_remote && ok; ++j) {
          const int mt = ((ga.rank + 1) * ga.tiles_per_rank + j) % tiles_g;
          const CUtensorMap* src = &ga.peer[mt / ga.tiles_per_rank];
          for (int p = ci; p < pieces; p += n_cop) {
            if (!mbar_wait(&cempty[stage], phase ^ 1, abort_flag, status, 57)) { ok = false; break; }
            mbar_arrive_expect_tx(&cfull[stage], PIECE);
            tma_load_2d(smem + stage * PIECE, src, &cfull[stage], (p >> 1) * T_BK, mt * T_BM + (p & 1) * 128);
            if (++stage == CS) { stage = 0; phase ^= 1; }
          }
        }
      } else if (warp == 1 && lane == 0) {
        // stores: ring -> this rank's buffer; a stage is handed back once its store has read it
        int stage = 0, oldest = 0, pending = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int j = 0; j < n_remote && ok; ++j) {
          const int mt = ((ga.rank + 1) * ga.tiles_per_rank + j) % tiles_g;
          for (int p = ci; p < pieces; p += n_cop) {
            if (!mbar_wait(&cfull[stage], phase, abort_flag, status, 58)) { ok = false; break; }
            tma_store_2d(store_map, smem + stage * PIECE, (p >> 1) * T_BK, mt * T_BM + (p & 1) * 128);
            tma_store_commit();
            if (++stage == CS) { stage = 0; phase ^= 1; }
            if (++pending > 4) {
              bulk_wait_group_read<4>();
              mbar_arrive(&cempty[oldest]);
              if (++oldest == CS) oldest = 0;
              --pending;
            }
          }
          if (!ok) break;
          tma_store_wait0();               // this copier's pieces of the tile are in memory
          for (; pending > 0; --pending) {
            mbar_arrive(&cempty[oldest]);
            if (++oldest == CS) oldest = 0;
          }
          asm volatile("fence.proxy.async;" ::: "memory");   // completed bulk stores before the release below
          red_release_gpu_add(ga.tile_count + mt, 1);
        }
        tma_store_wait0();
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = cluster_id; w < total && ok; w += n_clusters) {
        const Work2 wi = get_work(w);
        const int my_m = wi.m0 + (int)cta * 128;
        const int my_n = (FUSE == FUSE_SWIGLU_FWD) ? (wi.n0 >> 1) + (int)cta * fz.F : wi.n0 + (int)cta * 128;
        const CUtensorMap* map_b = &tma_b;
        if constexpr (GROUP == GROUP_ROWS) map_b = &ga.bmaps[wi.e];
        if constexpr (GROUP == GROUP_GATHER) {
          const int tmi = ga.gather_b ? wi.n0 / T_BN : wi.m0 / T_BM;
          if (tmi / ga.tiles_per_rank != ga.rank) {     // rows of another rank: wait until the copiers have brought them
            const long long t0 = clock64();
            while (ld_acquire_gpu_s32(ga.tile_count + tmi) - ga.target < 0) {
              if (*abort_flag) { ok = false; break; }
              if (clock64() - t0 > MB_WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, ST_TIMEOUT | (59 << 16));
                ok = false;
                break;
              }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");   // the copiers' bulk stores before this thread's bulk loads
          }
        }
        for (int kb = wi.kb0; kb < wi.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, status, 51)) { ok = false; break; }
          const uint32_t lbar = map_to_cta(smem_u32(&full[stage]), 0);
          if (leader) mbar_arrive_expect_tx(&full[stage], 2 * Cfg::STAGE_BYTES);
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          const int kc = wi.kofs + kb * T_BK;
          if (!A_MN) {
            tma_load_2d_pair(sa, &tma_a, lbar, kc, my_m);
          } else {
            tma_load_2d_pair(sa, &tma_a, lbar, my_m, kc);
            tma_load_2d_pair(sa + 8192, &tma_a, lbar, my_m + 64, kc);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, map_b, lbar, kc, my_n);
          } else {
            tma_load_2d_pair(sb, map_b, lbar, my_n, kc);
            tma_load_2d_pair(sb + 8192, map_b, lbar, my_n + 64, kc);
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
        const Work2 wi = get_work(w);
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
      const Work2 wi = get_work(w);
      void* Cw = Cout;                                   // output of this tile (per segment when K is ragged)
      if constexpr (GROUP == GROUP_K) Cw = ga.cptrs[wi.e];
      bool ok = mbar_wait(&tfull[acc], acc_phase, abort_flag, status, 54);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = wi.m0 + (int)cta * 128 + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * T_BN + ((uint32_t)(q * 32) << 16);
      if (FUSE == FUSE_SWIGLU_FWD) {
        // accumulator columns [0,128) = gate, [128,256) = up of ffn columns (n0/2) .. (n0/2)+127.
        // Stores go through the per-warp shared-memory tile so that a warp instruction writes 64
        // contiguous bytes of 8 rows instead of 16 bytes of 32 rows (see FUSE_SWIGLU_BWD below).
        uint8_t* sA = smem + Cfg::EPI_STAGE_OFFSET + q * 4096;
        uint8_t* sB = sA + 2048;
        const int row0 = wi.m0 + (int)cta * 128 + q * 32;
        const int crow = lane >> 2, cpiece = lane & 3;
        const int colg0 = wi.n0 >> 1;
        __nv_bfloat16* gu_base = reinterpret_cast<__nv_bfloat16*>(Cw);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t rg[32], ru[32];
          tmem_ld32(t_row + c * 32, rg);
          tmem_ld32(t_row + 128 + c * 32, ru);
          tmem_ld_wait();
          uint4 hq[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float g[8], u[8], h[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              g[i] = alpha * __uint_as_float(rg[8 * j + i]);
              u[i] = alpha * __uint_as_float(ru[8 * j + i]);
              h[i] = g[i] * sigmoid_fast(g[i]) * u[i];
            }
            const uint32_t off = lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4);
            *reinterpret_cast<uint4*>(sA + off) = pack8_bf16(g);
            *reinterpret_cast<uint4*>(sB + off) = pack8_bf16(u);
            hq[j] = pack8_bf16(h);
          }
          __syncwarp();
          const int col = colg0 + c * 32 + cpiece * 8;
          if (gu_base != nullptr) {
#pragma unroll
            for (int it = 0; it < 4; ++it) {
              const int rr = it * 8 + crow;
              if (row0 + rr < M) {
                const uint32_t off = rr * 64 + ((cpiece ^ ((rr >> 1) & 3)) << 4);
                __nv_bfloat16* p = gu_base + (long long)(row0 + rr) * ldc + col;
                *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(sA + off);
                *reinterpret_cast<uint4*>(p + fz.F) = *reinterpret_cast<const uint4*>(sB + off);
              }
            }
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(sA + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) = hq[j];
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int rr = it * 8 + crow;
            if (row0 + rr < M)
              *reinterpret_cast<uint4*>(fz.out2 + (long long)(row0 + rr) * fz.ld_out2 + col) =
                  *reinterpret_cast<const uint4*>(sA + rr * 64 + ((cpiece ^ ((rr >> 1) & 3)) << 4));
          }
          __syncwarp();
        }
      } else if (FUSE == FUSE_SWIGLU_BWD) {
        // accumulator = dL/dh for ffn columns n0 .. n0+255; pre-activations come from fz.aux [M, 2F].
        // A thread owns one accumulator row, but 32 rows x 16 bytes per instruction would make every
        // global access of the warp 32 separate sectors, and this epilogue moves four times the bytes
        // of a plain store. So global memory is touched in the transposed arrangement (4 lanes per
        // row, 64 contiguous bytes, 8 rows per instruction) and a per-warp shared-memory tile
        // (two 32 x 64-byte buffers, 16-byte pieces XOR-swizzled by row pair) converts between the two.
        uint8_t* sA = smem + Cfg::EPI_STAGE_OFFSET + (warp - 2) * 4096;
        uint8_t* sB = sA + 2048;
        const int row0 = wi.m0 + (int)cta * 128 + q * 32;
        const int cbase = ((warp - 2) >> 2) * 4;                // this warp's four chunks of the tile
        const int nchunks = min(4, max(0, (fz.F - wi.n0) / 32 - cbase));
        const int crow = lane >> 2, cpiece = lane & 3;          // coalesced phase: row within a group of 8, piece
        uint4 pg[2][4], pu[2][4];                               // two chunks of pre-activations in flight
        auto fetch = [&](int i, uint4* dg_, uint4* du_) {
          const int col = wi.n0 + (cbase + i) * 32 + cpiece * 8;
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int rr = it * 8 + crow;
            const __nv_bfloat16* p = fz.aux + (long long)min(row0 + rr, M - 1) * fz.ld_aux + col;
            dg_[it] = __ldg(reinterpret_cast<const uint4*>(p));
            du_[it] = __ldg(reinterpret_cast<const uint4*>(p + fz.F));
          }
        };
        if (nchunks > 0) fetch(0, pg[0], pu[0]);
        if (nchunks > 1) fetch(1, pg[1], pu[1]);
        {
          // Pull the pre-activations of this CTA's NEXT tile into L2 now, a whole main loop ahead:
          // the demand loads above then pay an L2 hit instead of a loaded-DRAM round trip.
          const int w2 = w + n_clusters;
          if (w2 < total) {
            const Work2 nx = get_work(w2);
            const int tid = (warp - 2) * 32 + lane;             // 256 threads, 1024 lines of 128 bytes
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int line = tid * 4 + i;
              const int prow = nx.m0 + (int)cta * 128 + (line >> 3), seg = line & 7;
              const int pcol = nx.n0 + (seg & 3) * 64;
              if (prow < M && pcol < fz.F) {
                const __nv_bfloat16* pp = fz.aux + (long long)prow * fz.ld_aux + pcol + (seg >> 2) * fz.F;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(pp));
              }
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (i >= nchunks) break;                              // uniform over the warp
          const int c = cbase + i;
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int rr = it * 8 + crow;
            const uint32_t off = rr * 64 + ((cpiece ^ ((rr >> 1) & 3)) << 4);
            *reinterpret_cast<uint4*>(sA + off) = pg[i & 1][it];
            *reinterpret_cast<uint4*>(sB + off) = pu[i & 1][it];
          }
          __syncwarp();
          uint4 gq[4], uq[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t off = lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4);
            gq[j] = *reinterpret_cast<const uint4*>(sA + off);
            uq[j] = *reinterpret_cast<const uint4*>(sB + off);
          }
          __syncwarp();
          if (i + 2 < nchunks) fetch(i + 2, pg[i & 1], pu[i & 1]);   // refill the buffer just consumed
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float g[8], u[8], dg[8], du[8];
            unpack8_bf16(gq[j], g);
            unpack8_bf16(uq[j], u);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float dh = alpha * __uint_as_float(r[8 * j + e]);
              const float sg = sigmoid_fast(g[e]);
              const float silu = g[e] * sg;
              dg[e] = dh * u[e] * (sg + silu * (1.f - sg));
              du[e] = dh * silu;
            }
            const uint32_t off = lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4);
            *reinterpret_cast<uint4*>(sA + off) = pack8_bf16(dg);
            *reinterpret_cast<uint4*>(sB + off) = pack8_bf16(du);
          }
          __syncwarp();
          const int col = wi.n0 + c * 32 + cpiece * 8;
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int rr = it * 8 + crow;
            if (row0 + rr < M) {
              const uint32_t off = rr * 64 + ((cpiece ^ ((rr >> 1) & 3)) << 4);
              __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(Cw) + (long long)(row0 + rr) * ldc + col;
              *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(sA + off);
              *reinterpret_cast<uint4*>(p + fz.F) = *reinterpret_cast<const uint4*>(sB + off);
            }
          }
          __syncwarp();
        }
      } else if (FUSE == FUSE_ROPE) {
        __nv_bfloat16* c_row = reinterpret_cast<__nv_bfloat16*>(Cw) + (long long)row * ldc;
        int p = (row < M) ? fz.pos[row] : 0;
        p = min(max(p, 0), fz.max_pos - 1);
        const float4* cs_row = reinterpret_cast<const float4*>(fz.cs + (long long)p * 64);
#pragma unroll 1
        for (int hb = 0; hb < 2; ++hb) {
          const int head_col = wi.n0 + hb * 128;
          if (head_col >= N) break;
          const bool rotate = head_col + 128 <= fz.rope_cols;
#pragma unroll 1
          for (int cc = 0; cc < 2; ++cc) {
            uint32_t lo[32], hi[32];
            tmem_ld32(t_row + hb * 128 + cc * 32, lo);
            tmem_ld32(t_row + hb * 128 + 64 + cc * 32, hi);
            tmem_ld_wait();
            if (row < M) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float a[8], b[8];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                  float x0 = alpha * __uint_as_float(lo[8 * j + i]), x1 = alpha * __uint_as_float(lo[8 * j + i + 1]);
                  float y0 = alpha * __uint_as_float(hi[8 * j + i]), y1 = alpha * __uint_as_float(hi[8 * j + i + 1]);
                  if (rotate) {
                    const float4 t = __ldg(cs_row + ((cc * 32 + 8 * j + i) >> 1));  // (cos, sin) of two pairs
                    a[i] = x0 * t.x - y0 * t.y;
                    b[i] = x0 * t.y + y0 * t.x;
                    a[i + 1] = x1 * t.z - y1 * t.w;
                    b[i + 1] = x1 * t.w + y1 * t.z;
                  } else {
                    a[i] = x0; b[i] = y0; a[i + 1] = x1; b[i + 1] = y1;
                  }
                }
                *reinterpret_cast<uint4*>(c_row + head_col + cc * 32 + 8 * j) = pack8_bf16(a);
                *reinterpret_cast<uint4*>(c_row + head_col + 64 + cc * 32 + 8 * j) = pack8_bf16(b);
              }
            }
          }
        }
      } else
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
        if (vec_ok == 2 && col + 32 <= N && epi != EPI_F32_ATOMIC) {
          // Full 32-column chunk (uniform over the warp): transpose through the warp's shared-memory
          // tile so that every store instruction writes whole contiguous row segments (bf16: 64 bytes
          // of 8 rows; fp32: 128 bytes of 4 rows) instead of 16 bytes of 32 different rows.
          const int row0 = wi.m0 + (int)cta * 128 + q * 32;
          uint8_t* stage = smem + Cfg::EPI_STAGE_OFFSET + q * 4096;
          if (epi == EPI_BF16) {
            uint8_t* sbuf = stage + (c & 1) * 2048;              // alternate halves: one warp barrier per chunk
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = alpha * __uint_as_float(r[8 * j + e]);
              *reinterpret_cast<uint4*>(sbuf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) = pack8_bf16(v);
            }
            __syncwarp();
            const int crow = lane >> 2, cpiece = lane & 3;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
              const int rr = it * 8 + crow;
              if (row0 + rr < M)
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(Cw) + (long long)(row0 + rr) * ldc + col +
                                          cpiece * 8) =
                    *reinterpret_cast<const uint4*>(sbuf + rr * 64 + ((cpiece ^ ((rr >> 1) & 3)) << 4));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 v = make_float4(alpha * __uint_as_float(r[4 * j]), alpha * __uint_as_float(r[4 * j + 1]),
                                     alpha * __uint_as_float(r[4 * j + 2]), alpha * __uint_as_float(r[4 * j + 3]));
              *reinterpret_cast<float4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
            }
            __syncwarp();
            const int crow = lane >> 3, cpiece = lane & 7;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int rr = it * 4 + crow;
              if (row0 + rr < M) {
                float4 v = *reinterpret_cast<const float4*>(stage + rr * 128 + ((cpiece ^ (rr & 7)) << 4));
                float4* gp = reinterpret_cast<float4*>(reinterpret_cast<float*>(Cw) + (long long)(row0 + rr) * ldc + col +
                                                       cpiece * 4);
                if (epi == EPI_F32_ACC) {
                  const float4 o = *gp;
                  v = make_float4(o.x + v.x, o.y + v.y, o.z + v.z, o.w + v.w);
                }
                *gp = v;
              }
            }
            __syncwarp();
          }
          continue;
        }
        if (row < M && col < N) {
          const int ncols = min(32, N - col);
          if (epi == EPI_BF16) {
            __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(Cw) + (long long)row * ldc + col;
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
            float* p = reinterpret_cast<float*>(Cw) + (long long)row * ldc + col;
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

template <bool A_MN, bool B_MN, int FUSE = FUSE_NONE, int GROUP = GROUP_NONE>
void launch2(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc, int k_splits,
             int epi, int vec_ok, float alpha, int* status, cudaStream_t stream, const PeerPtrs& scatter,
             int n_scatter, long long rows_per_rank, long long slot_off, const EpiFuse& fz = EpiFuse{},
             const GroupArgsT<GROUP>& ga = GroupArgsT<GROUP>{}) {
  auto kern = gemm_2cta_kernel<A_MN, B_MN, FUSE, GROUP>;
  static bool configured = false;
  if (!configured) {
    MB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg2::SMEM_BYTES));
    configured = true;
  }
  const int tiles_m = (M + T_BM - 1) / T_BM, tiles_n = (N + T_BN - 1) / T_BN;
  const int total = tiles_m * tiles_n * k_splits;
  int clusters = sm_count() / 2;
  if (GROUP == GROUP_NONE && total < clusters) clusters = total;   // grouped: the tile count is known on the device only
  kern<<<clusters * 2, cta_threads<FUSE>(), Cfg2::SMEM_BYTES, stream>>>(ta, tb, C, M, N, K, ldc, tiles_m, tiles_n, k_splits, epi,
                                                              vec_ok, alpha, status, scatter, n_scatter, rows_per_rank,
                                                              slot_off, fz, ga);
  count_launch();
  check_launch();
}

}  // namespace

namespace { int g_coalesced_epilogue = 1; }
void set_gemm_coalesced_epilogue(int on) { g_coalesced_epilogue = on; }

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

namespace {
void kmajor_map_dims(uint64_t* dims, uint32_t* box, int rows, int K) {
  dims[0] = K; dims[1] = rows; box[0] = T_BK; box[1] = 128;
}
}  // namespace

void gemm_swiglu_fwd(const void* x, long long ldx, const void* w_gate_up, long long ldw, void* gate_up, long long ld_gu,
                     void* h, long long ld_h, int M, int F, int K, int* status, cudaStream_t stream) {
  MB_REQUIRE(M > 0 && F > 0 && K > 0, "gemm_swiglu_fwd: empty problem");
  MB_REQUIRE(F % 128 == 0, "gemm_swiglu_fwd: the ffn width must be a multiple of 128");
  MB_REQUIRE(ldx % 8 == 0 && ldw % 8 == 0 && ld_h % 8 == 0 && (gate_up == nullptr || ld_gu % 8 == 0),
             "gemm_swiglu_fwd: row strides must be multiples of 8 elements");
  MB_REQUIRE((reinterpret_cast<uintptr_t>(h) & 15) == 0 && (reinterpret_cast<uintptr_t>(gate_up) & 15) == 0,
             "gemm_swiglu_fwd: outputs must be 16-byte aligned");
  uint64_t adims[2], astr[1] = {(uint64_t)ldx * 2}, bdims[2], bstr[1] = {(uint64_t)ldw * 2};
  uint32_t abox[2], bbox[2];
  kmajor_map_dims(adims, abox, M, K);
  kmajor_map_dims(bdims, bbox, 2 * F, K);
  const CUtensorMap ta = make_tensor_map(x, TmaDType::BF16, 2, adims, astr, abox, true);
  const CUtensorMap tb = make_tensor_map(w_gate_up, TmaDType::BF16, 2, bdims, bstr, bbox, true);
  EpiFuse fz{};
  fz.F = F;
  fz.out2 = reinterpret_cast<__nv_bfloat16*>(h);
  fz.ld_out2 = ld_h;
  // N = 2F: one 256-column tile is 128 gate + 128 up columns, so tiles_n = F / 128
  launch2<false, false, FUSE_SWIGLU_FWD>(ta, tb, gate_up, M, 2 * F, K, ld_gu, 1, EPI_BF16, 1, 1.f, status, stream,
                                         PeerPtrs{}, 0, 0, 0, fz);
}

void gemm_swiglu_bwd(const void* dy, long long ld_dy, const void* w_down, long long ldw, const void* gate_up,
                     long long ld_gu, void* d_gate_up, long long ld_dgu, int M, int F, int K, int* status,
                     cudaStream_t stream) {
  MB_REQUIRE(M > 0 && F > 0 && K > 0, "gemm_swiglu_bwd: empty problem");
  MB_REQUIRE(F % 64 == 0, "gemm_swiglu_bwd: the ffn width must be a multiple of 64");
  MB_REQUIRE(ld_dy % 8 == 0 && ldw % 8 == 0 && ld_gu % 8 == 0 && ld_dgu % 8 == 0,
             "gemm_swiglu_bwd: row strides must be multiples of 8 elements");
  MB_REQUIRE((reinterpret_cast<uintptr_t>(gate_up) & 15) == 0 && (reinterpret_cast<uintptr_t>(d_gate_up) & 15) == 0,
             "gemm_swiglu_bwd: pre-activation buffers must be 16-byte aligned");
  // dh[M, F] = dy[M, K] @ W_down[K, F]: A K-major, B MN-major
  uint64_t adims[2], astr[1] = {(uint64_t)ld_dy * 2}, bdims[2] = {(uint64_t)F, (uint64_t)K}, bstr[1] = {(uint64_t)ldw * 2};
  uint32_t abox[2], bbox[2] = {64, T_BK};
  kmajor_map_dims(adims, abox, M, K);
  const CUtensorMap ta = make_tensor_map(dy, TmaDType::BF16, 2, adims, astr, abox, true);
  const CUtensorMap tb = make_tensor_map(w_down, TmaDType::BF16, 2, bdims, bstr, bbox, true);
  EpiFuse fz{};
  fz.F = F;
  fz.aux = reinterpret_cast<const __nv_bfloat16*>(gate_up);
  fz.ld_aux = ld_gu;
  launch2<false, true, FUSE_SWIGLU_BWD>(ta, tb, d_gate_up, M, F, K, ld_dgu, 1, EPI_BF16, 1, 1.f, status, stream,
                                        PeerPtrs{}, 0, 0, 0, fz);
}

void gemm_rope(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo, int M, int N, int K,
               const int* pos, const float* cos_sin, int max_pos, int rope_cols, int* status, cudaStream_t stream) {
  MB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_rope: empty problem");
  MB_REQUIRE(N % 128 == 0 && rope_cols % 128 == 0 && rope_cols <= N, "gemm_rope: heads of 128 columns");
  MB_REQUIRE(ldx % 8 == 0 && ldw % 8 == 0 && ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(cos_sin) & 15) == 0,
             "gemm_rope: alignment");
  MB_REQUIRE(pos != nullptr && cos_sin != nullptr && max_pos > 0, "gemm_rope: positions and table");
  uint64_t adims[2], astr[1] = {(uint64_t)ldx * 2}, bdims[2], bstr[1] = {(uint64_t)ldw * 2};
  uint32_t abox[2], bbox[2];
  kmajor_map_dims(adims, abox, M, K);
  kmajor_map_dims(bdims, bbox, N, K);
  const CUtensorMap ta = make_tensor_map(x, TmaDType::BF16, 2, adims, astr, abox, true);
  const CUtensorMap tb = make_tensor_map(w, TmaDType::BF16, 2, bdims, bstr, bbox, true);
  EpiFuse fz{};
  fz.pos = pos;
  fz.cs = reinterpret_cast<const float2*>(cos_sin);
  fz.max_pos = max_pos;
  fz.rope_cols = rope_cols;
  launch2<false, false, FUSE_ROPE>(ta, tb, out, M, N, K, ldo, 1, EPI_BF16, 1, 1.f, status, stream, PeerPtrs{}, 0, 0, 0,
                                   fz);
}

// ---------------------------------------------------------------------------- grouped launches
void gemm_grouped_rows(const void* A, long long lda, int total_rows, const void* const* B, long long ldb, bool b_mn,
                       void* C, long long ldc, int N, int K, const int* seg_start, const int* seg_rows, int n_seg,
                       int fuse, const void* aux, long long ld_aux, void* out2, long long ld_out2, int* status,
                       cudaStream_t stream) {
  MB_REQUIRE(n_seg >= 1 && n_seg <= MAX_GROUPS, "gemm_grouped_rows: 1..16 segments per launch");
  MB_REQUIRE(total_rows > 0 && N > 0 && K > 0, "gemm_grouped_rows: empty problem");
  MB_REQUIRE(lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0, "gemm_grouped_rows: row strides must be multiples of 8 elements");
  MB_REQUIRE(fuse == FUSE_NONE || fuse == FUSE_SWIGLU_FWD || fuse == FUSE_SWIGLU_BWD, "gemm_grouped_rows: bad fusion id");
  MB_REQUIRE(!(fuse == FUSE_SWIGLU_FWD && b_mn) && !(fuse == FUSE_SWIGLU_BWD && !b_mn),
             "gemm_grouped_rows: SwiGLU forward takes K-major weights, SwiGLU backward MN-major weights");
  uint64_t adims[2], astr[1] = {(uint64_t)lda * 2};
  uint32_t abox[2];
  kmajor_map_dims(adims, abox, total_rows, K);
  const CUtensorMap ta = make_tensor_map(A, TmaDType::BF16, 2, adims, astr, abox, true);
  GroupArgsT<GROUP_ROWS> ga{};
  ga.seg_start = seg_start;
  ga.seg_rows = seg_rows;
  ga.n_seg = n_seg;
  EpiFuse fz{};
  // N is the number of weight rows of one segment: 2F for the fused gate/up projection
  const int F = fuse == FUSE_SWIGLU_FWD ? N / 2 : N;
  if (fuse != FUSE_NONE) {
    MB_REQUIRE(F % 128 == 0, "gemm_grouped_rows: the ffn width must be a multiple of 128");
    fz.F = F;
    fz.aux = reinterpret_cast<const __nv_bfloat16*>(aux);
    fz.ld_aux = ld_aux;
    fz.out2 = reinterpret_cast<__nv_bfloat16*>(out2);
    fz.ld_out2 = ld_out2;
    MB_REQUIRE(fuse != FUSE_SWIGLU_FWD || (out2 != nullptr && ld_out2 % 8 == 0), "gemm_grouped_rows: h output");
    MB_REQUIRE(fuse != FUSE_SWIGLU_BWD || (aux != nullptr && ld_aux % 8 == 0), "gemm_grouped_rows: pre-activations");
  }
  for (int e = 0; e < n_seg; ++e) {
    uint64_t bdims[2], bstr[1] = {(uint64_t)ldb * 2};
    uint32_t bbox[2];
    if (!b_mn) { kmajor_map_dims(bdims, bbox, N, K); }
    else { bdims[0] = (uint64_t)N; bdims[1] = (uint64_t)K; bbox[0] = 64; bbox[1] = T_BK; }
    ga.bmaps[e] = make_tensor_map(B[e], TmaDType::BF16, 2, bdims, bstr, bbox, true);
  }
  const int vec_ok = (reinterpret_cast<uintptr_t>(C) & 15) == 0 ? 2 : 0;
  MB_REQUIRE(vec_ok || fuse == FUSE_NONE, "gemm_grouped_rows: fused outputs must be 16-byte aligned");
  // the kernel's N: output columns of the accumulator tiles (2F for the fused forward, whose tiles hold
  // 128 gate + 128 up columns; F for the fused backward, whose output buffer is [rows, 2F])
  const PeerPtrs none{};
  if (fuse == FUSE_SWIGLU_FWD)
    launch2<false, false, FUSE_SWIGLU_FWD, GROUP_ROWS>(ta, ga.bmaps[0], C, total_rows, N, K, ldc, 1, EPI_BF16, 1, 1.f,
                                                       status, stream, none, 0, 0, 0, fz, ga);
  else if (fuse == FUSE_SWIGLU_BWD)
    launch2<false, true, FUSE_SWIGLU_BWD, GROUP_ROWS>(ta, ga.bmaps[0], C, total_rows, N, K, ldc, 1, EPI_BF16, 1, 1.f,
                                                      status, stream, none, 0, 0, 0, fz, ga);
  else if (!b_mn)
    launch2<false, false, FUSE_NONE, GROUP_ROWS>(ta, ga.bmaps[0], C, total_rows, N, K, ldc, 1, EPI_BF16, vec_ok, 1.f,
                                                 status, stream, none, 0, 0, 0, fz, ga);
  else
    launch2<false, true, FUSE_NONE, GROUP_ROWS>(ta, ga.bmaps[0], C, total_rows, N, K, ldc, 1, EPI_BF16, vec_ok, 1.f,
                                                status, stream, none, 0, 0, 0, fz, ga);
}

void gemm_grouped_k(const void* A, long long lda, const void* B, long long ldb, float* const* C, long long ldc, int M,
                    int N, int total_rows, const int* seg_start, const int* seg_rows, int n_seg, int* status,
                    cudaStream_t stream) {
  MB_REQUIRE(n_seg >= 1 && n_seg <= MAX_GROUPS, "gemm_grouped_k: 1..16 segments per launch");
  MB_REQUIRE(total_rows > 0 && M > 0 && N > 0, "gemm_grouped_k: empty problem");
  MB_REQUIRE(lda % 8 == 0 && ldb % 8 == 0 && ldc % 4 == 0, "gemm_grouped_k: strides");
  // both operands are row-indexed buffers read transposed: A [rows, M], B [rows, N] (MN-major)
  uint64_t adims[2] = {(uint64_t)M, (uint64_t)total_rows}, astr[1] = {(uint64_t)lda * 2};
  uint64_t bdims[2] = {(uint64_t)N, (uint64_t)total_rows}, bstr[1] = {(uint64_t)ldb * 2};
  uint32_t box[2] = {64, T_BK};
  const CUtensorMap ta = make_tensor_map(A, TmaDType::BF16, 2, adims, astr, box, true);
  const CUtensorMap tb = make_tensor_map(B, TmaDType::BF16, 2, bdims, bstr, box, true);
  GroupArgsT<GROUP_K> ga{};
  ga.seg_start = seg_start;
  ga.seg_rows = seg_rows;
  ga.n_seg = n_seg;
  int vec_ok = 2;
  for (int e = 0; e < n_seg; ++e) {
    ga.cptrs[e] = C[e];
    if (reinterpret_cast<uintptr_t>(C[e]) & 15) vec_ok = 0;
  }
  launch2<true, true, FUSE_NONE, GROUP_K>(ta, tb, nullptr, M, N, total_rows, ldc, 1, EPI_F32_ACC, vec_ok, 1.f, status,
                                          stream, PeerPtrs{}, 0, 0, 0, EpiFuse{}, ga);
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
  // 2 = vector accesses through the shared-memory transpose, 1 = vector accesses straight from registers
  const int vec_ok = ((ldc * esz) % 16 == 0 && (n_scatter > 0 || (reinterpret_cast<uintptr_t>(C) & 15) == 0))
                         ? (g_coalesced_epilogue && n_scatter == 0 ? 2 : 1) : 0;
  const int kblocks = (K + T_BK - 1) / T_BK;
  int k_splits = 1;
  if (epi == EPI_F32_ATOMIC) {
    const int clusters = sm_count() / 2;
    const long long tiles = (long long)((M + T_BM - 1) / T_BM) * ((N + T_BN - 1) / T_BN);
    // Split K only where whole waves of tiles leave SM pairs idle (few tiles per pair); every extra
    // split adds a pass of atomic traffic over C, charged here as 2 % of a wave (with many tiles per
    // pair, e.g. a vocabulary-sized wgrad, splitting measured 25 % slower).
    double best = 1e30;
    for (int s = 1; s <= 8; ++s) {
      if (s > 1 && (kblocks / s < 8 || tiles >= 6LL * clusters)) break;
      const double waves = (double)((tiles * s + clusters - 1) / clusters) / s * (1.0 + 0.02 * (s - 1));
      if (waves < best * 0.97) { best = waves; k_splits = s; }
    }
  }
  // one tile per output block: the plain read-add-store gives the same sum without atomic traffic
  if (epi == EPI_F32_ATOMIC && k_splits == 1) epi = EPI_F32_ACC;
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

// C[M, N] = A[M, K] * B[N, K]^T where A is sharded by rows over `world` ranks: a_bufs.p[r] is rank r's
// full-size [M, K] buffer (symmetric memory, as mapped in this process) in which rank r has written only
// its own rows [r * M / world, (r + 1) * M / world). The launch gathers the other ranks' rows into
// a_bufs.p[rank] while it multiplies (see GROUP_GATHER above); afterwards the local buffer holds all of A.
// The caller makes sure (flag barrier) that every rank has written its rows before any rank launches,
// and that a buffer is not rewritten while a peer may still read it (alternate two buffers).
// tile_count: [M / 256] int32 in local memory, zero before the first call; `call` counts the launches
// that used this counter array so far, this one included.
void gemm_allgather_a(const PeerPtrs& a_bufs, long long lda, const void* B, long long ldb, void* C, long long ldc, int M,
                      int N, int K, int rank, int world, int* tile_count, int call, int copier_clusters, int* status,
                      cudaStream_t stream) {
  MB_REQUIRE(world >= 1 && world <= AG_MAX_RANKS && rank >= 0 && rank < world, "gemm_allgather_a: bad rank / world");
  MB_REQUIRE(M > 0 && N > 0 && K > 0 && M % (T_BM * world) == 0, "gemm_allgather_a: M must be a multiple of 256 x world");
  MB_REQUIRE(K % T_BK == 0 && lda % 8 == 0 && ldb % 8 == 0, "gemm_allgather_a: K % 64 == 0 and 16-byte row strides");
  const int clusters = sm_count() / 2;
  if (world == 1) copier_clusters = 0;
  MB_REQUIRE(copier_clusters >= (world > 1 ? 1 : 0) && copier_clusters < clusters, "gemm_allgather_a: bad copier count");
  const int vec_ok = ((ldc * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? (g_coalesced_epilogue ? 2 : 1) : 0;
  uint64_t adims[2] = {(uint64_t)K, (uint64_t)M}, astr[1] = {(uint64_t)lda * 2};
  uint64_t bdims[2] = {(uint64_t)K, (uint64_t)N}, bstr[1] = {(uint64_t)ldb * 2};
  uint32_t box[2] = {T_BK, 128};
  GroupArgsT<GROUP_GATHER> ga{};
  for (int r = 0; r < world; ++r) ga.peer[r] = make_tensor_map(a_bufs.p[r], TmaDType::BF16, 2, adims, astr, box, true);
  for (int r = world; r < AG_MAX_RANKS; ++r) ga.peer[r] = ga.peer[0];
  ga.tile_count = tile_count;
  ga.target = 2 * copier_clusters * call;
  ga.rank = rank;
  ga.world = world;
  ga.tiles_per_rank = M / T_BM / world;
  ga.copier_clusters = copier_clusters;
  ga.gather_b = 0;
  const CUtensorMap tb = make_tensor_map(B, TmaDType::BF16, 2, bdims, bstr, box, true);
  launch2<false, false, FUSE_NONE, GROUP_GATHER>(ga.peer[rank], tb, C, M, N, K, ldc, 1, EPI_BF16, vec_ok, 1.f, status, stream,
                                                PeerPtrs{}, 0, 0, 0, EpiFuse{}, ga);
}

// The same with the roles of the operands exchanged: C[M, N] = A[M, K] * B[N, K]^T where the weight B is
// sharded by output rows over the ranks (b_bufs.p[r] = rank r's full-size [N, K] buffer holding its own rows
// [r * N / world, (r + 1) * N / world)). The launch gathers the other ranks' rows of B into b_bufs.p[rank]
// while it multiplies, own column block first; afterwards the local buffer holds all of B (a later product
// with the same weight, e.g. the data gradient, can read it from there). tile_count: [N / 256].
void gemm_allgather_b(const void* A, long long lda, const PeerPtrs& b_bufs, long long ldb, void* C, long long ldc, int M,
                      int N, int K, int rank, int world, int* tile_count, int call, int copier_clusters, int* status,
                      cudaStream_t stream) {
  MB_REQUIRE(world >= 1 && world <= AG_MAX_RANKS && rank >= 0 && rank < world, "gemm_allgather_b: bad rank / world");
  MB_REQUIRE(M > 0 && N > 0 && K > 0 && N % (T_BN * world) == 0, "gemm_allgather_b: N must be a multiple of 256 x world");
  MB_REQUIRE(K % T_BK == 0 && lda % 8 == 0 && ldb % 8 == 0, "gemm_allgather_b: K % 64 == 0 and 16-byte row strides");
  const int clusters = sm_count() / 2;
  if (world == 1) copier_clusters = 0;
  MB_REQUIRE(copier_clusters >= (world > 1 ? 1 : 0) && copier_clusters < clusters, "gemm_allgather_b: bad copier count");
  const int vec_ok = ((ldc * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? (g_coalesced_epilogue ? 2 : 1) : 0;
  uint64_t adims[2] = {(uint64_t)K, (uint64_t)M}, astr[1] = {(uint64_t)lda * 2};
  uint64_t bdims[2] = {(uint64_t)K, (uint64_t)N}, bstr[1] = {(uint64_t)ldb * 2};
  uint32_t box[2] = {T_BK, 128};
  GroupArgsT<GROUP_GATHER> ga{};
  for (int r = 0; r < world; ++r) ga.peer[r] = make_tensor_map(b_bufs.p[r], TmaDType::BF16, 2, bdims, bstr, box, true);
  for (int r = world; r < AG_MAX_RANKS; ++r) ga.peer[r] = ga.peer[0];
  ga.tile_count = tile_count;
  ga.target = 2 * copier_clusters * call;
  ga.rank = rank;
  ga.world = world;
  ga.tiles_per_rank = N / T_BN / world;
  ga.copier_clusters = copier_clusters;
  ga.gather_b = 1;
  const CUtensorMap ta = make_tensor_map(A, TmaDType::BF16, 2, adims, astr, box, true);
  launch2<false, false, FUSE_NONE, GROUP_GATHER>(ta, ga.peer[rank], C, M, N, K, ldc, 1, EPI_BF16, vec_ok, 1.f, status, stream,
                                                PeerPtrs{}, 0, 0, 0, EpiFuse{}, ga);
}

}  // namespace mb
