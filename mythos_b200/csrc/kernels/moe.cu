// Mixture-of-experts routing and the dispatch / combine exchange.
//
//   moe_topk      per token: top-k experts by router probability (probabilities come from a
//                 softmax over ALL experts and are used un-renormalised as combine weights, as in
//                 the reference's softmax_with_topk, src/moe_variants.cpp:25-62) and a slot for the
//                 token inside each chosen expert's batch (atomic counter per expert).
//   moe_dispatch  permutation + all-to-all in one kernel: every (token, k) row is stored straight
//                 into the receive buffer of the rank that owns the expert (peer store over NVLink;
//                 with one rank, a local permutation), grouped by (source rank, local expert).
//   moe_combine   all-to-all + weighted sum in one kernel: out[t] = sum_k w[t,k] * y[row(t,k)], the
//                 rows read from the owning ranks' output buffers (peer loads); optionally also
//                 dw[t,k] = <dout[t], y[row(t,k)]> for the backward pass.
//
// Together they implement the semantics of moe_dispatch_batched (src/moe_variants.cpp:695-755:
// group tokens per expert, one FFN call per expert, weighted scatter-add; no token is dropped)
// and replace cuda_moe_gather_kernel (src/kernels/cuda_kernels.cu:162-185).
//
// Receive-buffer layout on rank r: `world` segments of `cap` rows, segment s holding what rank s
// sent, rows ordered by local expert; send_off[e] is the sender's row offset of expert e inside
// its segment on the owning rank.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace mb {
namespace {

constexpr int MOE_MAX_E = 64;
constexpr int MOE_MAX_K = 8;

__global__ void moe_topk_kernel(const float* __restrict__ probs, int T, int E, int k, int* __restrict__ topk_idx,
                                int* __restrict__ slot, int* __restrict__ counts) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float p[MOE_MAX_E];
  for (int e = 0; e < E; ++e) p[e] = probs[(long long)t * E + e];
  for (int j = 0; j < k; ++j) {
    int best = 0;
    float bv = -1.f;
    for (int e = 0; e < E; ++e)
      if (p[e] > bv) { bv = p[e]; best = e; }  // first maximum wins
    p[best] = -2.f;
    topk_idx[(long long)t * k + j] = best;
    slot[(long long)t * k + j] = atomicAdd(&counts[best], 1);
  }
}

__global__ void moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx,
                                    const int* __restrict__ slot, const int* __restrict__ send_off,
                                    const float* __restrict__ row_scale, PeerPtrs recv, int T, int k, int dim,
                                    int experts_per_rank, int rank, long long cap, const int* __restrict__ send_limit) {
  const int per_row = dim >> 3;
  const long long total = (long long)T * k * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long tk = i / per_row;
    const int c = (int)(i % per_row) * 8;
    const int t = (int)(tk / k);
    const int e = topk_idx[tk];
    const int owner = e / experts_per_rank;
    const long long row = (long long)rank * cap + send_off[e] + slot[tk];
    // a row past the end of the expert's (clamped) segment does not fit into the owner's buffer: it is
    // not sent (moe_offsets has raised the status word for this step)
    if (send_limit != nullptr && send_off[e] + slot[tk] >= send_limit[e]) continue;
    bf16x8 v = ldg8(x, (long long)t * dim + c);
    if (row_scale) {
      float f[8];
      unpack8(v, f);
      const float s = row_scale[tk];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= s;
      v = pack8(f);
    }
    stg8(recv.p[owner], row * dim + c, v);
  }
}

// One warp per token.
__global__ void moe_combine_kernel(PeerPtrs ybuf, const int* __restrict__ topk_idx, const int* __restrict__ slot,
                                   const int* __restrict__ send_off, const float* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ out,
                                   float* __restrict__ dw, int T, int k, int dim, int experts_per_rank, int rank,
                                   long long cap, const int* __restrict__ send_limit) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const __nv_bfloat16* rows[MOE_MAX_K];
  float wk[MOE_MAX_K];
  for (int j = 0; j < k; ++j) {
    const int e = topk_idx[t * k + j];
    const long long row = (long long)rank * cap + send_off[e] + slot[t * k + j];
    const bool fits = send_limit == nullptr || send_off[e] + slot[t * k + j] < send_limit[e];
    rows[j] = fits ? reinterpret_cast<const __nv_bfloat16*>(ybuf.p[e / experts_per_rank]) + row * dim : nullptr;
    wk[j] = w ? w[t * k + j] : 1.f;
  }
  float dots[MOE_MAX_K];
  for (int j = 0; j < k; ++j) dots[j] = 0.f;
  for (int c = lane * 8; c < dim; c += 256) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    float g[8];
    if (dw) unpack8(ldg8(dout, t * dim + c), g);
    for (int j = 0; j < k; ++j) {
      float y[8];
      if (rows[j] == nullptr) continue;    // the row was not sent (receive buffer full): contributes nothing
      unpack8(ldg8(rows[j], c), y);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        acc[i] += wk[j] * y[i];
        if (dw) dots[j] += g[i] * y[i];
      }
    }
    if (out) stg8(out, t * dim + c, pack8(acc));
  }
  if (dw) {
    for (int j = 0; j < k; ++j) {
      const float d = warp_sum(dots[j]);
      if (lane == 0) dw[t * k + j] = d;
    }
  }
}

// ------------------------------------------------------------------------------ device-side router
// One thread per token: softmax over the E router logits (fp32), top-k by probability (first maximum
// wins), combine weights w = p[chosen] (not renormalised), a slot inside each chosen expert's batch and
// the statistics of the load-balance loss: counts[e] (tokens routed to e) and psum[e] (sum of p[t, e]).
// Slots of one expert are handed out warp-aggregated (one atomic per distinct expert per warp).
__global__ void moe_route_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int T, int E, int k,
                                 float* __restrict__ probs, int* __restrict__ topk_idx, int* __restrict__ slot,
                                 float* __restrict__ w, int* __restrict__ counts, float* __restrict__ psum) {
  __shared__ float s_psum[MOE_MAX_E];
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_psum[e] = 0.f;
  __syncthreads();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const bool live = t < T;
  float p[MOE_MAX_E];
  if (live) {
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) {
      p[e] = __bfloat162float(logits[(long long)t * ld + e]);
      mx = fmaxf(mx, p[e]);
    }
    float sum = 0.f;
    for (int e = 0; e < E; ++e) {
      p[e] = __expf(p[e] - mx);
      sum += p[e];
    }
    const float inv = 1.f / sum;
    for (int e = 0; e < E; ++e) {
      p[e] *= inv;
      probs[(long long)t * E + e] = p[e];
      atomicAdd(&s_psum[e], p[e]);
    }
  }
  for (int j = 0; j < k; ++j) {
    int best = -1;
    float bv = -1.f;
    if (live) {
      best = 0;
      for (int e = 0; e < E; ++e)
        if (p[e] > bv) { bv = p[e]; best = e; }
      p[best] = -2.f;
    }
    // lanes of the warp that chose the same expert share one atomic
    const unsigned peers = __match_any_sync(0xffffffffu, best);
    const int leader = __ffs(peers) - 1;
    int base = 0;
    if (lane == leader && best >= 0) base = atomicAdd(&counts[best], __popc(peers));
    base = __shfl_sync(0xffffffffu, base, leader);
    if (live) {
      topk_idx[(long long)t * k + j] = best;
      slot[(long long)t * k + j] = base + __popc(peers & ((1u << lane) - 1u));
      w[(long long)t * k + j] = bv;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) atomicAdd(&psum[e], s_psum[e]);
}

// dlogits[t, e] = p_e (g_e - sum_e' p_e' g_e') with g_e = sum_j dw[t, j] [idx[t, j] == e] + coef[e]
// (coef carries the load-balance term). Written as bf16 with `ld` columns, padding columns zero.
__global__ void moe_route_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ topk_idx,
                                     const float* __restrict__ dw, const float* __restrict__ coef, int T, int E, int k,
                                     __nv_bfloat16* __restrict__ dlogits, int ld) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float g[MOE_MAX_E];
  for (int e = 0; e < E; ++e) g[e] = coef ? coef[e] : 0.f;
  for (int j = 0; j < k; ++j) g[topk_idx[(long long)t * k + j]] += dw[(long long)t * k + j];
  float dot = 0.f;
  for (int e = 0; e < E; ++e) dot += probs[(long long)t * E + e] * g[e];
  for (int e = 0; e < ld; ++e)
    dlogits[(long long)t * ld + e] = __float2bfloat16(e < E ? probs[(long long)t * E + e] * (g[e] - dot) : 0.f);
}

// Every rank stores its per-expert counts into row `rank` of the count table of every rank.
__global__ void moe_publish_counts_kernel(const int* __restrict__ counts, PeerPtrs tables, int world, int E, int rank) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= world * E) return;
  const int r = i / E, e = i % E;
  reinterpret_cast<int*>(tables.p[r])[rank * E + e] = counts[e];
}

// From the table all_counts[world][E] (identical on every rank after the exchange): the segments of
// this rank's experts in its receive buffer (start aligned to 256 rows, rows = tokens from all sources,
// sources in rank order) and, for every expert, the first row this rank writes on the expert's owner.
// A segment that would not fit into `cap` rows raises the status word (routing is drop-free here).
__global__ void moe_offsets_kernel(const int* __restrict__ all_counts, int world, int E, int epr, int rank, int cap,
                                   int* __restrict__ seg_start, int* __restrict__ seg_rows,
                                   int* __restrict__ send_base, int* __restrict__ send_limit, int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int cap256 = cap / 256 * 256;      // whole 256-row tiles only: the grouped GEMMs store full tiles
  for (int r = 0; r < world; ++r) {
    int start = 0;
    for (int le = 0; le < epr; ++le) {
      const int e = r * epr + le;
      int rows = 0, before = 0;
      for (int s = 0; s < world; ++s) {
        if (s < rank) before += all_counts[s * E + e];
        rows += all_counts[s * E + e];
      }
      // A segment is cut where the owner's buffer ends; senders skip the rows past that point, so a
      // full buffer costs tokens (and raises the status word below) but never an out-of-bounds store.
      const int room = start < cap256 ? cap256 - start : 0;
      const int kept = rows < room ? rows : room;
      send_base[e] = start + before;
      if (send_limit) send_limit[e] = start + kept;
      if (r == rank) {
        seg_start[le] = start < cap256 ? start : 0;
        seg_rows[le] = kept;
      }
      start += (rows + 255) / 256 * 256;
    }
    if (start > cap256 && status) atomicCAS(status, 0, 2 | (60 << 16));  // bad argument, site 60;
  }
}

// Zero the rows between each segment's end and the next multiple of 256 in up to two row buffers.
__global__ void moe_zero_pad_kernel(const int* __restrict__ seg_start, const int* __restrict__ seg_rows, int dim,
                                    __nv_bfloat16* __restrict__ a, __nv_bfloat16* __restrict__ b, int cap) {
  const int le = blockIdx.y;
  const int rows = seg_rows[le];
  const long long first = (long long)seg_start[le] + rows;
  long long last = (long long)seg_start[le] + (rows + 255) / 256 * 256;
  if (last > cap) last = cap;
  const int per_row = dim >> 3;
  const long long n = (last - first) * per_row;
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long off = (first + i / per_row) * dim + (i % per_row) * 8;
    if (a) *reinterpret_cast<uint4*>(a + off) = z;
    if (b) *reinterpret_cast<uint4*>(b + off) = z;
  }
}

}  // namespace

void moe_route(const void* logits, int ld, int T, int E, int k, float* probs, int* topk_idx, int* slot, float* w,
               int* counts, float* psum, cudaStream_t stream) {
  MB_REQUIRE(E >= 1 && E <= MOE_MAX_E && ld >= E, "moe_route: at most 64 experts");
  MB_REQUIRE(k >= 1 && k <= MOE_MAX_K && k <= E, "moe_route: top-k must be 1..8 and <= experts");
  if (T == 0) return;
  moe_route_kernel<<<ceil_div(T, 128), 128, 0, stream>>>((const __nv_bfloat16*)logits, ld, T, E, k, probs, topk_idx, slot,
                                                        w, counts, psum);
  count_launch();
  check_launch();
}

void moe_route_bwd(const float* probs, const int* topk_idx, const float* dw, const float* coef, int T, int E, int k,
                   void* dlogits, int ld, cudaStream_t stream) {
  MB_REQUIRE(E >= 1 && E <= MOE_MAX_E && ld >= E && k <= MOE_MAX_K, "moe_route_bwd: bad sizes");
  if (T == 0) return;
  moe_route_bwd_kernel<<<ceil_div(T, 128), 128, 0, stream>>>(probs, topk_idx, dw, coef, T, E, k, (__nv_bfloat16*)dlogits, ld);
  count_launch();
  check_launch();
}

void moe_publish_counts(const int* counts, const PeerPtrs& tables, int world, int E, int rank, cudaStream_t stream) {
  MB_REQUIRE(world >= 1 && world <= MAX_PEERS && E <= MOE_MAX_E, "moe_publish_counts: bad sizes");
  moe_publish_counts_kernel<<<ceil_div(world * E, 128), 128, 0, stream>>>(counts, tables, world, E, rank);
  count_launch();
  check_launch();
}

void moe_offsets(const int* all_counts, int world, int E, int rank, int cap, int* seg_start, int* seg_rows,
                 int* send_base, int* status, cudaStream_t stream, int* send_limit) {
  MB_REQUIRE(world >= 1 && E % world == 0 && E <= MOE_MAX_E, "moe_offsets: experts must divide over the ranks");
  moe_offsets_kernel<<<1, 32, 0, stream>>>(all_counts, world, E, E / world, rank, cap, seg_start, seg_rows, send_base,
                                           send_limit, status);
  count_launch();
  check_launch();
}

void moe_zero_pad(const int* seg_start, const int* seg_rows, int n_seg, int dim, void* a, void* b, int cap,
                  cudaStream_t stream) {
  MB_REQUIRE(dim % 8 == 0 && n_seg >= 1, "moe_zero_pad: dim must be a multiple of 8");
  moe_zero_pad_kernel<<<dim3(16, n_seg), 256, 0, stream>>>(seg_start, seg_rows, dim, (__nv_bfloat16*)a, (__nv_bfloat16*)b, cap);
  count_launch();
  check_launch();
}

void moe_topk(const float* probs, int T, int E, int k, int* topk_idx, int* slot, int* counts, cudaStream_t stream) {
  MB_REQUIRE(E >= 1 && E <= MOE_MAX_E, "moe_topk: at most 64 experts");
  MB_REQUIRE(k >= 1 && k <= MOE_MAX_K && k <= E, "moe_topk: top-k must be 1..8 and <= experts");
  if (T == 0) return;
  moe_topk_kernel<<<ceil_div(T, 128), 128, 0, stream>>>(probs, T, E, k, topk_idx, slot, counts);
  count_launch();
  check_launch();
}

void moe_dispatch(const void* x, const int* topk_idx, const int* slot, const int* send_off, const float* row_scale,
                  const PeerPtrs& recv, int T, int k, int dim, int experts_per_rank, int rank, long long cap,
                  cudaStream_t stream, const int* send_limit) {
  MB_REQUIRE(dim % 8 == 0, "moe_dispatch: dim must be a multiple of 8");
  if (T == 0) return;
  long long g = ((long long)T * k * (dim / 8) + 255) / 256;
  const long long capg = (long long)sm_count() * 16;
  if (g > capg) g = capg;
  moe_dispatch_kernel<<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)x, topk_idx, slot, send_off, row_scale, recv, T,
                                                  k, dim, experts_per_rank, rank, cap, send_limit);
  count_launch();
  check_launch();
}

void moe_combine(const PeerPtrs& ybuf, const int* topk_idx, const int* slot, const int* send_off, const float* w,
                 const void* dout, void* out, float* dw, int T, int k, int dim, int experts_per_rank, int rank,
                 long long cap, cudaStream_t stream, const int* send_limit) {
  MB_REQUIRE(dim % 8 == 0, "moe_combine: dim must be a multiple of 8");
  MB_REQUIRE(k <= MOE_MAX_K, "moe_combine: top-k too large");
  MB_REQUIRE(dw == nullptr || dout != nullptr, "moe_combine: dw needs dout");
  if (T == 0) return;
  moe_combine_kernel<<<ceil_div(T, 8), 256, 0, stream>>>(ybuf, topk_idx, slot, send_off, w, (const __nv_bfloat16*)dout,
                                                         (__nv_bfloat16*)out, dw, T, k, dim, experts_per_rank, rank,
                                                         cap, send_limit);
  count_launch();
  check_launch();
}

}  // namespace mb
