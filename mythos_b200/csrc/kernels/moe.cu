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
                                    int experts_per_rank, int rank, long long cap) {
  const int per_row = dim >> 3;
  const long long total = (long long)T * k * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long tk = i / per_row;
    const int c = (int)(i % per_row) * 8;
    const int t = (int)(tk / k);
    const int e = topk_idx[tk];
    const int owner = e / experts_per_rank;
    const long long row = (long long)rank * cap + send_off[e] + slot[tk];
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
                                   long long cap) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const __nv_bfloat16* rows[MOE_MAX_K];
  float wk[MOE_MAX_K];
  for (int j = 0; j < k; ++j) {
    const int e = topk_idx[t * k + j];
    const long long row = (long long)rank * cap + send_off[e] + slot[t * k + j];
    rows[j] = reinterpret_cast<const __nv_bfloat16*>(ybuf.p[e / experts_per_rank]) + row * dim;
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

}  // namespace

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
                  cudaStream_t stream) {
  MB_REQUIRE(dim % 8 == 0, "moe_dispatch: dim must be a multiple of 8");
  if (T == 0) return;
  long long g = ((long long)T * k * (dim / 8) + 255) / 256;
  const long long capg = (long long)sm_count() * 16;
  if (g > capg) g = capg;
  moe_dispatch_kernel<<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)x, topk_idx, slot, send_off, row_scale, recv, T,
                                                  k, dim, experts_per_rank, rank, cap);
  count_launch();
  check_launch();
}

void moe_combine(const PeerPtrs& ybuf, const int* topk_idx, const int* slot, const int* send_off, const float* w,
                 const void* dout, void* out, float* dw, int T, int k, int dim, int experts_per_rank, int rank,
                 long long cap, cudaStream_t stream) {
  MB_REQUIRE(dim % 8 == 0, "moe_combine: dim must be a multiple of 8");
  MB_REQUIRE(k <= MOE_MAX_K, "moe_combine: top-k too large");
  MB_REQUIRE(dw == nullptr || dout != nullptr, "moe_combine: dw needs dout");
  if (T == 0) return;
  moe_combine_kernel<<<ceil_div(T, 8), 256, 0, stream>>>(ybuf, topk_idx, slot, send_off, w, (const __nv_bfloat16*)dout,
                                                         (__nv_bfloat16*)out, dw, T, k, dim, experts_per_rank, rank,
                                                         cap);
  count_launch();
  check_launch();
}

}  // namespace mb
