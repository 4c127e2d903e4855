// Look-up-table GEMMs over ternary weights with int8 activations: TL1 (weight pairs, 9-entry table
// per pair) and TL2 (weight triples, 27-entry table per triple), the arithmetic of the reference's
// kernel_tl (src/kernel_tl.cpp:13-168) in a weight-shared layout W[N, K]:
//
//     y[m, n] = (sum_k t(W[n, k]) * q(x[m, k])) / s_m,   q = round-half-away(x * s_m),  s_m = 127 / max|x_m|
//
// with exact int32 accumulation. One CTA owns one activation row m and a tile of outputs: it
// quantises the row, builds the row's tables in shared memory (entry (w_0 .. w_{g-1}) of group G is
// sum_j w_j * q[G*g + j], first weight = most significant base-3 digit; |entry| <= 381 fits int16),
// then every thread walks the packed trits of its output row and adds one table entry per group
// instead of g multiply-adds. Trits are 2-bit codes t + 1, four per byte, first weight in bits 0-1.
// The production ternary path is the I2_S dequant GEMM on tensor cores; these kernels exist because
// the table formulation is part of the reference's kernel set.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace mb {
namespace {

template <int G>
__global__ void __launch_bounds__(256) tl_gemm_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ x,
                                                     float* __restrict__ y, int N, int K) {
  constexpr int E = G == 2 ? 9 : 27;
  extern __shared__ int16_t smem_tl[];
  int16_t* q = smem_tl;                     // [K] quantised activations
  int16_t* lut = smem_tl + ((K + 7) & ~7);  // [K / G][E]
  __shared__ float red[32];
  const int m = blockIdx.y;
  const float* xr = x + (long long)m * K;
  float amax = 0.f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(xr[k]));
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) amax = fmaxf(amax, red[i]);
  const float scale = 127.f / fmaxf(amax, 1e-10f);
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const float v = xr[k];
    float r = floorf(fabsf(v) * scale + 0.5f);        // round half away from zero
    r = fminf(r, 127.f);
    q[k] = (int16_t)(v < 0.f ? -r : r);
  }
  __syncthreads();
  const int groups = K / G;
  for (int i = threadIdx.x; i < groups * E; i += blockDim.x) {
    const int grp = i / E, e = i - grp * E;
    int s;
    if (G == 2) {
      s = (e / 3 - 1) * q[grp * 2] + (e % 3 - 1) * q[grp * 2 + 1];
    } else {
      s = (e / 9 - 1) * q[grp * 3] + ((e / 3) % 3 - 1) * q[grp * 3 + 1] + (e % 3 - 1) * q[grp * 3 + 2];
    }
    lut[i] = (int16_t)s;
  }
  __syncthreads();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const uint8_t* row = packed + (long long)n * (K / 4);
  int acc = 0;
  if (G == 2) {
    // one byte = two pairs
    for (int b = 0; b < K / 4; ++b) {
      const unsigned v = row[b];
      const int i0 = (v & 3) * 3 + ((v >> 2) & 3);
      const int i1 = ((v >> 4) & 3) * 3 + ((v >> 6) & 3);
      acc += lut[(2 * b) * E + i0] + lut[(2 * b + 1) * E + i1];
    }
  } else {
    // three bytes = twelve trits = four triples
    for (int t = 0; t < K / 12; ++t) {
      const unsigned v = row[3 * t] | (row[3 * t + 1] << 8) | (row[3 * t + 2] << 16);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const unsigned c = (v >> (6 * j)) & 63u;
        const int idx = (c & 3) * 9 + ((c >> 2) & 3) * 3 + ((c >> 4) & 3);
        acc += lut[(4 * t + j) * E + idx];
      }
    }
  }
  y[(long long)m * N + n] = (float)acc / scale;
}

}  // namespace

void tl_gemm(const uint8_t* packed, const float* x, float* y, int M, int N, int K, int group, cudaStream_t stream) {
  MB_REQUIRE(group == 2 || group == 3, "tl_gemm: group must be 2 (TL1) or 3 (TL2)");
  MB_REQUIRE(K % 4 == 0 && (group == 2 || K % 12 == 0), "tl_gemm: K must be a multiple of 4 (TL1) / 12 (TL2)");
  if (M == 0 || N == 0) return;
  const int entries = group == 2 ? 9 : 27;
  const size_t smem = (size_t)(((K + 7) & ~7) + (K / group) * entries) * sizeof(int16_t);
  MB_REQUIRE(smem <= 200 * 1024, "tl_gemm: the row's tables do not fit into shared memory (K too large)");
  const dim3 grid((N + 255) / 256, M);
  if (group == 2) {
    static bool configured = false;
    if (!configured) {
      MB_CUDA_CHECK(cudaFuncSetAttribute(tl_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      configured = true;
    }
    tl_gemm_kernel<2><<<grid, 256, smem, stream>>>(packed, x, y, N, K);
  } else {
    static bool configured = false;
    if (!configured) {
      MB_CUDA_CHECK(cudaFuncSetAttribute(tl_gemm_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      configured = true;
    }
    tl_gemm_kernel<3><<<grid, 256, smem, stream>>>(packed, x, y, N, K);
  }
  count_launch();
  check_launch();
}

}  // namespace mb
