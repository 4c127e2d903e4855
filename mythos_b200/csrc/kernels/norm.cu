// RMSNorm (optionally fused with the residual add that precedes it) forward and backward,
// and LayerNorm forward. bf16 in/out, fp32 math, 128-bit loads, one CTA per row with the row
// cached in registers so x is read from HBM once.
// Formula parity: y = x * (mean(x^2)+eps)^-1/2 * gamma (reference src/math.cpp:182-205);
// backward as in src/autograd.cpp:1129-1160 but with the eps that the forward used.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace mb {
namespace {

constexpr int MAXC = 4;  // most 8-element chunks cached per thread (template NC <= MAXC)

template <int NC>
__global__ void __launch_bounds__(1024) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                   const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ resid_out, float* __restrict__ rstd_out, int dim,
                                   float eps) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const int nchunk = dim >> 3;
  float h[NC][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      unpack8(ldg8(x, row * dim + ch * 8), h[c]);
      if (residual) {
        float r[8];
        unpack8(ldg8(residual, row * dim + ch * 8), r);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[c][i] += r[i];
      }
      if (resid_out) {
        const bf16x8 hv = pack8(h[c]);
        stg8(resid_out, row * dim + ch * 8, hv);
        unpack8(hv, h[c]);  // normalise the rounded value that later layers will see
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += h[c][i] * h[c][i];
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / dim + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      float g[8], o[8];
      unpack8(ldg8(gamma, ch * 8), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = h[c][i] * rstd * g[i];
      stg8(y, row * dim + ch * 8, pack8(o));
    }
  }
}

// Each CTA walks rows blockIdx.x, +gridDim.x, ... and keeps its dgamma partial in registers.
template <int NC>
__global__ void __launch_bounds__(512) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ rstd,
                                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma_partial, int rows,
                                   int dim, const __nv_bfloat16* __restrict__ dres) {
  __shared__ float scratch[32];
  const int nchunk = dim >> 3;
  float g[NC][8], dg[NC][8];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) dg[c][i] = 0.f;
    if (ch < nchunk) unpack8(ldg8(gamma, ch * 8), g[c]);
  }
  // The loads of the next row (x, dy, residual gradient, rstd) are issued before the current row is
  // reduced, so a CTA always has one row in flight behind its block-wide sum: without this every row
  // paid two dependent trips to memory (x / dy, then the residual gradient after the reduction).
  bf16x8 nx[NC], ndy[NC], nres[NC];
  float nrs = 0.f;
  auto fetch = [&](long long row) {
    nrs = rstd[row];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunk) {
        nx[c] = ldg8(x, row * dim + ch * 8);
        ndy[c] = ldg8(dy, row * dim + ch * 8);
        if (dres) nres[c] = ldg8(dres, row * dim + ch * 8);
      }
    }
  };
  constexpr bool AHEAD = NC <= 2;             // wide rows (NC = 4) would spill with a second row in registers
  if (AHEAD && (long long)blockIdx.x < rows) fetch(blockIdx.x);
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    if (!AHEAD) fetch(row);
    const float rs = nrs;
    float xh[NC][8], dyg[NC][8], er[NC][8];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunk) {
        float d[8];
        unpack8(nx[c], xh[c]);
        unpack8(ndy[c], d);
        if (dres) unpack8(nres[c], er[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[c][i] *= rs;
          dg[c][i] += d[i] * xh[c][i];
          dyg[c][i] = d[i] * g[c][i];
          dot += dyg[c][i] * xh[c][i];
        }
      }
    }
    if (AHEAD && row + gridDim.x < rows) fetch(row + gridDim.x);
    dot = block_sum(dot, scratch) / dim;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunk) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rs * (dyg[c][i] - xh[c][i] * dot);
        if (dres) {  // gradient arriving through the residual stream, added here instead of in a second pass
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += er[c][i];
        }
        stg8(dx, row * dim + ch * 8, pack8(o));
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      float* p = dgamma_partial + (long long)blockIdx.x * dim + ch * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) p[i] = dg[c][i];
    }
  }
}

__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int n_partial, int dim,
                              int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= dim) return;
  float s = 0.f;
  for (int p = 0; p < n_partial; ++p) s += partial[(long long)p * dim + col];
  out[col] = accumulate ? out[col] + s : s;
}

template <int NC>
__global__ void __launch_bounds__(1024) layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                                     const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y, int dim,
                                     float eps) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const int nchunk = dim >> 3;
  float h[NC][8];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      unpack8(ldg8(x, row * dim + ch * 8), h[c]);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += h[c][i];
    }
  }
  const float mean = block_sum(s, scratch) / dim;
  float vs = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = h[c][i] - mean;
        vs += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(vs, scratch) / dim + eps);
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      float g[8], b[8], o[8];
      unpack8(ldg8(gamma, ch * 8), g);
      if (beta) unpack8(ldg8(beta, ch * 8), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (h[c][i] - mean) * rstd * g[i] + (beta ? b[i] : 0.f);
      stg8(y, row * dim + ch * 8, pack8(o));
    }
  }
}

// LayerNorm backward. mean and rstd are recomputed from x (one extra reduction, no saved statistics):
//   xhat = (x - mean) rstd,  a = gamma dy,  dx = rstd (a - mean(a) - xhat mean(a xhat)),
//   dgamma += dy xhat,  dbeta += dy.
// Each CTA walks rows blockIdx.x, +gridDim.x, ... and keeps its dgamma / dbeta partials in registers;
// partial[blockIdx.x] = [dgamma | dbeta] (2 * dim floats), summed over CTAs by the column-sum kernel.
template <int NC>
__global__ void __launch_bounds__(512) layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                     const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ dx,
                                     float* __restrict__ partial, int rows, int dim, float eps) {
  __shared__ float scratch[32];
  const int nchunk = dim >> 3;
  float g[NC][8], dg[NC][8], db[NC][8];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) { dg[c][i] = 0.f; db[c][i] = 0.f; g[c][i] = 0.f; }
    if (ch < nchunk) unpack8(ldg8(gamma, ch * 8), g[c]);
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    float h[NC][8], d[NC][8];
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunk) {
        unpack8(ldg8(x, row * dim + ch * 8), h[c]);
        unpack8(ldg8(dy, row * dim + ch * 8), d[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += h[c][i];
      }
    }
    const float mean = block_sum(s, scratch) / dim;
    float vs = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunk) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          h[c][i] -= mean;
          vs += h[c][i] * h[c][i];
        }
      }
    }
    const float rstd = rsqrtf(block_sum(vs, scratch) / dim + eps);
    float sa = 0.f, sax = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunk) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          h[c][i] *= rstd;                       // xhat
          dg[c][i] += d[c][i] * h[c][i];
          db[c][i] += d[c][i];
          d[c][i] *= g[c][i];                    // a
          sa += d[c][i];
          sax += d[c][i] * h[c][i];
        }
      }
    }
    sa = block_sum(sa, scratch) / dim;
    sax = block_sum(sax, scratch) / dim;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunk) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (d[c][i] - sa - h[c][i] * sax);
        stg8(dx, row * dim + ch * 8, pack8(o));
      }
    }
  }
  float* pr = partial + (long long)blockIdx.x * 2 * dim;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        pr[ch * 8 + i] = dg[c][i];
        pr[dim + ch * 8 + i] = db[c][i];
      }
    }
  }
}

int norm_threads(int dim, int max_threads = 1024) {
  MB_REQUIRE(dim % 8 == 0, "norm: dim must be a multiple of 8");
  const int chunks = dim / 8;
  MB_REQUIRE(chunks <= MAXC * max_threads, "norm: row too long for this kernel");
  int t = chunks <= 512 ? chunks : (chunks <= 2048 ? 512 : 1024);  // one chunk per thread for short rows
  t = ((t + 31) / 32) * 32;
  if (t > max_threads) t = max_threads;
  return t < 32 ? 32 : t;
}

int norm_nc(int dim, int threads) { return (dim / 8 + threads - 1) / threads; }

#define MB_NORM_DISPATCH(nc, KERNEL, ...)            \
  do {                                               \
    if ((nc) <= 1) KERNEL<1> __VA_ARGS__;            \
    else if ((nc) == 2) KERNEL<2> __VA_ARGS__;       \
    else KERNEL<4> __VA_ARGS__;                      \
  } while (0)

}  // namespace

void rmsnorm_fwd(const void* x, const void* residual, const void* gamma, void* y, void* resid_out, float* rstd,
                 int rows, int dim, float eps, cudaStream_t stream) {
  if (rows == 0) return;
  const int th = norm_threads(dim);
  MB_NORM_DISPATCH(norm_nc(dim, th), rmsnorm_fwd_kernel,
                   <<<rows, th, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)residual,
                                             (const __nv_bfloat16*)gamma, (__nv_bfloat16*)y,
                                             (__nv_bfloat16*)resid_out, rstd, dim, eps));
  count_launch();
  check_launch();
}

void rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx, float* dgamma_partial,
                 int rows, int dim, int n_partial, cudaStream_t stream, const void* dres) {
  if (rows == 0) return;
  MB_REQUIRE(dres != dx, "rmsnorm_bwd: the residual gradient must not alias dx");
  const int th = norm_threads(dim, 512);  // the backward keeps four row-sized arrays in registers
  MB_NORM_DISPATCH(norm_nc(dim, th), rmsnorm_bwd_kernel,
                   <<<n_partial, th, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                  (const __nv_bfloat16*)gamma, rstd, (__nv_bfloat16*)dx,
                                                  dgamma_partial, rows, dim, (const __nv_bfloat16*)dres));
  count_launch();
  check_launch();
}

void rmsnorm_bwd_reduce(const float* dgamma_partial, float* dgamma, int n_partial, int dim, bool accumulate,
                        cudaStream_t stream) {
  colsum_kernel<<<ceil_div(dim, 128), 128, 0, stream>>>(dgamma_partial, dgamma, n_partial, dim, accumulate ? 1 : 0);
  count_launch();
  check_launch();
}

void layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, int rows, int dim, float eps,
                   cudaStream_t stream) {
  if (rows == 0) return;
  const int th = norm_threads(dim);
  MB_NORM_DISPATCH(norm_nc(dim, th), layernorm_fwd_kernel,
                   <<<rows, th, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma,
                                             (const __nv_bfloat16*)beta, (__nv_bfloat16*)y, dim, eps));
  count_launch();
  check_launch();
}

// partial: [n_partial, 2 * dim] fp32; sum it with rmsnorm_bwd_reduce(partial, dgamma_dbeta, n_partial, 2 * dim).
void layernorm_bwd(const void* dy, const void* x, const void* gamma, void* dx, float* partial, int n_partial, int rows,
                   int dim, float eps, cudaStream_t stream) {
  MB_REQUIRE(n_partial > 0, "layernorm_bwd: needs at least one partial row");
  const int th = norm_threads(dim, 512);
  MB_NORM_DISPATCH(norm_nc(dim, th), layernorm_bwd_kernel,
                   <<<n_partial, th, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                  (const __nv_bfloat16*)gamma, (__nv_bfloat16*)dx, partial, rows, dim, eps));
  count_launch();
  check_launch();
}

}  // namespace mb
