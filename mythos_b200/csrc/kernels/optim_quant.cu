// Optimizer and train-in-format kernels.
//   * AdamW with decoupled decay in the standard form: p -= lr*wd*p; p -= lr * (m/bc1) / (sqrt(v/bc2) + eps)
//     with bc1 = 1-beta1^t, bc2 = 1-beta2^t. This deviates on purpose from the reference
//     (src/optimizer.cpp:91-119), which computes lr*sqrt(bc2)/bc1 * m/(sqrt(v/bc2)+eps) and so applies
//     the second-moment correction twice (a sqrt(1-beta2^t) smaller step early on, ~30x at t=1).
//     The state files (.opt, CHPK) are interchangeable; the trajectories are not.
//   * STE fake quantisation: nearest centroid in a sorted codebook (first minimum wins, as the
//     brute-force search of src/codebook.cpp:172-186 does), I2_S ternary with absmean scale.
//   * Codebook EMA statistics (counts / sums per centroid), src/codebook.cpp:137-170.
//   * fp32 sum of squares (global-norm clip, src/trainer.cpp:608-630) and dtype casts.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace mb {
namespace {

__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ g, __nv_bfloat16* __restrict__ p_bf16, long long n, AdamWArgs a,
                             const float* __restrict__ clip_coef) {
  const float gs = a.grad_scale * (clip_coef ? *clip_coef : 1.f);
  const long long n4 = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float* pa = &pp.x; float* ma = &mm.x; float* va = &vv.x; const float* ga = &gg.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = ga[k] * gs;
      pa[k] -= a.lr * a.weight_decay * pa[k];
      ma[k] = a.beta1 * ma[k] + (1.f - a.beta1) * gk;
      va[k] = a.beta2 * va[k] + (1.f - a.beta2) * gk * gk;
      pa[k] -= a.lr * (ma[k] / a.bc1) / (sqrtf(va[k] / a.bc2) + a.eps);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (p_bf16) {
      uint2 o;
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(p_bf16)[i] = o;
    }
  }
  // tail
  if (blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) {
      const float gk = g[i] * gs;
      float pk = p[i];
      pk -= a.lr * a.weight_decay * pk;
      const float mk = a.beta1 * m[i] + (1.f - a.beta1) * gk;
      const float vk = a.beta2 * v[i] + (1.f - a.beta2) * gk * gk;
      pk -= a.lr * (mk / a.bc1) / (sqrtf(vk / a.bc2) + a.eps);
      p[i] = pk; m[i] = mk; v[i] = vk;
      if (p_bf16) p_bf16[i] = __float2bfloat16(pk);
    }
  }
}

__global__ void sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float scratch[32];
  float s = 0.f;
  const long long n4 = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) s += x[i] * x[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// Index of the nearest centroid in an ascending codebook held in shared memory.
template <int CB>
__device__ __forceinline__ int nearest_sorted(const float* cb, float w) {
  int lo = 0;  // first index with cb[i] >= w (or CB)
#pragma unroll
  for (int step = CB >> 1; step > 0; step >>= 1)
    if (cb[lo + step - 1] < w) lo += step;
  if (lo < CB && cb[lo] < w) ++lo;
  int j;
  if (lo == 0) j = 0;
  else if (lo >= CB) j = CB - 1;
  else j = (w - cb[lo - 1] <= cb[lo] - w) ? lo - 1 : lo;
  while (j > 0 && cb[j - 1] == cb[j]) --j;  // first minimum wins among duplicates
  return j;
}

// One warp per work item = (codebook block, up to 1024 consecutive weights of it).
template <int CB>
__global__ void oil_fake_quant_kernel(const float* __restrict__ w, const float* __restrict__ codebooks,
                                      const int* __restrict__ cb_map, int bs, long long n,
                                      __nv_bfloat16* __restrict__ w_bf16, uint8_t* __restrict__ idx) {
  extern __shared__ float cb_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  float* cb = cb_smem + warp * CB;
  const int sub = (bs + 1023) / 1024;  // work items per block
  const long long nblocks = (n + bs - 1) / bs;
  const long long items = nblocks * sub;
  int cached = -1;
  for (long long it = (long long)blockIdx.x * wpb + warp; it < items; it += (long long)gridDim.x * wpb) {
    const long long b = it / sub;
    const int s = (int)(it % sub);
    const int cbi = cb_map ? cb_map[b] : (int)b;
    if (cbi != cached) {
      __syncwarp();
      for (int i = lane; i < CB; i += 32) cb[i] = codebooks[(long long)cbi * CB + i];
      cached = cbi;
      __syncwarp();
    }
    const long long start = b * bs + (long long)s * 1024;
    long long end = b * bs + bs;
    if (end > n) end = n;
    if (end > start + 1024) end = start + 1024;
    for (long long i = start + lane; i < end; i += 32) {
      const int j = nearest_sorted<CB>(cb, w[i]);
      if (w_bf16) w_bf16[i] = __float2bfloat16(cb[j]);
      if (idx) idx[i] = (uint8_t)j;
    }
  }
}

// One warp per block: absmean scale, trits in {-1,0,+1} stored as code t+1 (0,1,2).
__global__ void i2s_fake_quant_kernel(const float* __restrict__ w, int bs, long long n,
                                      __nv_bfloat16* __restrict__ w_bf16, uint8_t* __restrict__ trits,
                                      float* __restrict__ scales) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const long long nblocks = (n + bs - 1) / bs;
  for (long long b = (long long)blockIdx.x * wpb + warp; b < nblocks; b += (long long)gridDim.x * wpb) {
    const long long start = b * bs;
    const long long end = (start + bs < n) ? start + bs : n;
    float s = 0.f, amax = 0.f;
    for (long long i = start + lane; i < end; i += 32) {
      const float a = fabsf(w[i]);
      s += a;
      amax = fmaxf(amax, a);
    }
    s = warp_sum(s);
    amax = warp_max(amax);
    // A block that already is {-a, 0, +a} keeps a as its scale: quantising is idempotent.
    int exact = 1;
    for (long long i = start + lane; i < end; i += 32) {
      const float a = fabsf(w[i]);
      if (a != 0.f && a != amax) exact = 0;
    }
    exact = __all_sync(0xffffffffu, exact);
    const float scale = exact ? amax : s / (float)(end - start);
    const float inv = scale > 0.f ? 1.f / scale : 0.f;
    if (lane == 0 && scales) scales[b] = scale;
    for (long long i = start + lane; i < end; i += 32) {
      float t = rintf(w[i] * inv);
      t = fminf(1.f, fmaxf(-1.f, t));
      if (w_bf16) w_bf16[i] = __float2bfloat16(t * scale);
      if (trits) trits[i] = (uint8_t)((int)t + 1);
    }
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  const long long n4 = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    reinterpret_cast<uint2*>(y)[i] = o;
  }
  if (blockIdx.x == 0)
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) y[i] = __float2bfloat16(x[i]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ y, long long n, int acc) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(x[i]);
    y[i] = acc ? y[i] + v : v;
  }
}

__global__ void codebook_stats_kernel(const float* __restrict__ w, const uint8_t* __restrict__ idx,
                                      const int* __restrict__ cb_map, int cb_size, int bs, long long n,
                                      float* __restrict__ counts, float* __restrict__ sums) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long b = i / bs;
    const long long cbi = cb_map ? cb_map[b] : b;
    const long long slot = cbi * cb_size + idx[i];
    atomicAdd(counts + slot, 1.f);
    atomicAdd(sums + slot, w[i]);
  }
}

inline int ew_grid(long long work, int threads) {
  long long g = (work + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

void adamw_step(float* p, float* m, float* v, const float* g, void* p_bf16, long long n, AdamWArgs a,
                const float* clip_coef, cudaStream_t stream) {
  if (n == 0) return;
  adamw_kernel<<<ew_grid(n / 4 + 1, 256), 256, 0, stream>>>(p, m, v, g, (__nv_bfloat16*)p_bf16, n, a, clip_coef);
  count_launch();
  check_launch();
}

void sumsq_f32(const float* x, long long n, float* out_accum, cudaStream_t stream) {
  if (n == 0) return;
  sumsq_kernel<<<ew_grid(n / 4 + 1, 256) > 1024 ? 1024 : ew_grid(n / 4 + 1, 256), 256, 0, stream>>>(x, n, out_accum);
  count_launch();
  check_launch();
}

void oil_fake_quant(const float* w, const float* codebooks, const int* cb_map, int cb_size, int bs, long long n,
                    void* w_bf16, uint8_t* idx, cudaStream_t stream) {
  MB_REQUIRE(cb_size == 256 || cb_size == 16, "oil_fake_quant: codebook size must be 256 (OIL8) or 16 (OIL4)");
  MB_REQUIRE(bs > 0, "oil_fake_quant: block size must be positive");
  if (n == 0) return;
  const int threads = 256, wpb = threads / 32;
  const long long items = ((n + bs - 1) / bs) * ((bs + 1023) / 1024);
  long long grid = (items + wpb - 1) / wpb;
  const long long cap = (long long)sm_count() * 8;
  if (grid > cap) grid = cap;
  if (cb_size == 256)
    oil_fake_quant_kernel<256><<<(int)grid, threads, wpb * 256 * sizeof(float), stream>>>(
        w, codebooks, cb_map, bs, n, (__nv_bfloat16*)w_bf16, idx);
  else
    oil_fake_quant_kernel<16><<<(int)grid, threads, wpb * 16 * sizeof(float), stream>>>(
        w, codebooks, cb_map, bs, n, (__nv_bfloat16*)w_bf16, idx);
  count_launch();
  check_launch();
}

void i2s_fake_quant(const float* w, int bs, long long n, void* w_bf16, uint8_t* trits, float* scales,
                    cudaStream_t stream) {
  MB_REQUIRE(bs > 0, "i2s_fake_quant: block size must be positive");
  if (n == 0) return;
  const long long nblocks = (n + bs - 1) / bs;
  long long grid = (nblocks + 7) / 8;
  const long long cap = (long long)sm_count() * 8;
  if (grid > cap) grid = cap;
  i2s_fake_quant_kernel<<<(int)grid, 256, 0, stream>>>(w, bs, n, (__nv_bfloat16*)w_bf16, trits, scales);
  count_launch();
  check_launch();
}

void cast_f32_to_bf16(const float* x, void* y, long long n, cudaStream_t stream) {
  if (n == 0) return;
  cast_f32_bf16_kernel<<<ew_grid(n / 4 + 1, 256), 256, 0, stream>>>(x, (__nv_bfloat16*)y, n);
  count_launch();
  check_launch();
}
void cast_bf16_to_f32(const void* x, float* y, long long n, bool accumulate, cudaStream_t stream) {
  if (n == 0) return;
  cast_bf16_f32_kernel<<<ew_grid(n, 256), 256, 0, stream>>>((const __nv_bfloat16*)x, y, n, accumulate ? 1 : 0);
  count_launch();
  check_launch();
}

void oil_codebook_stats(const float* w, const uint8_t* idx, const int* cb_map, int cb_size, int bs, long long n,
                        float* counts, float* sums, cudaStream_t stream) {
  if (n == 0) return;
  codebook_stats_kernel<<<ew_grid(n, 256), 256, 0, stream>>>(w, idx, cb_map, cb_size, bs, n, counts, sums);
  count_launch();
  check_launch();
}

}  // namespace mb
