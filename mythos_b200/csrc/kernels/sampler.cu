// Token sampler: one CTA per sequence, logits read straight from the lm_head output.
//
// Semantics of the reference Sampler (src/sampler.cpp:12-120): repetition penalty divides
// positive and multiplies negative logits of tokens already generated (:31-40); temperature
// below 1e-5 means greedy; top-p keeps tokens in decreasing probability until the cumulative
// probability exceeds p, inclusive (:87-93); top-k keeps the k most probable tokens. top-p is
// used when top_p < 1, otherwise top-k (:108-120). Instead of sorting the vocabulary the cut-off
// is found by a 4-round radix select over order-preserving keys of the adjusted logits (count
// histogram for top-k, probability-mass histogram for top-p), then one token is drawn by an
// inverse-CDF walk over the surviving tokens. An optional byte mask restricts the vocabulary
// (grammar-constrained decoding).
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace mb {
namespace {

constexpr int SAMP_THREADS = 1024;

__device__ __forceinline__ uint32_t float_key(float f) {  // larger float -> larger key
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

struct RowView {
  const __nv_bfloat16* logits;
  const unsigned char* allow;
  const uint32_t* seen;  // bitmap of tokens subject to the repetition penalty (shared memory)
  float inv_temp, penalty;
  bool use_penalty;
  __device__ __forceinline__ float at(int i) const {
    if (allow && !allow[i]) return -INFINITY;
    float v = __bfloat162float(logits[i]);
    if (use_penalty && (seen[i >> 5] >> (i & 31)) & 1u) v = v > 0.f ? v / penalty : v * penalty;
    return v * inv_temp;
  }
};

__global__ void __launch_bounds__(SAMP_THREADS)
sampler_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int vocab, const int* __restrict__ history,
               int history_len, const unsigned char* __restrict__ allow_mask, SamplerArgs a,
               int* __restrict__ out_tokens, float* __restrict__ out_logprob) {
  extern __shared__ uint32_t seen[];  // ceil(vocab/32) words
  __shared__ float scratch[32];
  __shared__ float hist[256];
  __shared__ int s_arg;
  __shared__ uint32_t s_prefix;
  __shared__ float s_remaining, s_running;
  __shared__ int s_choice;
  const int row = blockIdx.x, tid = threadIdx.x;
  const int words = (vocab + 31) >> 5;
  const bool greedy = a.temperature < 1e-5f;
  const bool use_pen = history_len > 0 && a.repetition_penalty != 1.f;
  if (use_pen) {
    for (int i = tid; i < words; i += blockDim.x) seen[i] = 0u;
    __syncthreads();
    for (int i = tid; i < history_len; i += blockDim.x) {
      const int t = history[(long long)row * history_len + i];
      if (t >= 0 && t < vocab) atomicOr(&seen[t >> 5], 1u << (t & 31));
    }
    __syncthreads();
  }
  RowView rv{logits + (long long)row * ld, allow_mask ? allow_mask + (long long)row * vocab : nullptr, seen,
             greedy ? 1.f : 1.f / a.temperature, a.repetition_penalty, use_pen};

  // ---- max / argmax (first maximum wins)
  float best = -INFINITY;
  int arg = 0x7fffffff;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = rv.at(i);
    if (v > best) { best = v; arg = i; }
  }
  const float gmax = block_max(best, scratch);
  if (tid == 0) s_arg = 0x7fffffff;
  __syncthreads();
  if (best == gmax) atomicMin(&s_arg, arg);
  __syncthreads();
  // ---- normaliser
  float se = 0.f;
  for (int i = tid; i < vocab; i += blockDim.x) se += __expf(rv.at(i) - gmax);
  const float total = block_sum(se, scratch);
  if (greedy) {
    if (tid == 0) {
      out_tokens[row] = s_arg;
      if (out_logprob) out_logprob[row] = -logf(total);
    }
    return;
  }
  // ---- cut-off key: radix select, 8 bits per round, from the top
  const bool by_mass = a.top_p < 1.f;
  const bool filter = by_mass || (a.top_k > 0 && a.top_k < vocab);
  uint32_t prefix = 0, prefix_mask = 0;
  if (filter) {
    float remaining = by_mass ? a.top_p * total : (float)a.top_k;
    for (int round = 0; round < 4; ++round) {
      const int shift = 24 - 8 * round;
      for (int i = tid; i < 256; i += blockDim.x) hist[i] = 0.f;
      __syncthreads();
      for (int i = tid; i < vocab; i += blockDim.x) {
        const float v = rv.at(i);
        const uint32_t key = float_key(v);
        if ((key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFF], by_mass ? __expf(v - gmax) : 1.f);
      }
      __syncthreads();
      if (tid == 0) {
        float run = 0.f;
        int bin = 0;
        for (int b = 255; b >= 0; --b) {
          // top-p: stop in the bin where the cumulative mass first exceeds the target (inclusive);
          // top-k: stop in the bin that contains the k-th largest.
          if (run + hist[b] >= remaining || b == 0) { bin = b; break; }
          run += hist[b];
        }
        s_prefix = prefix | ((uint32_t)bin << shift);
        s_remaining = remaining - run;
      }
      __syncthreads();
      prefix = s_prefix;
      prefix_mask |= 0xFFu << shift;
      remaining = s_remaining;
      __syncthreads();
    }
  }
  const uint32_t cut = filter ? prefix : 0u;
  // ---- mass of the survivors
  float kept = 0.f;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = rv.at(i);
    if (float_key(v) >= cut) kept += __expf(v - gmax);
  }
  const float kept_total = block_sum(kept, scratch);
  const unsigned long long r = splitmix64(a.seed ^ splitmix64((unsigned long long)row + 0x1234567ull));
  const float u = (float)((r >> 40) * (1.0 / 16777216.0)) * kept_total;
  // ---- inverse CDF in index order, SAMP_THREADS tokens at a time
  if (tid == 0) { s_running = 0.f; s_choice = -1; }
  __syncthreads();
  const int lane = tid & 31, warp = tid >> 5;
  for (int base = 0; base < vocab && s_choice < 0; base += blockDim.x) {
    const int i = base + tid;
    float e = 0.f;
    if (i < vocab) {
      const float v = rv.at(i);
      if (float_key(v) >= cut) e = __expf(v - gmax);
    }
    float inc = e;  // inclusive scan inside the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      float w = scratch[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += n;
      }
      scratch[lane] = w;  // inclusive scan of the warp totals
    }
    __syncthreads();
    const float before = s_running + (warp > 0 ? scratch[warp - 1] : 0.f);
    const float hi = before + inc, lo = hi - e;
    if (e > 0.f && u >= lo && u < hi) atomicMax(&s_choice, i);
    __syncthreads();
    if (tid == 0) s_running += scratch[31];
    __syncthreads();
  }
  if (tid == 0) {
    int tok = s_choice >= 0 ? s_choice : s_arg;  // numerical edge (u == kept_total): fall back to the mode
    out_tokens[row] = tok;
    if (out_logprob) out_logprob[row] = rv.at(tok) - gmax - logf(total);
  }
}

// ---- plain greedy decoding (no penalty, mask or log-probability): argmax over the row, spread
// over several CTAs per row. Each CTA folds its chunk into one 64-bit key (order-preserving image of
// the value in the high word, inverted index in the low word, so ties go to the smallest index),
// atomicMax-es it into the row's slot, and the last CTA of the row writes the token and clears the
// slot for the next launch.
constexpr int ARGMAX_MAX_ROWS = 4096;
static __device__ unsigned long long g_argmax_key[ARGMAX_MAX_ROWS];
static __device__ int g_argmax_count[ARGMAX_MAX_ROWS];

__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
  const uint32_t b = __float_as_uint(v);
  const uint32_t ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((unsigned long long)ord << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)idx);
}

__global__ void __launch_bounds__(256)
argmax_rows_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int vocab, int chunks,
                   int* __restrict__ out_tokens) {
  __shared__ unsigned long long s_key[8];
  const int row = blockIdx.x, chunk = blockIdx.y, tid = threadIdx.x;
  const __nv_bfloat16* lp = logits + (long long)row * ld;
  const int vec = vocab >> 3;                                   // whole 8-element groups
  const int per = (vec + chunks - 1) / chunks;
  const int v0 = chunk * per, v1 = min(vec, v0 + per);
  unsigned long long best = 0ull;
  const bool aligned = ((reinterpret_cast<uintptr_t>(lp) & 15) == 0);
  for (int g = v0 + tid; g < v1; g += blockDim.x) {
    float f[8];
    if (aligned) {
      unpack8(ldg8(lp, (long long)g * 8), f);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(lp[g * 8 + j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned long long k = argmax_key(f[j], g * 8 + j);
      best = k > best ? k : best;
    }
  }
  if (chunk == chunks - 1)                                      // ragged tail of the row
    for (int i = vec * 8 + tid; i < vocab; i += blockDim.x) {
      const unsigned long long k = argmax_key(__bfloat162float(lp[i]), i);
      best = k > best ? k : best;
    }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((tid & 31) == 0) s_key[tid >> 5] = best;
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) best = s_key[w] > best ? s_key[w] : best;
    atomicMax(&g_argmax_key[row], best);
    __threadfence();
    if (atomicAdd(&g_argmax_count[row], 1) == chunks - 1) {
      __threadfence();
      const unsigned long long k = atomicExch(&g_argmax_key[row], 0ull);
      g_argmax_count[row] = 0;
      out_tokens[row] = (int)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
    }
  }
}

}  // namespace

void sample_tokens(const void* logits, long long ld, int rows, int vocab, const int* history, int history_len,
                   const unsigned char* allow_mask, SamplerArgs a, int* out_tokens, float* out_logprob, float* scratch,
                   cudaStream_t stream) {
  (void)scratch;
  if (rows == 0) return;
  const bool plain_greedy = a.temperature < 1e-5f && allow_mask == nullptr && out_logprob == nullptr &&
                            !(history_len > 0 && a.repetition_penalty != 1.f);
  if (plain_greedy && rows <= ARGMAX_MAX_ROWS) {
    int chunks = (2 * sm_count() + rows - 1) / rows;
    const int max_chunks = (vocab / 8 + 2047) / 2048;          // at least 8 vectors per thread
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks < 1) chunks = 1;
    argmax_rows_kernel<<<dim3(rows, chunks), 256, 0, stream>>>((const __nv_bfloat16*)logits, ld, vocab, chunks,
                                                               out_tokens);
    count_launch();
    check_launch();
    return;
  }
  const size_t smem = (size_t)((vocab + 31) / 32) * 4;
  MB_REQUIRE(smem <= 48 * 1024, "sample_tokens: vocabulary too large for the repetition bitmap");
  sampler_kernel<<<rows, SAMP_THREADS, smem, stream>>>((const __nv_bfloat16*)logits, ld, vocab, history, history_len,
                                                       allow_mask, a, out_tokens, out_logprob);
  count_launch();
  check_launch();
}

}  // namespace mb
