// C entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for embedders of this
// library that run under a fixed memory budget or inside a region where the CUDA allocator may
// not be called (a real-time serving loop, a host application that hands the GPU a fixed arena,
// a plugin loaded into a process that forbids cudaMalloc after start-up).
//
// mythos_rmsnorm_bwd_noalloc is the RMSNorm backward pass (the same kernels as the regular
// rmsnorm_bwd + rmsnorm_bwd_reduce pair). The regular path needs a caller-allocated fp32 scratch
// of [n_partial, dim] for the per-CTA partial sums of dgamma; here that scratch is a fixed
// array in device global memory that is part of the library image:
//
//   * size: MYTHOS_NOALLOC_PARTIALS (128) x MYTHOS_NOALLOC_MAX_DIM (8192) floats = 4 MiB, held by
//     every GPU that loads the library until the process exits;
//   * dim must be a multiple of 8 and at most MYTHOS_NOALLOC_MAX_DIM, otherwise the call is
//     rejected with MYTHOS_NOALLOC_E_TOO_LARGE / _E_BAD_ARG and nothing is launched;
//   * the first call on a device looks up the array's device address (a host-side query, no
//     allocation); make that first call before any CUDA stream capture begins;
//   * all calls share the one array: the partial sums of a call are fully overwritten by the next
//     call before they are read, so nothing has to be cleared, but two calls that overlap on the
//     GPU (different streams, no ordering between them) race on it. Serialise them.
//
// The function calls no cudaMalloc / cudaFree and no allocating library routine. Inputs and
// outputs are device pointers supplied by the caller: dy, x, dx are bf16 [rows, dim]; gamma is
// bf16 [dim]; rstd is fp32 [rows] as produced by the forward pass; dgamma is fp32 [dim]
// (overwritten, or added to when accumulate != 0; with rows == 0 that means zeros, or no change).
// `stream` is a cudaStream_t (null = default).
// Returns 0 on success, a negative MYTHOS_NOALLOC_E_* code otherwise; mythos_noalloc_last_error()
// gives the message of the last failure on the calling thread.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define MYTHOS_NOALLOC_PARTIALS 128
#define MYTHOS_NOALLOC_MAX_DIM 8192

#define MYTHOS_NOALLOC_OK 0
#define MYTHOS_NOALLOC_E_BAD_ARG (-1)
#define MYTHOS_NOALLOC_E_TOO_LARGE (-2)
#define MYTHOS_NOALLOC_E_CUDA (-3)

int mythos_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx,
                               float* dgamma, int rows, int dim, int accumulate, void* stream);
const char* mythos_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
