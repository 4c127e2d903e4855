// Allocation-free RMSNorm backward: see no_alloc.h for the contract. The partial-sum scratch is a
// file-scope device array; its device address is looked up once per device with
// cudaGetSymbolAddress (in host code the array's name is only a handle, not a device address).
#include "no_alloc.h"

#include <mutex>
#include <string>

#include "api.h"
#include "host_util.h"

namespace {

static __device__ __align__(256) float g_noalloc_scratch[MYTHOS_NOALLOC_PARTIALS * MYTHOS_NOALLOC_MAX_DIM];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;
thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

// Device address of the scratch array on the current device (set up on first use per device).
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MYTHOS_NOALLOC_E_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(MYTHOS_NOALLOC_E_BAD_ARG, "device index out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(MYTHOS_NOALLOC_E_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return MYTHOS_NOALLOC_OK;
}

}  // namespace

extern "C" int mythos_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* rstd,
                                          void* dx, float* dgamma, int rows, int dim, int accumulate, void* stream) {
  if (!dy || !x || !gamma || !rstd || !dx || !dgamma) return fail(MYTHOS_NOALLOC_E_BAD_ARG, "null pointer argument");
  if (rows < 0 || dim <= 0 || dim % 8 != 0)
    return fail(MYTHOS_NOALLOC_E_BAD_ARG, "rows must be >= 0 and dim a positive multiple of 8");
  if (dim > MYTHOS_NOALLOC_MAX_DIM)
    return fail(MYTHOS_NOALLOC_E_TOO_LARGE, "dim " + std::to_string(dim) + " exceeds the built-in scratch (max " +
                                                std::to_string(MYTHOS_NOALLOC_MAX_DIM) + ")");
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != MYTHOS_NOALLOC_OK) return rc;
  const int n_partial = rows < MYTHOS_NOALLOC_PARTIALS ? rows : MYTHOS_NOALLOC_PARTIALS;
  try {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
      // no rows: the gradient of gamma is zero. Overwrite mode still has to write it; a reduction
      // over zero partial rows does exactly that (accumulate mode leaves dgamma as it is).
      if (!accumulate) mb::rmsnorm_bwd_reduce(scratch, dgamma, 0, dim, false, s);
      return MYTHOS_NOALLOC_OK;
    }
    // Every one of the n_partial CTAs writes its full [dim] row of partial sums before the
    // reduction reads them, so stale contents of the shared array are never observed.
    mb::rmsnorm_bwd(dy, x, gamma, rstd, dx, scratch, rows, dim, n_partial, s);
    mb::rmsnorm_bwd_reduce(scratch, dgamma, n_partial, dim, accumulate != 0, s);
  } catch (const std::exception& ex) {
    return fail(MYTHOS_NOALLOC_E_CUDA, ex.what());
  }
  return MYTHOS_NOALLOC_OK;
}

extern "C" const char* mythos_noalloc_last_error(void) { return g_last_error.c_str(); }
