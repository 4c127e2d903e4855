// Host-side helpers shared by the kernel launchers: error type, launch counter and the
// TMA tensor-map encoder (resolved from the driver at run time, so the library links
// against the CUDA runtime only).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>
#include <stdexcept>
#include <string>

namespace mb {

struct CudaError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

#define MB_CUDA_CHECK(expr)                                                                       \
  do {                                                                                            \
    cudaError_t _e = (expr);                                                                      \
    if (_e != cudaSuccess)                                                                        \
      throw ::mb::CudaError(std::string(#expr) + " failed: " + cudaGetErrorString(_e) + " at " + \
                            __FILE__ + ":" + std::to_string(__LINE__));                           \
  } while (0)

#define MB_REQUIRE(cond, msg)                                                        \
  do {                                                                               \
    if (!(cond)) throw std::invalid_argument(std::string("mythos_b200: ") + (msg)); \
  } while (0)

// Number of kernels this library has launched in this process (all launchers bump it).
std::atomic<long long>& launch_counter();
inline void count_launch(int n = 1) { launch_counter().fetch_add(n, std::memory_order_relaxed); }
inline void check_launch() { MB_CUDA_CHECK(cudaGetLastError()); }

enum class TmaDType { BF16, F32, U8 };

// 2-D..4-D tiled tensor map. dims/strides are innermost-first; strides[i] is the byte stride
// of dimension i+1 (dimension 0 is contiguous). swizzle128: 128-byte swizzle (box inner
// extent must then be exactly 128 bytes); otherwise no swizzle.
CUtensorMap make_tensor_map(const void* base, TmaDType dt, int rank, const uint64_t* dims,
                            const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128);

int sm_count();

}  // namespace mb
