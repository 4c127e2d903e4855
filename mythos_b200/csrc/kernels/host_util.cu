#include "host_util.h"

#include <mutex>

namespace mb {

std::atomic<long long>& launch_counter() {
  static std::atomic<long long> c{0};
  return c;
}

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
      throw CudaError("cuTensorMapEncodeTiled is not available from this driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}
}  // namespace

CUtensorMap make_tensor_map(const void* base, TmaDType dt, int rank, const uint64_t* dims,
                            const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  MB_REQUIRE(rank >= 1 && rank <= 5, "tensor map rank must be 1..5");
  MB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base address must be 16-byte aligned");
  CUtensorMapDataType cdt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  size_t esz = 2;
  if (dt == TmaDType::F32) { cdt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; esz = 4; }
  if (dt == TmaDType::U8) { cdt = CU_TENSOR_MAP_DATA_TYPE_UINT8; esz = 1; }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    MB_REQUIRE(box[i] >= 1 && box[i] <= 256, "TMA box extent must be 1..256");
  }
  for (int i = 0; i + 1 < rank; ++i) {
    gstr[i] = strides_bytes[i];
    MB_REQUIRE((strides_bytes[i] & 15) == 0, "TMA strides must be multiples of 16 bytes");
  }
  MB_REQUIRE((box[0] * esz) % 16 == 0, "TMA box inner extent must be a multiple of 16 bytes");
  if (swizzle128) MB_REQUIRE(box[0] * esz == 128, "128-byte swizzle needs a 128-byte inner box");
  // The encoder is a driver entry point and needs this thread's context to be current; a thread
  // that has made no runtime call yet (an autograd worker) has none until the runtime binds one.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    MB_CUDA_CHECK(cudaFree(nullptr));
    ctx_bound = true;
  }
  CUtensorMap m;
  CUresult r = encode_fn()(&m, cdt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, gbox, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw CudaError("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return m;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    MB_CUDA_CHECK(cudaGetDevice(&dev));
    MB_CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
  }
  return n;
}

}  // namespace mb
