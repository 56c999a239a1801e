// TMA tensor-map encoding shared by the GEMM and attention launchers.
//
// cuTensorMapEncodeTiled is resolved through cudaGetDriverEntryPoint, so the library has no link-time dependency
// on libcuda.  The call needs a CUDA context bound to the calling thread; launchers are also called from PyTorch's
// autograd worker threads, where the driver may report "invalid context" although the runtime has a device
// selected - in that case the primary context is bound to the thread and the call is repeated.
#include <cuda.h>
#include <cuda_runtime.h>

#include "tmap.h"

namespace ffb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*CtxGetCurrentFn)(CUcontext*);
typedef CUresult (*CtxSetCurrentFn)(CUcontext);
typedef CUresult (*PrimaryRetainFn)(CUcontext*, CUdevice);

static void* entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
  return p;
}

static void bind_primary_context() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  cudaSetDevice(dev);
  static CtxGetCurrentFn get_cur = reinterpret_cast<CtxGetCurrentFn>(entry("cuCtxGetCurrent"));
  static CtxSetCurrentFn set_cur = reinterpret_cast<CtxSetCurrentFn>(entry("cuCtxSetCurrent"));
  static PrimaryRetainFn retain = reinterpret_cast<PrimaryRetainFn>(entry("cuDevicePrimaryCtxRetain"));
  if (!get_cur || !set_cur || !retain) return;
  CUcontext ctx = nullptr;
  if (get_cur(&ctx) == CUDA_SUCCESS && ctx != nullptr) return;
  if (retain(&ctx, dev) == CUDA_SUCCESS && ctx != nullptr) set_cur(ctx);   // the primary context outlives the process' use of it
}

int encode_tmap3_bf16(CUtensorMap* map, const void* ptr, long long d0, long long d1, long long d2, long long s1, long long s2,
                      int b0, int b1, int swizzle_bytes) {
  static EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(entry("cuTensorMapEncodeTiled"));
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)(d2 > 0 ? d2 : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)s1 * 2, (cuuint64_t)(d2 > 1 ? s2 : d1 * s1) * 2};
  if (strides[1] == 0) strides[1] = (cuuint64_t)s1 * 2 * (cuuint64_t)d1;
  cuuint32_t box[3] = {(cuuint32_t)b0, (cuuint32_t)b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                       : (swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE));
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT && r != CUDA_ERROR_NOT_INITIALIZED) break;
    bind_primary_context();
  }
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace ffb
