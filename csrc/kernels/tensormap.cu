#include "tensormap.h"

#include <cuda_runtime.h>

#include <mutex>

namespace pccl {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encoder() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}
}  // namespace

bool makeTensorMap2D(CUtensorMap* out, const void* base, TmDType dt, uint64_t inner, uint64_t outer, uint64_t row_stride,
                     uint32_t box_inner, uint32_t box_outer, std::string* err) {
  // The driver call needs a current context; a thread that has only made runtime calls that do
  // not touch the device (an autograd worker, say) may not have bound the primary context yet.
  static thread_local bool ctx_ready = false;
  if (!ctx_ready) {
    cudaFree(nullptr);
    ctx_ready = true;
  }
  EncodeFn fn = encoder();
  if (!fn) {
    if (err) *err = "cuTensorMapEncodeTiled is not available from this driver";
    return false;
  }
  const uint32_t es = dt == TM_BF16 ? 2 : (dt == TM_F32 ? 4 : 1);
  CUtensorMapDataType cdt = dt == TM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                          : (dt == TM_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  if (box_inner * es != 128 || box_outer > 256 || (row_stride * es) % 16 || reinterpret_cast<uintptr_t>(base) % 16) {
    if (err) *err = "tensor map: box must be 128 bytes wide and at most 256 rows; stride and base 16-byte aligned";
    return false;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride * es};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(out, cdt, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (err) *err = "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r));
    return false;
  }
  return true;
}

}  // namespace pccl
