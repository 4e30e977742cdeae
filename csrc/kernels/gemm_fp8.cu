// Block-scaled fp8 GEMM on the tcgen05 pipeline of gemm_fp8_pipeline.cuh: e4m3 operands with 1 x 128
// activation scales and 128 x 128 weight scales, fp32 promotion in registers, the same fused store
// epilogue as the bf16 GEMM (bias, GELU, bf16 or fp32, accumulate).  The reference has no GEMM.
#include <cuda.h>

#include <string>

#include "gemm_api.h"
#include "gemm_epilogue.cuh"
#include "gemm_fp8_pipeline.cuh"
#include "tensormap.h"

namespace pccl {

namespace {

__global__ void __launch_bounds__(gemm8::NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, gemm::StoreEpi epi,
                gemm8::Scales sc, int K, uint32_t* status) {
  gemm::GroupedSched sched{(epi.M + gemm8::BM - 1) / gemm8::BM, (epi.N + gemm8::BN - 1) / gemm8::BN, static_cast<int>(blockIdx.x),
                           static_cast<int>(gridDim.x)};
  gemm::NoGate gate;
  gemm8::run(&tmA, &tmB, K, sc, sched, gate, epi, status);
}

thread_local std::string g_err8;

}  // namespace

const char* gemmFp8LastError() { return g_err8.c_str(); }

int gemmFp8(const void* A, int64_t lda, const float* sa, int ld_sa, const void* B, int64_t ldb, const float* sb, int ld_sb,
            void* D, int64_t ldd, int M, int N, int K, uint32_t flags, const void* bias, void* D2, int sms, uint32_t* status,
            cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda | ldb) % 16 || ldd % 8 || K % 128 ||
      (reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D)) % 16) {
    g_err8 = "gemmFp8: K must be a multiple of 128, operand strides multiples of 16, pointers 16-byte aligned";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (flags & (GEMM_A_MN | GEMM_B_MN | GEMM_PAIR)) {
    g_err8 = "gemmFp8: operands are K-major and tiles belong to single CTAs";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if ((flags & GEMM_GELU) && (!D2 || (flags & GEMM_OUT_F32))) {
    g_err8 = "gemmFp8: the GELU side output needs D2 and a bf16 D";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (ld_sa < K / 128 || ld_sb < K / 128) {
    g_err8 = "gemmFp8: scale rows are shorter than K / 128";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  CUtensorMap ta, tb;
  if (!makeTensorMap2D(&ta, A, TM_U8, K, M, lda, gemm8::BK, gemm8::BM, &g_err8)) return static_cast<int>(cudaErrorInvalidValue);
  if (!makeTensorMap2D(&tb, B, TM_U8, K, N, ldb, gemm8::BK, gemm8::BN, &g_err8)) return static_cast<int>(cudaErrorInvalidValue);
  gemm::StoreEpi epi{D, D2, static_cast<const __nv_bfloat16*>(bias), ldd, M, N, flags};
  gemm8::Scales sc{sa, sb, ld_sa, ld_sb, M, N};
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm8::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  int tiles = ((M + gemm8::BM - 1) / gemm8::BM) * ((N + gemm8::BN - 1) / gemm8::BN);
  int n_sm = deviceSmCount();
  if (sms > 0 && sms < n_sm) n_sm = sms;
  int grid = tiles < n_sm ? tiles : n_sm;
  gemm_fp8_kernel<<<grid, gemm8::NUM_THREADS, gemm8::SMEM_BYTES, stream>>>(ta, tb, epi, sc, K, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace pccl
