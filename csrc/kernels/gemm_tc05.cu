// Plain bf16 GEMM on the tcgen05 pipeline (see gemm_pipeline.cuh) with a fused epilogue:
// optional bias, optional GELU side output, bf16 or fp32 store, optional accumulation into D.
// The reference has no GEMM of any kind (cutlass and composable_kernel are empty submodules,
// .gitmodules:4-9); this is the "computation" half of its "communication & computation" claim.
#include <cuda.h>

#include <mutex>
#include <string>

#include "gemm_api.h"
#include "gemm_pipeline.cuh"
#include "tensormap.h"

namespace pccl {

namespace {

using namespace gemm;

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}

struct StoreEpi {
  void* D;
  void* D2;
  const __nv_bfloat16* bias;
  long long ldd;
  int M, N;
  uint32_t flags;

  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return t.m * BM; }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return t.n * BN; }
  __device__ __forceinline__ void tile_begin(const TileCoord&) {}
  __device__ __forceinline__ void tile_done(const TileCoord&, const volatile uint32_t*) {}

  __device__ __forceinline__ void strip(const TileCoord& t, int row_in_tile, int col_in_tile, uint32_t* r) {
    const int row = t.m * BM + row_in_tile, col = t.n * BN + col_in_tile;
    if (row >= M || col >= N) return;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    const bool full = col + 32 <= N;
    if (flags & GEMM_BIAS) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (full || col + i < N) v[i] += __bfloat162float(bias[col + i]);
    }
    if (flags & GEMM_OUT_F32) {
      float* d = static_cast<float*>(D) + static_cast<long long>(row) * ldd + col;
      if (full) {
        if (flags & GEMM_ACCUMULATE) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 o = *reinterpret_cast<float4*>(d + i);
            v[i] += o.x; v[i + 1] += o.y; v[i + 2] += o.z; v[i + 3] += o.w;
          }
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(d + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (col + i < N) d[i] = (flags & GEMM_ACCUMULATE) ? d[i] + v[i] : v[i];
      }
      return;
    }
    __nv_bfloat16* d = static_cast<__nv_bfloat16*>(D) + static_cast<long long>(row) * ldd + col;
    if (full) {
      if (flags & GEMM_ACCUMULATE) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          dev::Vec16 o = dev::ld16(d + i);
          float f[8];
          dev::unpack<DT_BF16>(o, f);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i + j] += f[j];
        }
      }
#pragma unroll
      for (int i = 0; i < 32; i += 8) dev::st16(d + i, dev::pack<DT_BF16>(v + i));
      if (flags & GEMM_GELU) {
        __nv_bfloat16* d2 = static_cast<__nv_bfloat16*>(D2) + static_cast<long long>(row) * ldd + col;
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
#pragma unroll
        for (int i = 0; i < 32; i += 8) dev::st16(d2 + i, dev::pack<DT_BF16>(v + i));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (col + i >= N) continue;
        float x = (flags & GEMM_ACCUMULATE) ? v[i] + __bfloat162float(d[i]) : v[i];
        d[i] = __float2bfloat16_rn(x);
        if (flags & GEMM_GELU)
          (static_cast<__nv_bfloat16*>(D2) + static_cast<long long>(row) * ldd + col)[i] = __float2bfloat16_rn(gelu_tanh(x));
      }
    }
  }
};

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, StoreEpi epi, int K,
                 uint32_t* status) {
  GroupedSched sched{(epi.M + BM - 1) / BM, (epi.N + BN - 1) / BN, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x)};
  NoGate gate;
  run<A_MN, B_MN>(&tmA, &tmB, K, sched, gate, epi, status);
}

thread_local std::string g_err;

template <bool A_MN, bool B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const StoreEpi& epi, int K, int grid, uint32_t* status, cudaStream_t stream) {
  static bool attr_set = false;
  auto kern = gemm_bf16_kernel<A_MN, B_MN>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, epi, K, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

const char* gemmLastError() { return g_err.c_str(); }

int gemmBf16(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K,
             uint32_t flags, const void* bias, void* D2, int sms, uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda | ldb | ldd) % 8 || (reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D)) % 16) {
    g_err = "gemmBf16: strides must be multiples of 8 elements and pointers 16-byte aligned";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if ((flags & GEMM_GELU) && (!D2 || (flags & GEMM_OUT_F32))) {
    g_err = "gemmBf16: the GELU side output needs D2 and a bf16 D";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  const bool a_mn = flags & GEMM_A_MN, b_mn = flags & GEMM_B_MN;
  CUtensorMap ta, tb;
  // K-major: dims {K, rows}; MN-major: dims {rows, K}
  if (!a_mn ? !makeTensorMap2D(&ta, A, TM_BF16, K, M, lda, BK, BM, &g_err) : !makeTensorMap2D(&ta, A, TM_BF16, M, K, lda, 64, BK, &g_err))
    return static_cast<int>(cudaErrorInvalidValue);
  if (!b_mn ? !makeTensorMap2D(&tb, B, TM_BF16, K, N, ldb, BK, BN, &g_err) : !makeTensorMap2D(&tb, B, TM_BF16, N, K, ldb, 64, BK, &g_err))
    return static_cast<int>(cudaErrorInvalidValue);
  StoreEpi epi{D, D2, static_cast<const __nv_bfloat16*>(bias), ldd, M, N, flags};
  int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int n_sm = deviceSmCount();
  if (sms > 0 && sms < n_sm) n_sm = sms;
  int grid = tiles < n_sm ? tiles : n_sm;
  if (a_mn) return b_mn ? launch<true, true>(ta, tb, epi, K, grid, status, stream) : launch<true, false>(ta, tb, epi, K, grid, status, stream);
  return b_mn ? launch<false, true>(ta, tb, epi, K, grid, status, stream) : launch<false, false>(ta, tb, epi, K, grid, status, stream);
}

}  // namespace pccl
