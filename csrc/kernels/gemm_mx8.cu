// fp8 GEMM with hardware block scaling (gemm_mx8_pipeline.cuh) and the quantisers that produce its operands:
// e4m3 values with power-of-two (UE8M0) scales, one per row and 128 values of K for activations, one per
// 128 x 128 block for weights.  The reference has no GEMM and no quantiser.
#include <cuda.h>
#include <cuda_fp8.h>

#include <string>

#include "gemm_api.h"
#include "gemm_epilogue.cuh"
#include "gemm_mx8_pipeline.cuh"
#include "tensormap.h"

namespace pccl {

namespace {

__global__ void __launch_bounds__(gemmx::NUM_THREADS, 1)
gemm_mx8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, gemm::StoreEpi epi,
                gemmx::Scales sc, int K, uint32_t* status) {
  gemm::GroupedSched sched{(epi.M + gemmx::BM - 1) / gemmx::BM, (epi.N + gemmx::BN - 1) / gemmx::BN, static_cast<int>(blockIdx.x),
                           static_cast<int>(gridDim.x)};
  gemm::NoGate gate;
  gemmx::run(&tmA, &tmB, K, sc, sched, gate, epi, status);
}

// Smallest power of two >= amax / 448 (so that the scaled block fits e4m3), as a float and as its UE8M0 byte.
__device__ __forceinline__ float pow2_scale(float amax, uint8_t* byte) {
  if (!(amax > 0.f)) { *byte = 127; return 1.0f; }
  const float v = amax * (1.0f / 448.0f);
  uint32_t bits = __float_as_uint(v);
  uint32_t e = (bits >> 23) & 0xff;
  if (bits & 0x7fffff) e += 1;                 // round the mantissa up
  e = e < 1 ? 1 : (e > 254 ? 254 : e);
  *byte = static_cast<uint8_t>(e);
  return __uint_as_float(e << 23);
}

__device__ __forceinline__ uint2 quant8_mx(const float* f, float inv) {
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * h] * inv, f[4 * h + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * h + 2] * inv, f[4 * h + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    w[h] = (lo & 0xffffu) | (hi << 16);
  }
  return make_uint2(w[0], w[1]);
}

// 16 consecutive lanes own one 1 x 128 block (8 values each)
__global__ void __launch_bounds__(256) quant_rows_mx_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                            uint8_t* __restrict__ scales, long long rows, int k) {
  const int nvec = k >> 3, G = k >> 7;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    for (int v = threadIdx.x; v < ((nvec + 31) & ~31); v += blockDim.x) {
      float f[8];
      float amax = 0.f;
      if (v < nvec) {
        dev::unpack<DT_BF16>(dev::ld16(x + r * k + v * 8), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      uint8_t byte;
      const float scale = pow2_scale(amax, &byte);
      if (v < nvec) {
        *reinterpret_cast<uint2*>(q + r * k + v * 8) = quant8_mx(f, 1.0f / scale);
        if ((v & 15) == 0) scales[r * G + (v >> 4)] = byte;
      }
    }
  }
}

// one CTA per 128 x 128 block of a weight matrix
__global__ void __launch_bounds__(256) quant_blocks_mx_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                                                              uint8_t* __restrict__ scales, int rows, int cols) {
  __shared__ float red[8];
  const int bc = blockIdx.x, br = blockIdx.y;
  const __nv_bfloat16* base = w + static_cast<long long>(br) * 128 * cols + bc * 128;
  float f[8][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = threadIdx.x + i * 256, r = idx >> 4, v = idx & 15;
    dev::unpack<DT_BF16>(dev::ld16(base + static_cast<long long>(r) * cols + v * 8), f[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[i][j]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  uint8_t byte;
  const float scale = pow2_scale(amax, &byte);
  if (threadIdx.x == 0) scales[br * (cols >> 7) + bc] = byte;
  const float inv = 1.0f / scale;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = threadIdx.x + i * 256, r = idx >> 4, v = idx & 15;
    *reinterpret_cast<uint2*>(q + (static_cast<long long>(br) * 128 + r) * cols + bc * 128 + v * 8) = quant8_mx(f[i], inv);
  }
}

thread_local std::string g_errx;

}  // namespace

const char* gemmMx8LastError() { return g_errx.c_str(); }

int launchQuantMx8Rows(const void* x, void* q, uint8_t* scales, long long rows, int k, cudaStream_t stream) {
  if (k % 128 || rows <= 0) return static_cast<int>(cudaErrorInvalidValue);
  const long long blocks = rows < 4096 ? rows : 4096;
  quant_rows_mx_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scales, rows, k);
  return static_cast<int>(cudaGetLastError());
}

int launchQuantMx8Blocks(const void* w, void* q, uint8_t* scales, int rows, int cols, cudaStream_t stream) {
  if (rows % 128 || cols % 128 || rows <= 0 || cols <= 0) return static_cast<int>(cudaErrorInvalidValue);
  dim3 grid(cols / 128, rows / 128);
  quant_blocks_mx_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q), scales, rows, cols);
  return static_cast<int>(cudaGetLastError());
}

int gemmMx8(const void* A, int64_t lda, const uint8_t* sa, int ld_sa, const void* B, int64_t ldb, const uint8_t* sb, int ld_sb,
            void* D, int64_t ldd, int M, int N, int K, uint32_t flags, const void* bias, void* D2, int sms, uint32_t* status,
            cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda | ldb) % 16 || ldd % 8 || K % 128 ||
      (reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D)) % 16) {
    g_errx = "gemmMx8: K must be a multiple of 128, operand strides multiples of 16, pointers 16-byte aligned";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (flags & (GEMM_A_MN | GEMM_B_MN | GEMM_PAIR)) {
    g_errx = "gemmMx8: operands are K-major and tiles belong to single CTAs";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if ((flags & GEMM_GELU) && (!D2 || (flags & GEMM_OUT_F32))) {
    g_errx = "gemmMx8: the GELU side output needs D2 and a bf16 D";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (ld_sa < K / 128 || ld_sb < K / 128) {
    g_errx = "gemmMx8: scale rows are shorter than K / 128";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  CUtensorMap ta, tb;
  if (!makeTensorMap2D(&ta, A, TM_U8, K, M, lda, gemmx::BK, gemmx::BM, &g_errx)) return static_cast<int>(cudaErrorInvalidValue);
  if (!makeTensorMap2D(&tb, B, TM_U8, K, N, ldb, gemmx::BK, gemmx::BN, &g_errx)) return static_cast<int>(cudaErrorInvalidValue);
  gemm::StoreEpi epi{D, D2, static_cast<const __nv_bfloat16*>(bias), ldd, M, N, flags};
  gemmx::Scales sc{sa, sb, ld_sa, ld_sb, M, N};
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mx8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemmx::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  int tiles = ((M + gemmx::BM - 1) / gemmx::BM) * ((N + gemmx::BN - 1) / gemmx::BN);
  int n_sm = deviceSmCount();
  if (sms > 0 && sms < n_sm) n_sm = sms;
  int grid = tiles < n_sm ? tiles : n_sm;
  gemm_mx8_kernel<<<grid, gemmx::NUM_THREADS, gemmx::SMEM_BYTES, stream>>>(ta, tb, epi, sc, K, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace pccl
