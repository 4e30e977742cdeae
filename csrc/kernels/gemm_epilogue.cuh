// Epilogue that stores a GEMM tile to local memory: optional bias, optional GELU side output, bf16 or
// fp32, optional accumulation into D.  Shared by the plain GEMM and the all-gather -> GEMM kernel.
#pragma once
#include "gemm_api.h"
#include "gemm_pipeline.cuh"

namespace pccl {
namespace gemm {

// Hardware tanh (one MUFU instruction, relative error near 2^-11: below the bf16 rounding of the results it feeds).
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.0f + tanh_fast(u));
}

// d/dx of gelu_tanh
__device__ __forceinline__ float dgelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float x2 = x * x;
  const float t = tanh_fast(k0 * (x + k1 * x * x2));
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * k0 * (1.0f + 3.0f * k1 * x2);
}

// Sums v[0..31] of the 32 lanes column by column: afterwards lane l holds (in v[0]) the sum over the warp of v[l].
// A butterfly that halves the number of live values per step: 31 shuffles instead of 32 five-step reductions.
__device__ __forceinline__ void warp_transpose_sum32(float* v, int lane) {
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) {
    const bool upper = (lane & s) != 0;
#pragma unroll
    for (int i = 0; i < s; ++i) {
      const float send = upper ? v[i] : v[i + s];
      const float keep = upper ? v[i + s] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
    }
  }
}

// Backward of a GELU that sits between two linear layers, fused into the GEMM that produces the gradient of the
// activation: D = (A * B^T) .* gelu'(pre), and the column sums of D (the bias gradient of the first layer) are added
// to `colsum` (fp32, zeroed by the caller).  Full tiles only (M % 128 == 0, N % 256 == 0); `pre` has D's layout.
struct DgeluEpi {
  static constexpr bool kRow128 = false;
  __nv_bfloat16* D;
  const __nv_bfloat16* pre;
  float* colsum;
  long long ldd;
  int M, N;

  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return t.m * BM; }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return t.n * BN; }
  __device__ __forceinline__ void attach_smem(uint8_t*) {}
  __device__ __forceinline__ void tile_begin(const TileCoord&) {}
  __device__ __forceinline__ void tile_done(const TileCoord&, const volatile uint32_t*) {}

  __device__ __forceinline__ void strip(const TileCoord& t, int row_in_tile, int col_in_tile, uint32_t* r) {
    const int row = t.m * BM + row_in_tile, col = t.n * BN + col_in_tile;
    const long long at = static_cast<long long>(row) * ldd + col;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      float x[8];
      dev::unpack<DT_BF16>(dev::ld16(pre + at + i), x);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i + j] = __uint_as_float(r[i + j]) * dgelu_tanh(x[j]);
    }
#pragma unroll
    for (int i = 0; i < 32; i += 8) dev::st16(D + at + i, dev::pack<DT_BF16>(v + i));
    if (colsum) {
      const int lane = threadIdx.x & 31;       // an epilogue warp holds 32 consecutive rows, one per lane
      warp_transpose_sum32(v, lane);
      atomicAdd(colsum + col + lane, v[0]);
    }
  }
};

struct StoreEpi {
  static constexpr bool kRow128 = false;   // takes 32-column strips
  void* D;
  void* D2;
  const __nv_bfloat16* bias;
  long long ldd;
  int M, N;
  uint32_t flags;

  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return t.m * BM; }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return t.n * BN; }
  __device__ __forceinline__ void attach_smem(uint8_t*) {}
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
      if (flags & GEMM_ADD_D2) {        // D = A*B^T (+bias) + D2: the residual connection around a linear layer
        const __nv_bfloat16* res = static_cast<const __nv_bfloat16*>(D2) + static_cast<long long>(row) * ldd + col;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          float f[8];
          dev::unpack<DT_BF16>(dev::ld16(res + i), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i + j] += f[j];
        }
      }
      if (flags & GEMM_GELU_INPLACE) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
      }
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
        if (flags & GEMM_ADD_D2) v[i] += __bfloat162float((static_cast<const __nv_bfloat16*>(D2) + static_cast<long long>(row) * ldd + col)[i]);
        float x = (flags & GEMM_ACCUMULATE) ? v[i] + __bfloat162float(d[i]) : v[i];
        d[i] = __float2bfloat16_rn(x);
        if (flags & GEMM_GELU)
          (static_cast<__nv_bfloat16*>(D2) + static_cast<long long>(row) * ldd + col)[i] = __float2bfloat16_rn(gelu_tanh(x));
      }
    }
  }
};

}  // namespace gemm
}  // namespace pccl
