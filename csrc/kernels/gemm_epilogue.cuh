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

// d/dx of gelu_tanh, in eight multiply-adds and one tanh:
//   u = k0 (x + k1 x^3),  t = tanh u,  gelu'(x) = (1 + t)/2 + (1 - t^2) * x * (k0/2) (1 + 3 k1 x^2)
__device__ __forceinline__ float dgelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float a = x * x;
  const float t = tanh_fast(x * fmaf(a, k0 * k1, k0));
  const float q = x * fmaf(a, 1.5f * k0 * k1, 0.5f * k0);
  return fmaf(q, fmaf(-t, t, 1.0f), fmaf(0.5f, t, 0.5f));
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

// ---- coalescing patch ------------------------------------------------------------------------------------------------
// After tcgen05.ld a lane holds 32 consecutive columns of ONE row, so a 16-byte store per lane touches 32 different rows:
// 32 half-filled 32-byte sectors per instruction.  Through a small per-warp patch of shared memory (32 rows x 64 bytes,
// rows 80 bytes apart so that neither side has bank conflicts worth the name) the strip is turned around: four lanes cover
// one row's 64 bytes, an instruction writes eight rows in full sectors.  Half the sector operations at the L2 for the same
// bytes; an epilogue with two outputs (pre-activation and GELU) or a side input is bound by exactly that.
constexpr int kPatchRowBytes = 80;
constexpr int kPatchBytes = 32 * kPatchRowBytes;          // per epilogue warp
constexpr int kPatchBytesPerCta = 8 * kPatchBytes;       // up to eight epilogue warps
// the calling epilogue warp's patch: warps 2, 3, ... of the CTA are the epilogue warps
__device__ __forceinline__ uint8_t* my_patch(uint8_t* base) { return base + (((threadIdx.x >> 5) - 2) & 7) * kPatchBytes; }

// the lane's 32 values -> bf16 -> rows [0, rows_valid) of the 32 x 32 strip at g0 (row stride ldd elements)
__device__ __forceinline__ void patch_store_bf16(uint8_t* P, int lane, __nv_bfloat16* g0, long long ldd, const float* v, int rows_valid) {
  uint8_t* mine = P + lane * kPatchRowBytes;
#pragma unroll
  for (int i = 0; i < 4; ++i) *reinterpret_cast<dev::Vec16*>(mine + i * 16) = dev::pack<DT_BF16>(v + 8 * i);
  __syncwarp();
  const int chunk = lane & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int rr = (lane >> 2) + 8 * j;
    const dev::Vec16 x = *reinterpret_cast<const dev::Vec16*>(P + rr * kPatchRowBytes + chunk * 16);
    if (rr < rows_valid) dev::st16(g0 + rr * ldd + chunk * 8, x);
  }
  __syncwarp();
}

// rows [0, rows_valid) of the 32 x 32 bf16 strip at g0 -> the lane's own row as 32 floats (rows past rows_valid: zeros)
__device__ __forceinline__ void patch_load_bf16(uint8_t* P, int lane, const __nv_bfloat16* g0, long long ldd, float* out, int rows_valid) {
  const int chunk = lane & 3;
  dev::Vec16 x[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int rr = (lane >> 2) + 8 * j;
    x[j] = rr < rows_valid ? dev::ld16(g0 + rr * ldd + chunk * 8) : dev::Vec16{{0u, 0u, 0u, 0u}};
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) *reinterpret_cast<dev::Vec16*>(P + ((lane >> 2) + 8 * j) * kPatchRowBytes + chunk * 16) = x[j];
  __syncwarp();
  const uint8_t* mine = P + lane * kPatchRowBytes;
#pragma unroll
  for (int i = 0; i < 4; ++i) dev::unpack<DT_BF16>(*reinterpret_cast<const dev::Vec16*>(mine + i * 16), out + 8 * i);
  __syncwarp();
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
  uint8_t* patch = nullptr;      // kPatchBytesPerCta of shared memory when the pipeline provides it (see above)

  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return t.m * BM; }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return t.n * BN; }
  __device__ __forceinline__ void attach_smem(uint8_t*) {}
  __device__ __forceinline__ void attach_patch(uint8_t* p) {
    if ((ldd & 7) == 0 && ((reinterpret_cast<uintptr_t>(D) | reinterpret_cast<uintptr_t>(pre)) & 15) == 0) patch = p;
  }
  // The pre-activations of a strip are fetched one strip ahead (four 16-byte loads per lane, eight rows per instruction)
  // and parked in registers: their latency passes behind the previous strip's arithmetic instead of in front of this one's.
  dev::Vec16 ahead[4];
  __device__ __forceinline__ void fetch_ahead(const TileCoord& t, int quarter, int lane, int col_in_tile) {
    const __nv_bfloat16* g0 = pre + static_cast<long long>(t.m * BM + quarter * 32) * ldd + t.n * BN + col_in_tile + (lane & 3) * 8;
#pragma unroll
    for (int j = 0; j < 4; ++j) ahead[j] = dev::ld16(g0 + ((lane >> 2) + 8 * j) * ldd);
  }
  // columns that one epilogue warp walks through: the whole tile, or half of it where two warps share a lane quarter
  __device__ __forceinline__ int span() const { return blockDim.x > 192 ? BN / 2 : BN; }
  __device__ __forceinline__ void tile_begin(const TileCoord& t) {
    if (patch) fetch_ahead(t, (threadIdx.x >> 5) & 3, threadIdx.x & 31, (((threadIdx.x >> 5) - 2) >> 2) * span());
  }
  __device__ __forceinline__ void tile_done(const TileCoord&, const volatile uint32_t*) {}

  __device__ __forceinline__ void strip(const TileCoord& t, int row_in_tile, int col_in_tile, uint32_t* r) {
    const int row = t.m * BM + row_in_tile, col = t.n * BN + col_in_tile;
    const long long at = static_cast<long long>(row) * ldd + col;
    float v[32];
    if (patch) {
      const int lane = row_in_tile & 31, quarter = (row_in_tile >> 5) & 3;
      uint8_t* P = my_patch(patch);
      const long long at0 = static_cast<long long>(row - lane) * ldd + col;
      float x[32];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<dev::Vec16*>(P + ((lane >> 2) + 8 * j) * kPatchRowBytes + (lane & 3) * 16) = ahead[j];
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 4; ++i) dev::unpack<DT_BF16>(*reinterpret_cast<const dev::Vec16*>(P + lane * kPatchRowBytes + i * 16), x + 8 * i);
      __syncwarp();
      if (((col_in_tile + 32) & (span() - 1)) != 0) fetch_ahead(t, quarter, lane, col_in_tile + 32);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * dgelu_tanh(x[i]);
      patch_store_bf16(P, lane, D + at0, ldd, v, 32);
    } else {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        float x[8];
        dev::unpack<DT_BF16>(dev::ld16(pre + at + i), x);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i + j] = __uint_as_float(r[i + j]) * dgelu_tanh(x[j]);
      }
#pragma unroll
      for (int i = 0; i < 32; i += 8) dev::st16(D + at + i, dev::pack<DT_BF16>(v + i));
    }
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
  uint8_t* patch = nullptr;      // kPatchBytesPerCta of shared memory when the pipeline provides it (see above)

  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return t.m * BM; }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return t.n * BN; }
  __device__ __forceinline__ void attach_smem(uint8_t*) {}
  __device__ __forceinline__ void attach_patch(uint8_t* p) { patch = p; }
  __device__ __forceinline__ void tile_begin(const TileCoord&) {}
  __device__ __forceinline__ void tile_done(const TileCoord&, const volatile uint32_t*) {}

  // bf16 output, whole 32-column strip, through the coalescing patch: every lane of the warp takes part (rows past M are
  // computed and dropped at the store)
  __device__ __forceinline__ void strip_patched(int row, int col, int row_in_tile, float* v) {
    const int lane = row_in_tile & 31;
    uint8_t* P = my_patch(patch);
    const int row0 = row - lane, rows_valid = M - row0;
    const long long at0 = static_cast<long long>(row0) * ldd + col;
    if (flags & GEMM_BIAS) {
      if ((reinterpret_cast<uintptr_t>(bias) & 15) == 0) {
        float b[32];
#pragma unroll
        for (int i = 0; i < 32; i += 8) dev::unpack<DT_BF16>(dev::ld16(bias + col + i), b + i);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += b[i];
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += __bfloat162float(bias[col + i]);
      }
    }
    if (flags & GEMM_ADD_D2) {
      float res[32];
      patch_load_bf16(P, lane, static_cast<const __nv_bfloat16*>(D2) + at0, ldd, res, rows_valid);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] += res[i];
    }
    if (flags & GEMM_GELU_INPLACE) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
    }
    if (flags & GEMM_ACCUMULATE) {
      float old[32];
      patch_load_bf16(P, lane, static_cast<const __nv_bfloat16*>(D) + at0, ldd, old, rows_valid);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] += old[i];
    }
    patch_store_bf16(P, lane, static_cast<__nv_bfloat16*>(D) + at0, ldd, v, rows_valid);
    if (flags & GEMM_GELU) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
      patch_store_bf16(P, lane, static_cast<__nv_bfloat16*>(D2) + at0, ldd, v, rows_valid);
    }
  }

  __device__ __forceinline__ void strip(const TileCoord& t, int row_in_tile, int col_in_tile, uint32_t* r) {
    const int row = t.m * BM + row_in_tile, col = t.n * BN + col_in_tile;
    if (col >= N) return;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    const bool full = col + 32 <= N;
    // uniform over the warp: the patch needs all 32 lanes; 16-byte alignment of every row's strip comes with ldd % 8 == 0
    if (patch && full && !(flags & (GEMM_OUT_F32 | GEMM_ROW_STORES)) && (col & 7) == 0 && row - (row_in_tile & 31) < M && (ldd & 7) == 0 &&
        ((reinterpret_cast<uintptr_t>(D) | ((flags & (GEMM_GELU | GEMM_ADD_D2)) ? reinterpret_cast<uintptr_t>(D2) : 0)) & 15) == 0) {
      strip_patched(row, col, row_in_tile, v);
      return;
    }
    if (row >= M) return;
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
