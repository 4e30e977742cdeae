// Block-scaled fp8 forms of the fused tensor-parallel kernels (protocols: fused_tp.cu; GEMM pipeline:
// gemm_fp8_pipeline.cuh).
//
//   all-gather -> GEMM   the copy CTAs push e4m3 rows AND their 1 x 128 scales (half the NVLink bytes of
//       bf16); the epilogue either stores bf16, or applies bias/GELU and re-quantises: every epilogue
//       thread holds 128 consecutive columns of one row, which is exactly one 1 x 128 block, so the
//       block maximum needs no exchange between threads.  The quantised output feeds the second GEMM.
//   GEMM -> reduce-scatter   e4m3 operands, fp32 promotion, and the same bf16 partial-tile exchange
//       as the bf16 kernel, run by eight epilogue warps.
//
// The reference has no fused path and no fp8 arithmetic.
#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_fp8.h>

#include <string>

#include "fused_api.h"
#include "fused_tp.cuh"
#include "gemm_fp8_pipeline.cuh"
#include "gemm_mx8_pipeline.cuh"
#include "tensormap.h"

namespace pccl {

namespace {

using namespace fused;
using gemm::TileCoord;

// Output of the first GEMM as a block-scaled fp8 activation.
struct QuantEpi {
  static constexpr bool kRow128 = true;
  uint8_t* Dq;
  float* Ds;
  const __nv_bfloat16* bias;
  long long ldq;
  int ld_s, M, N;
  uint32_t flags;

  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return t.m * gemm8::BM; }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return t.n * gemm8::BN; }
  __device__ __forceinline__ void attach_smem(uint8_t*) {}
  __device__ __forceinline__ void tile_begin(const TileCoord&) {}
  __device__ __forceinline__ void tile_done(const TileCoord&, const volatile uint32_t*) {}
  __device__ __forceinline__ void strip(const TileCoord&, int, int, uint32_t*) {}

  __device__ __forceinline__ void row128(const TileCoord& t, int row_in_tile, int col_in_tile, float* v) {
    const int row = t.m * gemm8::BM + row_in_tile, col = t.n * gemm8::BN + col_in_tile;
    if (row >= M || col >= N) return;            // N is a multiple of 128 here
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 128; ++i) {
      float x = v[i];
      if (flags & GEMM_BIAS) x += __bfloat162float(bias[col + i]);
      if (flags & GEMM_GELU_INPLACE) x = gemm::gelu_tanh(x);
      v[i] = x;
      amax = fmaxf(amax, fabsf(x));
    }
    const float scale = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
    const float inv = 1.0f / scale;
    Ds[static_cast<long long>(row) * ld_s + (col >> 7)] = scale;
    uint8_t* d = Dq + static_cast<long long>(row) * ldq + col;
#pragma unroll
    for (int i = 0; i < 128; i += 16) {
      uint32_t w[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[i + 4 * h] * inv, v[i + 4 * h + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[i + 4 * h + 2] * inv, v[i + 4 * h + 3] * inv), __NV_SATFINITE, __NV_E4M3);
        w[h] = (lo & 0xffffu) | (hi << 16);
      }
      *reinterpret_cast<uint4*>(d + i) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
};

template <bool QUANT_OUT>
__global__ void __launch_bounds__(gemm8::NUM_THREADS, 1) ag_gemm_fp8_kernel(const __grid_constant__ AgGemmArgs A) {
  const AgGemmRank& R = A.r[blockIdx.y];
  if (static_cast<int>(blockIdx.x) < A.n_copy) {
    if (A.w.world > 1) ag_push_role(A, R);
    return;
  }
  const int tiles_ml = A.M_local / gemm8::BM, tiles_n = A.N / gemm8::BN;
  AgSched sched{R.rank, A.w.world, tiles_ml, tiles_n, static_cast<int>(blockIdx.x) - A.n_copy, static_cast<int>(gridDim.x) - A.n_copy, 0,
                static_cast<long long>(A.w.world) * tiles_ml * tiles_n};
  AgGate gate{reinterpret_cast<const uint32_t*>(A.w.heap[R.rank] + A.ready_off), R.rank,
              static_cast<uint32_t>(A.epoch) * static_cast<uint32_t>(A.n_copy), A.spin_ns};
  gemm8::Scales sc{reinterpret_cast<const float*>(A.w.heap[R.rank] + A.xs_off), R.w_scale, A.K / 128, R.ld_ws, A.M, A.N};
  if constexpr (QUANT_OUT) {
    QuantEpi epi{static_cast<uint8_t*>(R.Dq), R.Ds, static_cast<const __nv_bfloat16*>(R.bias), R.ldq, A.N / 128, A.M, A.N, A.flags};
    gemm8::run(&R.tmA, &R.tmB, A.K, sc, sched, gate, epi, R.status);
  } else {
    gemm::StoreEpi epi{R.D, nullptr, static_cast<const __nv_bfloat16*>(R.bias), R.ldd, A.M, A.N, A.flags};
    gemm8::run(&R.tmA, &R.tmB, A.K, sc, sched, gate, epi, R.status);
  }
}

// all-gather -> GEMM with hardware block scaling: e4m3 rows and their UE8M0 scale bytes are pushed, the tensor core
// applies the scales (gemm_mx8_pipeline.cuh), 224-column tiles.
__global__ void __launch_bounds__(gemmx::NUM_THREADS, 1) ag_gemm_mx8_kernel(const __grid_constant__ AgGemmArgs A) {
  const AgGemmRank& R = A.r[blockIdx.y];
  if (static_cast<int>(blockIdx.x) < A.n_copy) {
    if (A.w.world > 1) ag_push_role(A, R);
    return;
  }
  const int tiles_ml = A.M_local / gemmx::BM, tiles_n = (A.N + gemmx::BN - 1) / gemmx::BN;
  AgSched sched{R.rank, A.w.world, tiles_ml, tiles_n, static_cast<int>(blockIdx.x) - A.n_copy, static_cast<int>(gridDim.x) - A.n_copy, 0,
                static_cast<long long>(A.w.world) * tiles_ml * tiles_n};
  AgGate gate{reinterpret_cast<const uint32_t*>(A.w.heap[R.rank] + A.ready_off), R.rank,
              static_cast<uint32_t>(A.epoch) * static_cast<uint32_t>(A.n_copy), A.spin_ns};
  gemmx::Scales sc{reinterpret_cast<const uint8_t*>(A.w.heap[R.rank] + A.xs_off), reinterpret_cast<const uint8_t*>(R.w_scale), A.K / 128,
                   R.ld_ws, A.M, A.N};
  gemm::StoreEpi epi{R.D, nullptr, static_cast<const __nv_bfloat16*>(R.bias), R.ldd, A.M, A.N, A.flags};
  gemmx::run(&R.tmA, &R.tmB, A.K, sc, sched, gate, epi, R.status);
}

constexpr int kRs8StageBytes = gemm8::EPI_WARPS * 32 * kRsPitch;
constexpr int kRs8Stages = 3;                      // 3 x 48 KiB of operands leave room for the staging rows
constexpr int RS8_SMEM_BYTES = gemm8::smem_bytes(kRs8Stages) + kRs8StageBytes;

__global__ void __launch_bounds__(gemm8::NUM_THREADS, 1) gemm_rs_fp8_kernel(const __grid_constant__ GemmRsArgs A) {
  const GemmRsRank& R = A.r[blockIdx.y];
  const int tiles_ml = A.M_local / gemm8::BM, tiles_n = A.N / gemm8::BN;
  RsSched sched{R.rank, A.w.world, tiles_ml, tiles_n, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x)};
  gemm::NoGate gate;
  RsEpiT<gemm8::EPI_WARPS> epi{&A, &R, nullptr, R.rank, tiles_ml, tiles_n};
  gemm8::Scales sc{R.y_scale, R.w_scale, R.ld_ys, R.ld_ws, A.M, A.N};
  gemm8::run<kRs8Stages>(&R.tmA, &R.tmB, A.K, sc, sched, gate, epi, R.status);
}

thread_local std::string g_err;

}  // namespace

int launchAgGemmFp8(AgGemmArgs& A, const AgGemmHost* host, int ctas, cudaStream_t stream) {
  const int nv = A.nvirt > 1 ? A.nvirt : 1;
  if (nv > kMaxVirt || A.M_local % gemm8::BM || A.M != A.M_local * A.w.world || A.K % 128 || A.N % gemm8::BN || !A.xs_off) {
    g_err = "ag_gemm fp8: rows per rank % 128, K % 128, N % 256, and a gathered-scale buffer are required";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  A.elem_bytes = 1;
  bool quant = A.r[0].Dq != nullptr;
  for (int v = 0; v < nv; ++v) {
    const void* xg = A.w.heap[A.r[v].rank] + A.x_off;     // TMA reads local memory only
    if (!makeTensorMap2D(&A.r[v].tmA, xg, TM_U8, A.K, A.M, A.K, gemm8::BK, gemm8::BM, &g_err)) return static_cast<int>(cudaErrorInvalidValue);
    if (host[v].b_mn || !A.r[v].w_scale || (A.r[v].Dq != nullptr) != quant) {
      g_err = "ag_gemm fp8: W is K-major with scales; all ranks use the same output form";
      return static_cast<int>(cudaErrorInvalidValue);
    }
    if (!makeTensorMap2D(&A.r[v].tmB, host[v].W, TM_U8, A.K, A.N, host[v].ldw, gemm8::BK, gemm8::BN, &g_err)) return static_cast<int>(cudaErrorInvalidValue);
  }
  if (A.w.world == 1) A.n_copy = 0;
  if (ctas <= A.n_copy) { g_err = "ag_gemm fp8: need more CTAs than copy CTAs"; return static_cast<int>(cudaErrorInvalidValue); }
  auto kern = quant ? ag_gemm_fp8_kernel<true> : ag_gemm_fp8_kernel<false>;
  static bool set[2] = {false, false};
  if (!set[quant]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm8::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    set[quant] = true;
  }
  dim3 grid(ctas, nv);
  void* args[] = {&A};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kern), grid, dim3(gemm8::NUM_THREADS), args, gemm8::SMEM_BYTES, stream));
}

int launchAgGemmMx8(AgGemmArgs& A, const AgGemmHost* host, int ctas, cudaStream_t stream) {
  const int nv = A.nvirt > 1 ? A.nvirt : 1;
  if (nv > kMaxVirt || A.M_local % gemmx::BM || A.M != A.M_local * A.w.world || A.K % 128 || A.N % 32 || !A.xs_off) {
    g_err = "ag_gemm mx8: rows per rank % 128, K % 128, N % 32, and a gathered-scale buffer are required";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  A.elem_bytes = 1;
  A.scale_bytes = 1;
  for (int v = 0; v < nv; ++v) {
    const void* xg = A.w.heap[A.r[v].rank] + A.x_off;     // TMA reads local memory only
    if (!makeTensorMap2D(&A.r[v].tmA, xg, TM_U8, A.K, A.M, A.K, gemmx::BK, gemmx::BM, &g_err)) return static_cast<int>(cudaErrorInvalidValue);
    if (host[v].b_mn || !A.r[v].w_scale || !A.r[v].D) {
      g_err = "ag_gemm mx8: W is K-major with scale bytes; the output is bf16";
      return static_cast<int>(cudaErrorInvalidValue);
    }
    if (!makeTensorMap2D(&A.r[v].tmB, host[v].W, TM_U8, A.K, A.N, host[v].ldw, gemmx::BK, gemmx::BN, &g_err)) return static_cast<int>(cudaErrorInvalidValue);
  }
  if (A.w.world == 1) A.n_copy = 0;
  if (ctas <= A.n_copy) { g_err = "ag_gemm mx8: need more CTAs than copy CTAs"; return static_cast<int>(cudaErrorInvalidValue); }
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(ag_gemm_mx8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemmx::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    set = true;
  }
  dim3 grid(ctas, nv);
  void* args[] = {&A};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ag_gemm_mx8_kernel), grid, dim3(gemmx::NUM_THREADS), args, gemmx::SMEM_BYTES, stream));
}

int launchGemmRsFp8(GemmRsArgs& A, const GemmRsHost* host, int ctas, cudaStream_t stream) {
  const int nv = A.nvirt > 1 ? A.nvirt : 1;
  if (nv > kMaxVirt || A.M_local % gemm8::BM || A.M != A.M_local * A.w.world || A.N % gemm8::BN || A.K % 128) {
    g_err = "gemm_rs fp8: rows per rank % 128, N % 256 and K % 128 are required";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  for (int v = 0; v < nv; ++v) {
    if (host[v].b_mn || !A.r[v].y_scale || !A.r[v].w_scale) { g_err = "gemm_rs fp8: K-major operands with scales"; return static_cast<int>(cudaErrorInvalidValue); }
    if (!makeTensorMap2D(&A.r[v].tmA, host[v].Y, TM_U8, A.K, A.M, host[v].ldy, gemm8::BK, gemm8::BM, &g_err)) return static_cast<int>(cudaErrorInvalidValue);
    if (!makeTensorMap2D(&A.r[v].tmB, host[v].W, TM_U8, A.K, A.N, host[v].ldw, gemm8::BK, gemm8::BN, &g_err)) return static_cast<int>(cudaErrorInvalidValue);
  }
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_rs_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RS8_SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    set = true;
  }
  dim3 grid(ctas, nv);
  void* args[] = {&A};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(gemm_rs_fp8_kernel), grid, dim3(gemm8::NUM_THREADS), args, RS8_SMEM_BYTES, stream));
}

}  // namespace pccl
