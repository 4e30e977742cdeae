// Tensor/sequence-parallel MLP halves with the collective fused into the GEMM kernel, tile by tile.
//
//   all-gather -> GEMM   Y[M,N] = gather_rows(X)[M,K] * W1[N,K]^T.  Every rank keeps its own row
//       block of X inside a symmetric [M,K] buffer.  A few CTAs of the kernel push the rank's rows
//       into every peer's buffer over NVLink (posted 16-byte stores, peers served in the order in
//       which they will consume the panel) in 128-row chunks and bump a counter per chunk on the
//       receiver; the other CTAs run the tcgen05 pipeline, starting with the local rows and taking
//       the remote panels in arrival order; a tile's TMA loads are issued once its chunk's counter
//       is complete.  TMA only ever reads local memory and nothing uses cluster multicast.
//   GEMM -> reduce-scatter   Z_r = sum over ranks of (Y*W2^T)[rows of r].  Tiles are computed owner
//       by owner, the local owner last.  A tile owned by a peer is rounded to bf16, staged through
//       shared memory and written into that peer's staging slot with bulk copies, followed by a
//       release flag; a tile owned by this rank waits for the seven peer partials of the same tile
//       (which were computed earlier) and folds them into its own fp32 accumulator in the epilogue,
//       so the reduction needs no extra pass and no tail.
//
// The reference lists "communication-computation overlap" as a feature and contains no code for it.
#include <cooperative_groups.h>
#include <cuda.h>

#include <string>

#include "fused_api.h"
#include "fused_tp.cuh"
#include "gemm_pipeline2.cuh"
#include "tensormap.h"

namespace pccl {

namespace {

using namespace gemm;
using namespace fused;

template <bool B_MN, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1) ag_gemm_kernel(const __grid_constant__ AgGemmArgs A) {
  const AgGemmRank& R = A.r[blockIdx.y];
  if (static_cast<int>(blockIdx.x) < A.n_copy) {      // n_copy is even with PAIR: whole clusters copy
    if (A.w.world > 1) ag_push_role(A, R);
    return;
  }
  const int tiles_ml = A.M_local / BM, tiles_n = (A.N + BN - 1) / BN;
  if constexpr (PAIR) {
    AgSched sched{R.rank, A.w.world, tiles_ml / 2, tiles_n, (static_cast<int>(blockIdx.x) - A.n_copy) >> 1,
                  (static_cast<int>(gridDim.x) - A.n_copy) >> 1};
    AgGate gate{reinterpret_cast<const uint32_t*>(A.w.heap[R.rank] + A.ready_off), R.rank,
                static_cast<uint32_t>(A.epoch) * static_cast<uint32_t>(A.n_copy), A.spin_ns};
    StoreEpi epi{R.D, nullptr, static_cast<const __nv_bfloat16*>(R.bias), R.ldd, A.M, A.N, A.flags};
    const int cta = static_cast<int>(tc::cluster_ctarank());
    gemm2::PairEpi<StoreEpi> pe{epi, cta};
    gemm2::PairGate<AgGate> pg{gate, cta};
    gemm2::run<false, B_MN>(&R.tmA, &R.tmB, A.K, sched, pg, pe, R.status);
    return;
  }
  AgSched sched{R.rank, A.w.world, tiles_ml, tiles_n, static_cast<int>(blockIdx.x) - A.n_copy, static_cast<int>(gridDim.x) - A.n_copy};
  AgGate gate{reinterpret_cast<const uint32_t*>(A.w.heap[R.rank] + A.ready_off), R.rank, static_cast<uint32_t>(A.epoch) * static_cast<uint32_t>(A.n_copy), A.spin_ns};
  StoreEpi epi{R.D, nullptr, static_cast<const __nv_bfloat16*>(R.bias), R.ldd, A.M, A.N, A.flags};
  run<false, B_MN>(&R.tmA, &R.tmB, A.K, sched, gate, epi, R.status);
}

template <bool B_MN, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_rs_kernel(const __grid_constant__ GemmRsArgs A) {
  const GemmRsRank& R = A.r[blockIdx.y];
  const int tiles_ml = A.M_local / BM, tiles_n = A.N / BN;
  if constexpr (PAIR) {
    RsSched sched{R.rank, A.w.world, tiles_ml / 2, tiles_n, static_cast<int>(blockIdx.x) >> 1, static_cast<int>(gridDim.x) >> 1};
    NoGate gate;
    RsEpi epi{&A, &R, nullptr, R.rank, tiles_ml, tiles_n};
    const int cta = static_cast<int>(tc::cluster_ctarank());
    gemm2::PairEpi<RsEpi> pe{epi, cta};
    gemm2::PairGate<NoGate> pg{gate, cta};
    gemm2::run<false, B_MN>(&R.tmA, &R.tmB, A.K, sched, pg, pe, R.status);
    return;
  }
  RsSched sched{R.rank, A.w.world, tiles_ml, tiles_n, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x)};
  NoGate gate;
  RsEpi epi{&A, &R, nullptr, R.rank, tiles_ml, tiles_n};
  run<false, B_MN>(&R.tmA, &R.tmB, A.K, sched, gate, epi, R.status);
}

thread_local std::string g_err;

}  // namespace

const char* fusedLastError() { return g_err.c_str(); }

int launchAgGemm(AgGemmArgs& A, const AgGemmHost* host, int ctas, cudaStream_t stream) {
  const int nv = A.nvirt > 1 ? A.nvirt : 1;
  if (nv > kMaxVirt) { g_err = "ag_gemm: at most 4 emulated ranks"; return static_cast<int>(cudaErrorInvalidValue); }
  if (A.M_local % BM || A.M != A.M_local * A.w.world || A.K % 8) {
    g_err = "ag_gemm: rows per rank must be a multiple of 128 and K a multiple of 8";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  for (int v = 0; v < nv; ++v) {
    // gathered X lives at x_off of this rank's own heap: TMA reads local memory only
    const void* xg = A.w.heap[A.r[v].rank] + A.x_off;
    if (!makeTensorMap2D(&A.r[v].tmA, xg, TM_BF16, A.K, A.M, A.K, BK, BM, &g_err)) return static_cast<int>(cudaErrorInvalidValue);
    if (host[v].b_mn != host[0].b_mn) { g_err = "ag_gemm: all ranks must use the same operand form"; return static_cast<int>(cudaErrorInvalidValue); }
    const bool okB = host[v].b_mn ? makeTensorMap2D(&A.r[v].tmB, host[v].W, TM_BF16, A.N, A.K, host[v].ldw, 64, BK, &g_err)
                                  : makeTensorMap2D(&A.r[v].tmB, host[v].W, TM_BF16, A.K, A.N, host[v].ldw, BK, BN, &g_err);
    if (!okB) return static_cast<int>(cudaErrorInvalidValue);
  }
  if (A.w.world == 1) A.n_copy = 0;
  if (ctas <= A.n_copy) { g_err = "ag_gemm: need more CTAs than copy CTAs"; return static_cast<int>(cudaErrorInvalidValue); }
  const bool pair = A.M_local % 256 == 0 && ctas % 2 == 0;
  if (pair && (A.n_copy & 1)) A.n_copy += 1;
  // per-CTA TMA boxes: 128 rows of A; 256 rows of B (single CTA) or 128 (pair)
  if (pair) {
    for (int v = 0; v < nv; ++v) {
      const bool okB = host[v].b_mn ? true : makeTensorMap2D(&A.r[v].tmB, host[v].W, TM_BF16, A.K, A.N, host[v].ldw, BK, 128, &g_err);
      if (!okB) return static_cast<int>(cudaErrorInvalidValue);
    }
  }
  dim3 grid(ctas, nv);
  const int which = (host[0].b_mn ? 1 : 0) + (pair ? 2 : 0);
  static bool set[4] = {false, false, false, false};
  auto k00 = ag_gemm_kernel<false, false>; auto k10 = ag_gemm_kernel<true, false>;
  auto k01 = ag_gemm_kernel<false, true>;  auto k11 = ag_gemm_kernel<true, true>;
  auto kern = which == 0 ? k00 : which == 1 ? k10 : which == 2 ? k01 : k11;
  if (!set[which]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    set[which] = true;
  }
  if (pair) return static_cast<int>(gemm2::launch_pairs(kern, grid, NUM_THREADS, SMEM_BYTES, stream, true, A));
  void* args[] = {&A};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kern), grid, dim3(NUM_THREADS), args, SMEM_BYTES, stream));
}

int launchGemmRs(GemmRsArgs& A, const GemmRsHost* host, int ctas, cudaStream_t stream) {
  const int nv = A.nvirt > 1 ? A.nvirt : 1;
  if (nv > kMaxVirt) { g_err = "gemm_rs: at most 4 emulated ranks"; return static_cast<int>(cudaErrorInvalidValue); }
  if (A.M_local % BM || A.M != A.M_local * A.w.world || A.N % BN || A.K % 8) {
    g_err = "gemm_rs: rows per rank must be a multiple of 128, N a multiple of 256, K a multiple of 8";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  for (int v = 0; v < nv; ++v) {
    if (!makeTensorMap2D(&A.r[v].tmA, host[v].Y, TM_BF16, A.K, A.M, host[v].ldy, BK, BM, &g_err)) return static_cast<int>(cudaErrorInvalidValue);
    if (host[v].b_mn != host[0].b_mn) { g_err = "gemm_rs: all ranks must use the same operand form"; return static_cast<int>(cudaErrorInvalidValue); }
    const bool okB = host[v].b_mn ? makeTensorMap2D(&A.r[v].tmB, host[v].W, TM_BF16, A.N, A.K, host[v].ldw, 64, BK, &g_err)
                                  : makeTensorMap2D(&A.r[v].tmB, host[v].W, TM_BF16, A.K, A.N, host[v].ldw, BK, BN, &g_err);
    if (!okB) return static_cast<int>(cudaErrorInvalidValue);
  }
  const bool pair = A.M_local % 256 == 0 && ctas % 2 == 0;
  if (pair) {
    for (int v = 0; v < nv; ++v) {
      const bool okB = host[v].b_mn ? true : makeTensorMap2D(&A.r[v].tmB, host[v].W, TM_BF16, A.K, A.N, host[v].ldw, BK, 128, &g_err);
      if (!okB) return static_cast<int>(cudaErrorInvalidValue);
    }
  }
  dim3 grid(ctas, nv);
  const int which = (host[0].b_mn ? 1 : 0) + (pair ? 2 : 0);
  static bool set[4] = {false, false, false, false};
  auto k00 = gemm_rs_kernel<false, false>; auto k10 = gemm_rs_kernel<true, false>;
  auto k01 = gemm_rs_kernel<false, true>;  auto k11 = gemm_rs_kernel<true, true>;
  auto kern = which == 0 ? k00 : which == 1 ? k10 : which == 2 ? k01 : k11;
  if (!set[which]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, RS_SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    set[which] = true;
  }
  if (pair) return static_cast<int>(gemm2::launch_pairs(kern, grid, NUM_THREADS, RS_SMEM_BYTES, stream, true, A));
  void* args[] = {&A};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kern), grid, dim3(NUM_THREADS), args, RS_SMEM_BYTES, stream));
}

}  // namespace pccl
