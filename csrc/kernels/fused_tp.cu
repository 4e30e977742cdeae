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

__device__ __forceinline__ unsigned long long* cta_probe(unsigned long long* probe) {
  return probe ? probe + static_cast<long long>(blockIdx.y * gridDim.x + blockIdx.x) * kProbeWords : nullptr;
}
__device__ __forceinline__ void probe_stamp(unsigned long long* p, int word) {
  if (p && threadIdx.x == 0) p[word] = dev::global_timer_ns();
}

template <bool B_MN, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1) ag_gemm_kernel(const __grid_constant__ AgGemmArgs A) {
  const AgGemmRank& R = A.r[blockIdx.y];
  unsigned long long* const probe = cta_probe(A.probe);
  probe_stamp(probe, 4);
  const bool copier = static_cast<int>(blockIdx.x) < A.n_copy;      // n_copy is even with PAIR: whole clusters copy
  if (copier) {
    if (A.w.world > 1) ag_push_role(A, R);
    if (A.tail_tiles <= 0) {
      probe_stamp(probe, 5);
      return;
    }
  }
  // The tile order is cut in two: the GEMM CTAs take all but the last tail_tiles, the copy CTAs take those once their
  // rows are on their way (otherwise their SMs would sit idle for the rest of the kernel).
  const int tiles_ml = A.M_local / BM, tiles_n = (A.N + BN - 1) / BN;
  const int unit = PAIR ? 2 : 1;
  const long long total = static_cast<long long>(A.w.world) * (tiles_ml / unit) * tiles_n;
  const long long tail = A.n_copy > 0 ? (A.tail_tiles < total ? A.tail_tiles : total) : 0;
  const int group_first = copier ? static_cast<int>(blockIdx.x) / unit : (static_cast<int>(blockIdx.x) - A.n_copy) / unit;
  const int group_size = copier ? A.n_copy / unit : (static_cast<int>(gridDim.x) - A.n_copy) / unit;
  AgSched sched{R.rank, A.w.world, tiles_ml / unit, tiles_n, group_first, group_size, copier ? total - tail : 0, copier ? total : total - tail};
  AgGate gate{reinterpret_cast<const uint32_t*>(A.w.heap[R.rank] + A.ready_off), R.rank,
              static_cast<uint32_t>(A.epoch) * static_cast<uint32_t>(A.n_copy), A.spin_ns, probe};
  StoreEpi epi{R.D, nullptr, static_cast<const __nv_bfloat16*>(R.bias), R.ldd, A.M, A.N, A.flags};
  if constexpr (PAIR) {
    const int cta = static_cast<int>(tc::cluster_ctarank());
    gemm2::PairEpi<StoreEpi> pe{epi, cta};
    gemm2::PairGate<AgGate> pg{gate, cta};
    gemm2::run<false, B_MN>(&R.tmA, &R.tmB, A.K, sched, pg, pe, R.status);
  } else {
    run<false, B_MN>(&R.tmA, &R.tmB, A.K, sched, gate, epi, R.status);
  }
  probe_stamp(probe, 5);
}

template <bool B_MN, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_rs_kernel(const __grid_constant__ GemmRsArgs A) {
  const GemmRsRank& R = A.r[blockIdx.y];
  unsigned long long* const probe = cta_probe(A.probe);
  probe_stamp(probe, 4);
  const int tiles_ml = A.M_local / BM, tiles_n = A.N / BN;
  if constexpr (PAIR) {
    RsSched sched{R.rank, A.w.world, tiles_ml / 2, tiles_n, static_cast<int>(blockIdx.x) >> 1, static_cast<int>(gridDim.x) >> 1};
    NoGate gate;
    RsEpiRow epi{{&A, &R, nullptr, R.rank, tiles_ml, tiles_n, probe}};
    const int cta = static_cast<int>(tc::cluster_ctarank());
    gemm2::PairEpi<RsEpiRow> pe{epi, cta};
    gemm2::PairGate<NoGate> pg{gate, cta};
    gemm2::run<false, B_MN, RsSched, gemm2::PairGate<NoGate>, gemm2::PairEpi<RsEpiRow>, 5>(&R.tmA, &R.tmB, A.K, sched, pg, pe, R.status);
  } else {
    RsSched sched{R.rank, A.w.world, tiles_ml, tiles_n, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x)};
    NoGate gate;
    RsEpi epi{&A, &R, nullptr, R.rank, tiles_ml, tiles_n, probe};
    run<false, B_MN>(&R.tmA, &R.tmB, A.K, sched, gate, epi, R.status);
  }
  probe_stamp(probe, 5);
}

// shared memory of the CTA-pair reduce-scatter kernel: five operand stages, barriers, 64 KiB of row staging
constexpr int RS_PAIR_SMEM_BYTES = 5 * gemm2::STAGE_BYTES + 1024 + gemm2::BAR_BYTES + kRsRowStageBytes;
static_assert(RS_PAIR_SMEM_BYTES <= 227 * 1024, "reduce-scatter pair kernel: shared memory");

unsigned long long* g_probe = nullptr;

thread_local std::string g_err;

}  // namespace

const char* fusedLastError() { return g_err.c_str(); }

void setFusedProbe(unsigned long long* device_buffer) { g_probe = device_buffer; }

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
  A.probe = g_probe;
  if (A.tail_tiles < 0 && A.n_copy > 0) {
    // Size of the tail from a cost model: the copy CTAs are busy for about t_copy (a copy CTA was measured to push about
    // 6.6 GB/s: 24 KiB in flight against a few microseconds of store round trip), a tile takes t_tile at ~1.5 PFLOP/s over
    // the whole GPU; the tail makes both groups finish together:
    //   (T - R) / G = t_copy / t_tile + R / C   with T tiles, G GEMM groups, C copy groups.
    const int unit = pair ? 2 : 1;
    const double T = static_cast<double>(A.w.world) * (A.M_local / (BM * unit)) * ((A.N + BN - 1) / BN);
    const double C = A.n_copy / unit, G = (ctas - A.n_copy) / unit;
    const double t_tile = 2.0 * BM * unit * BN * A.K / (1.5e15 / (148.0 / unit));
    const bool mc = A.w.mc_heap != nullptr && A.nvirt <= 1;      // one multicast store reaches every peer
    const double bytes = static_cast<double>(mc ? 1 : A.w.world - 1) * A.M_local * A.K * (A.elem_bytes ? A.elem_bytes : 2);
    const double t_copy = bytes / (6.6e9 * A.n_copy) + 20e-6;
    double Rt = (T - G * t_copy / t_tile) * C / (G + C);
    A.tail_tiles = Rt > 0 ? static_cast<int>(Rt) : 0;
  }
  if (A.tail_tiles < 0) A.tail_tiles = 0;
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
  const int smem_bytes = pair ? gemm2::SMEM_BYTES : SMEM_BYTES;      // the pair pipeline's ring and barrier area are its own
  if (!set[which]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    set[which] = true;
  }
  if (pair) return static_cast<int>(gemm2::launch_pairs(kern, grid, NUM_THREADS, smem_bytes, stream, true, A));
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
  A.probe = g_probe;
  if (pair) {
    for (int v = 0; v < nv; ++v) {
      const bool okB = host[v].b_mn ? true : makeTensorMap2D(&A.r[v].tmB, host[v].W, TM_BF16, A.K, A.N, host[v].ldw, BK, 128, &g_err);
      if (!okB) return static_cast<int>(cudaErrorInvalidValue);
    }
  }
  dim3 grid(ctas, nv);
  const int which = (host[0].b_mn ? 1 : 0) + (pair ? 2 : 0);
  const int smem_bytes = pair ? RS_PAIR_SMEM_BYTES : RS_SMEM_BYTES;
  static bool set[4] = {false, false, false, false};
  auto k00 = gemm_rs_kernel<false, false>; auto k10 = gemm_rs_kernel<true, false>;
  auto k01 = gemm_rs_kernel<false, true>;  auto k11 = gemm_rs_kernel<true, true>;
  auto kern = which == 0 ? k00 : which == 1 ? k10 : which == 2 ? k01 : k11;
  if (!set[which]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    set[which] = true;
  }
  if (pair) return static_cast<int>(gemm2::launch_pairs(kern, grid, NUM_THREADS, smem_bytes, stream, true, A));
  void* args[] = {&A};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kern), grid, dim3(NUM_THREADS), args, smem_bytes, stream));
}

}  // namespace pccl
