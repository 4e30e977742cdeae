// Plain bf16 GEMM on the tcgen05 pipeline (see gemm_pipeline.cuh) with a fused epilogue:
// optional bias, optional GELU side output, bf16 or fp32 store, optional accumulation into D.
// The reference has no GEMM of any kind (cutlass and composable_kernel are empty submodules,
// .gitmodules:4-9); this is the "computation" half of its "communication & computation" claim.
#include <cuda.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <string>
#include <utility>

#include "gemm_api.h"
#include "gemm_epilogue.cuh"
#include "gemm_pipeline.cuh"
#include "gemm_pipeline2.cuh"
#include "tensormap.h"

namespace pccl {

namespace {

using namespace gemm;

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, StoreEpi epi, int K,
                 uint32_t* status) {
  GroupedSched sched{(epi.M + BM - 1) / BM, (epi.N + BN - 1) / BN, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x)};
  NoGate gate;
  run<A_MN, B_MN>(&tmA, &tmB, K, sched, gate, epi, status);
}

// ---- CTA-pair kernel ---------------------------------------------------------------------------------
// GroupedSched's order, handed out tile by tile at run time (gemm2::run, DYN): `counter` is a zeroed word that belongs to
// the launching stream.
struct DynGroupedSched {
  int tiles_m, tiles_n;
  uint32_t* counter;
  uint32_t total;
  __device__ __forceinline__ bool at(int idx, TileCoord* t) const {
    const int per_group = GroupedSched::GROUP_M * tiles_n;
    const int g = idx / per_group, r = idx % per_group;
    const int gm = min(GroupedSched::GROUP_M, tiles_m - g * GroupedSched::GROUP_M);
    t->m = g * GroupedSched::GROUP_M + r % gm;
    t->n = r / gm;
    t->extra = 0;
    return true;
  }
};

template <bool A_MN, bool B_MN, class Epi = StoreEpi, bool DYN = false>
__global__ void __launch_bounds__(gemm2::NUM_THREADS_WIDE, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Epi epi, int K,
                      uint32_t* status, uint32_t* counter) {
  const int tiles_m = (epi.M + gemm2::PAIR_M - 1) / gemm2::PAIR_M, tiles_n = (epi.N + gemm2::BN - 1) / gemm2::BN;
  NoGate gate;
  const int cta = static_cast<int>(tc::cluster_ctarank());
  gemm2::PairEpi<Epi> pe{epi, cta};
  gemm2::PairGate<NoGate> pg{gate, cta};
  if constexpr (DYN) {
    DynGroupedSched sched{tiles_m, tiles_n, counter, static_cast<uint32_t>(tiles_m * tiles_n)};
    gemm2::run<A_MN, B_MN, DynGroupedSched, gemm2::PairGate<NoGate>, gemm2::PairEpi<Epi>, gemm2::STAGES, 1, true, 8>(&tmA, &tmB, K, sched, pg, pe, status);
  } else {
    GroupedSched sched{tiles_m, tiles_n, static_cast<int>(blockIdx.x >> 1), static_cast<int>(gridDim.x >> 1)};
    gemm2::run<A_MN, B_MN, GroupedSched, gemm2::PairGate<NoGate>, gemm2::PairEpi<Epi>, gemm2::STAGES, 1, false, 8>(&tmA, &tmB, K, sched, pg, pe, status);
  }
}

// ---- two GEMMs with one K as one tile list ---------------------------------------------------------------------------
struct DualMaps { CUtensorMap a[2], b[2]; };

struct DualSched {
  int tiles_m[2], tiles_n[2], first, stride;
  uint32_t* counter;       // dynamic scheduling: see DynGroupedSched; null = round-robin
  uint32_t total;
  __device__ __forceinline__ bool get(int it, TileCoord* t) const { return at(first + static_cast<long long>(it) * stride, t); }
  __device__ __forceinline__ bool at(long long idx, TileCoord* t) const {
    const long long n0 = static_cast<long long>(tiles_m[0]) * tiles_n[0];
    const int q = idx >= n0 ? 1 : 0;
    if (q) idx -= n0;
    if (idx >= static_cast<long long>(tiles_m[q]) * tiles_n[q]) return false;
    const int per_group = GroupedSched::GROUP_M * tiles_n[q];
    const int g = static_cast<int>(idx / per_group), r = static_cast<int>(idx % per_group);
    const int gm = min(GroupedSched::GROUP_M, tiles_m[q] - g * GroupedSched::GROUP_M);
    t->m = g * GroupedSched::GROUP_M + r % gm;
    t->n = r / gm;
    t->extra = q;
    return true;
  }
};

struct DualEpi {
  static constexpr bool kRow128 = false;
  StoreEpi e[2];
  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return e[t.extra].a_row0(t); }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return e[t.extra].b_row0(t); }
  __device__ __forceinline__ void attach_smem(uint8_t*) {}
  __device__ __forceinline__ void attach_patch(uint8_t* p) { e[0].attach_patch(p); e[1].attach_patch(p); }
  __device__ __forceinline__ void tile_begin(const TileCoord&) {}
  __device__ __forceinline__ void tile_done(const TileCoord&, const volatile uint32_t*) {}
  __device__ __forceinline__ void strip(const TileCoord& t, int row, int col, uint32_t* r) { e[t.extra].strip(t, row, col, r); }
};

template <bool A_MN, bool B_MN, bool DYN>
__global__ void __launch_bounds__(gemm2::NUM_THREADS_WIDE, 1)
gemm_bf16_pair_dual_kernel(const __grid_constant__ DualMaps maps, DualEpi epi, int K, uint32_t* status, uint32_t* counter) {
  DualSched sched{{(epi.e[0].M + gemm2::PAIR_M - 1) / gemm2::PAIR_M, (epi.e[1].M + gemm2::PAIR_M - 1) / gemm2::PAIR_M},
                  {(epi.e[0].N + gemm2::BN - 1) / gemm2::BN, (epi.e[1].N + gemm2::BN - 1) / gemm2::BN},
                  static_cast<int>(blockIdx.x >> 1), static_cast<int>(gridDim.x >> 1), counter, 0u};
  sched.total = static_cast<uint32_t>(sched.tiles_m[0] * sched.tiles_n[0] + sched.tiles_m[1] * sched.tiles_n[1]);
  NoGate gate;
  const int cta = static_cast<int>(tc::cluster_ctarank());
  gemm2::PairEpi<DualEpi> pe{epi, cta};
  gemm2::PairGate<NoGate> pg{gate, cta};
  gemm2::run<A_MN, B_MN, DualSched, gemm2::PairGate<NoGate>, gemm2::PairEpi<DualEpi>, gemm2::STAGES, 2, DYN, 8>(maps.a, maps.b, K, sched, pg, pe, status);
}

thread_local std::string g_err;

// The zeroed counter word that dynamic tile scheduling of launches on `stream` uses (kernels on one stream run one after
// the other, and each leaves the word zeroed).  One 128-byte line per stream out of a pool made on first use; a null
// pointer (pool used up, or PCCL_GEMM_DYNAMIC=0) selects the round-robin kernels.
int g_dynamic = -1;      // -1: PCCL_GEMM_DYNAMIC decides (default on); 0 / 1: set by gemmSetDynamic
std::mutex g_counter_mu;
std::map<int, std::pair<uint32_t*, int>> g_counter_pools;      // device -> (base, lines handed out)
constexpr int kCounterPool = 64, kCounterStride = 32;          // lines per device, words per line

uint32_t* tileCounterFor(cudaStream_t stream) {
  static const bool env_off = std::getenv("PCCL_GEMM_DYNAMIC") && std::getenv("PCCL_GEMM_DYNAMIC")[0] == '0';
  if (g_dynamic == 0 || (g_dynamic < 0 && env_off)) return nullptr;
  constexpr int kPool = kCounterPool, kStride = kCounterStride;
  static std::map<std::pair<int, cudaStream_t>, uint32_t*> by_stream;
  auto& pools = g_counter_pools;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> g(g_counter_mu);
  auto it = by_stream.find({dev, stream});
  if (it != by_stream.end()) return it->second;
  auto& pool = pools[dev];
  if (!pool.first) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
    uint32_t* base = nullptr;
    if (cudaMalloc(&base, kPool * kStride * sizeof(uint32_t)) != cudaSuccess) return nullptr;
    if (cudaMemset(base, 0, kPool * kStride * sizeof(uint32_t)) != cudaSuccess) return nullptr;
    pool = {base, 0};
  }
  if (pool.second >= kPool) return nullptr;
  uint32_t* p = pool.first + static_cast<size_t>(pool.second++) * kStride;
  by_stream[{dev, stream}] = p;
  return p;
}

template <class Kern>
int setPairSmem(Kern kern, bool* done) {
  if (*done) return 0;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm2::SMEM_BYTES);
  if (e != cudaSuccess) return static_cast<int>(e);
  *done = true;
  return 0;
}

template <bool A_MN, bool B_MN, class Epi = StoreEpi>
int launchPair(const CUtensorMap& ta, const CUtensorMap& tb, const Epi& epi, int K, int grid, uint32_t* status, cudaStream_t stream) {
  static bool attr_set = false, attr_set_dyn = false;
  uint32_t* counter = tileCounterFor(stream);
  if (counter) {
    auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, Epi, true>;
    if (int e = setPairSmem(kern, &attr_set_dyn)) return e;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(gemm2::NUM_THREADS_WIDE);
    cfg.dynamicSmemBytes = gemm2::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int Kc = K;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, ta, tb, epi, Kc, status, counter));
  }
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, Epi, false>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm2::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(gemm2::NUM_THREADS_WIDE);
  cfg.dynamicSmemBytes = gemm2::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int Kc = K;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, ta, tb, epi, Kc, status, static_cast<uint32_t*>(nullptr)));
}

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

void gemmSetDynamic(int mode) { g_dynamic = mode < 0 ? -1 : (mode ? 1 : 0); }

int gemmResetTileCounters() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> g(g_counter_mu);
  auto it = g_counter_pools.find(dev);
  if (it == g_counter_pools.end() || !it->second.first) return 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return static_cast<int>(cudaGetLastError());
  return static_cast<int>(cudaMemset(it->second.first, 0, kCounterPool * kCounterStride * sizeof(uint32_t)));
}

int gemmBf16(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K,
             uint32_t flags, const void* bias, void* D2, int sms, uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda | ldb | ldd) % 8 || (reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D)) % 16) {
    g_err = "gemmBf16: strides must be multiples of 8 elements and pointers 16-byte aligned";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if ((flags & GEMM_ADD_D2) && (!D2 || (flags & (GEMM_OUT_F32 | GEMM_GELU)))) {
    g_err = "gemmBf16: the residual input needs D2 and a bf16 D, and excludes the GELU side output";
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
  if (flags & GEMM_PAIR) {
    // per-CTA boxes: 128 rows of A and 128 rows (half of N) of B
    CUtensorMap pa, pb;
    if (!a_mn ? !makeTensorMap2D(&pa, A, TM_BF16, K, M, lda, BK, 128, &g_err) : !makeTensorMap2D(&pa, A, TM_BF16, M, K, lda, 64, BK, &g_err))
      return static_cast<int>(cudaErrorInvalidValue);
    if (!b_mn ? !makeTensorMap2D(&pb, B, TM_BF16, K, N, ldb, BK, 128, &g_err) : !makeTensorMap2D(&pb, B, TM_BF16, N, K, ldb, 64, BK, &g_err))
      return static_cast<int>(cudaErrorInvalidValue);
    int pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
    int n_sm2 = deviceSmCount();
    if (sms > 0 && sms < n_sm2) n_sm2 = sms;
    int grid2 = 2 * (pair_tiles < n_sm2 / 2 ? pair_tiles : n_sm2 / 2);
    if (a_mn) return b_mn ? launchPair<true, true>(pa, pb, epi, K, grid2, status, stream) : launchPair<true, false>(pa, pb, epi, K, grid2, status, stream);
    return b_mn ? launchPair<false, true>(pa, pb, epi, K, grid2, status, stream) : launchPair<false, false>(pa, pb, epi, K, grid2, status, stream);
  }
  int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int n_sm = deviceSmCount();
  if (sms > 0 && sms < n_sm) n_sm = sms;
  int grid = tiles < n_sm ? tiles : n_sm;
  if (a_mn) return b_mn ? launch<true, true>(ta, tb, epi, K, grid, status, stream) : launch<true, false>(ta, tb, epi, K, grid, status, stream);
  return b_mn ? launch<false, true>(ta, tb, epi, K, grid, status, stream) : launch<false, false>(ta, tb, epi, K, grid, status, stream);
}

int gemmBf16Dgelu(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, const void* pre, float* colsum,
                  int M, int N, int K, uint32_t flags, int sms, uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda | ldb | ldd) % 8 || M % 256 || N % 256 ||
      (reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D) | reinterpret_cast<uintptr_t>(pre)) % 16) {
    g_err = "gemmBf16Dgelu: M and N must be multiples of 256, strides multiples of 8 elements, pointers 16-byte aligned";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  const bool a_mn = flags & GEMM_A_MN, b_mn = flags & GEMM_B_MN;
  if (a_mn) {
    g_err = "gemmBf16Dgelu: an MN-major A operand is not built";
    return static_cast<int>(cudaErrorInvalidValue);
  }
  CUtensorMap pa, pb;
  if (!makeTensorMap2D(&pa, A, TM_BF16, K, M, lda, BK, 128, &g_err)) return static_cast<int>(cudaErrorInvalidValue);
  if (!b_mn ? !makeTensorMap2D(&pb, B, TM_BF16, K, N, ldb, BK, 128, &g_err) : !makeTensorMap2D(&pb, B, TM_BF16, N, K, ldb, 64, BK, &g_err))
    return static_cast<int>(cudaErrorInvalidValue);
  DgeluEpi epi{static_cast<__nv_bfloat16*>(D), static_cast<const __nv_bfloat16*>(pre), colsum, ldd, M, N};
  int pair_tiles = (M / 256) * (N / 256);
  int n_sm = deviceSmCount();
  if (sms > 0 && sms < n_sm) n_sm = sms;
  int grid = 2 * (pair_tiles < n_sm / 2 ? pair_tiles : n_sm / 2);
  return b_mn ? launchPair<false, true, DgeluEpi>(pa, pb, epi, K, grid, status, stream)
              : launchPair<false, false, DgeluEpi>(pa, pb, epi, K, grid, status, stream);
}

int gemmBf16Dual(const GemmProblem& p0, const GemmProblem& p1, int K, uint32_t flags, int sms, uint32_t* status, cudaStream_t stream) {
  const GemmProblem* ps[2] = {&p0, &p1};
  const bool a_mn = flags & GEMM_A_MN, b_mn = flags & GEMM_B_MN;
  if (K <= 0) return 0;
  DualMaps maps;
  DualEpi epi;
  for (int q = 0; q < 2; ++q) {
    const GemmProblem& p = *ps[q];
    if (p.M <= 0 || p.N <= 0 || (p.lda | p.ldb | p.ldd) % 8 ||
        (reinterpret_cast<uintptr_t>(p.A) | reinterpret_cast<uintptr_t>(p.B) | reinterpret_cast<uintptr_t>(p.D)) % 16) {
      g_err = "gemmBf16Dual: sizes must be positive, strides multiples of 8 elements, pointers 16-byte aligned";
      return static_cast<int>(cudaErrorInvalidValue);
    }
    if (!a_mn ? !makeTensorMap2D(&maps.a[q], p.A, TM_BF16, K, p.M, p.lda, BK, 128, &g_err) : !makeTensorMap2D(&maps.a[q], p.A, TM_BF16, p.M, K, p.lda, 64, BK, &g_err))
      return static_cast<int>(cudaErrorInvalidValue);
    if (!b_mn ? !makeTensorMap2D(&maps.b[q], p.B, TM_BF16, K, p.N, p.ldb, BK, 128, &g_err) : !makeTensorMap2D(&maps.b[q], p.B, TM_BF16, p.N, K, p.ldb, 64, BK, &g_err))
      return static_cast<int>(cudaErrorInvalidValue);
    epi.e[q] = StoreEpi{p.D, nullptr, nullptr, p.ldd, p.M, p.N, (flags & GEMM_OUT_F32) | (p.accumulate ? GEMM_ACCUMULATE : 0u)};
  }
  const long long tiles = static_cast<long long>((p0.M + 255) / 256) * ((p0.N + 255) / 256) + static_cast<long long>((p1.M + 255) / 256) * ((p1.N + 255) / 256);
  int n_sm = deviceSmCount();
  if (sms > 0 && sms < n_sm) n_sm = sms;
  const int grid = 2 * static_cast<int>(tiles < n_sm / 2 ? tiles : n_sm / 2);
  static bool attr_set[8] = {false, false, false, false, false, false, false, false};   // per kernel: the instantiations share one function type
  uint32_t* counter = tileCounterFor(stream);
  bool& attr = attr_set[(counter ? 4 : 0) | (a_mn ? 2 : 0) | (b_mn ? 1 : 0)];
  auto go = [&](auto kern) {
    if (int e = setPairSmem(kern, &attr)) return e;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(gemm2::NUM_THREADS_WIDE);
    cfg.dynamicSmemBytes = gemm2::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int Kc = K;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, maps, epi, Kc, status, counter));
  };
  if (counter) {
    if (a_mn) return b_mn ? go(gemm_bf16_pair_dual_kernel<true, true, true>) : go(gemm_bf16_pair_dual_kernel<true, false, true>);
    return b_mn ? go(gemm_bf16_pair_dual_kernel<false, true, true>) : go(gemm_bf16_pair_dual_kernel<false, false, true>);
  }
  if (a_mn) return b_mn ? go(gemm_bf16_pair_dual_kernel<true, true, false>) : go(gemm_bf16_pair_dual_kernel<true, false, false>);
  return b_mn ? go(gemm_bf16_pair_dual_kernel<false, true, false>) : go(gemm_bf16_pair_dual_kernel<false, false, false>);
}

}  // namespace pccl
