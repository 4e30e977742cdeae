// CTA-pair variant of the tcgen05 GEMM pipeline: two CTAs of a cluster (cta_group::2) compute one
// 256 x 256 tile.  Each CTA loads its own 128 rows of A and its own 128 rows of B (half of N) per
// k-block -- 32 KiB instead of 48 KiB per 128 x 256 of output, which takes a third off the L2 -> SM
// traffic that bounds the single-CTA kernel -- into a 6-stage ring; the leader CTA issues
// tcgen05.mma.cta_group::2 (M = 256) that reads both CTAs' shared memory and writes both CTAs'
// tensor memory; each CTA runs the epilogue of its own 128 accumulator rows.
//
// No load uses cluster multicast: the operands are not shared between the CTAs, only the completion
// of both CTAs' loads is counted on the leader's barrier.  tcgen05.commit multicasts the "stage free"
// and "accumulator ready" arrivals to both CTAs.  Same hooks (Sched / Gate / Epi) and the same bounded
// waits as gemm_pipeline.cuh; every thread of both CTAs reaches the closing cluster barrier.
#pragma once
#include <cstdlib>
#include <type_traits>
#include <utility>

#include "gemm_pipeline.cuh"

namespace pccl {
namespace gemm2 {

using gemm::TileCoord;
constexpr int BM = 128;            // rows per CTA; the pair's tile is 2*BM x BN
constexpr int PAIR_M = 256, BN = 256, HALF_N = 128, BK = 64, UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = HALF_N * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;   // 32 KiB
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 192;            // producer warp, MMA warp, four epilogue warps
constexpr int NUM_THREADS_WIDE = 320;       // ... or eight epilogue warps (run<..., EPI_WARPS = 8>): two per TMEM lane quarter, each
                                            // taking half of a tile's strips, for epilogues that are bound by their own latency
constexpr int BAR_BYTES = 512;     // barriers and the tile-index ring, between the operand ring and an epilogue's staging area
constexpr int PATCH_BYTES = 8 * 32 * 80;   // the (up to eight) epilogue warps' coalescing patches (gemm_epilogue.cuh), behind the barriers
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + BAR_BYTES + PATCH_BYTES;
constexpr int EPI_SMEM_OFFSET = STAGES * STAGE_BYTES + BAR_BYTES;

constexpr int SCHED_SLOTS = 4;     // tile indices in flight between the roles (dynamic scheduling)
struct Barriers {
  uint64_t full[STAGES];        // used in the leader: both CTAs' loads of the stage have landed
  uint64_t empty[STAGES];       // per CTA: the MMAs that read this stage have retired
  uint64_t tmem_full[2];        // per CTA: accumulator ready
  uint64_t tmem_empty[2];       // used in the leader: both CTAs' epilogues have drained the accumulator
  uint64_t drain;
  uint64_t sched_full[SCHED_SLOTS];    // per CTA: the slot holds the tile index of iteration it (it % SCHED_SLOTS)
  uint64_t sched_empty[SCHED_SLOTS];   // used in the leader: every role of both CTAs has read the slot
  uint64_t inbox_full[SCHED_SLOTS];    // used in the peer: the leader has stored the index into `inbox`
  int32_t sched_tile[SCHED_SLOTS];     // per CTA: tile index, or -1 for "no more tiles"; written by this CTA's producer
  int32_t inbox[SCHED_SLOTS];          // used in the peer: written by the leader's producer, read by the peer's producer
  uint32_t tmem_base;
  uint32_t abort;
};
static_assert(sizeof(Barriers) <= BAR_BYTES, "barriers overrun their area");

// An epilogue may declare `static constexpr bool kVarN = true` and `int tile_n(const TileCoord&)`: the tile then spans only
// that many of the BN accumulator columns (a multiple of 16).  The MMA is issued with that N -- each CTA contributes the
// first tile_n / 2 rows of its B box -- and the epilogue is handed only the strips below it, so a ragged last tile costs
// tensor time in proportion to its width.  `int b_box(const TileCoord&)` then picks one of several B descriptors (`tmB` is an
// array) whose boxes hold 128 >> b_box rows, so a narrow tile does not fetch rows it will not multiply.
// An epilogue with `attach_patch(uint8_t*)` is handed PATCH_BYTES of shared memory behind the barrier area (only where the
// kernel was launched with SMEM_BYTES of this header and the epilogue's own staging, if any, does not live there).
template <class E, class = void> struct HasPatch : std::false_type {};
template <class E> struct HasPatch<E, std::void_t<decltype(std::declval<E&>().attach_patch(nullptr))>> : std::true_type {};
template <class E, class = void> struct HasVarN : std::false_type {};
template <class E> struct HasVarN<E, std::void_t<decltype(E::kVarN)>> : std::true_type {};

// `sched` enumerates pair tiles: t.m indexes 256-row blocks.  Epi sees per-CTA coordinates through
// a_row0 / b_row0 (which must add cta_rank * 128) and strip(t, row_in_cta_tile, col, r).
// NSTAGES (<= STAGES) shortens the operand ring; an epilogue that needs a large staging area of its own (the
// reduce-scatter epilogue stages whole 512-byte rows) gives up one stage for it.
// NPROB > 1: `tmA` / `tmB` are arrays of that many descriptors and a tile's `extra` field says which pair it loads from --
// several GEMMs with the same K walked as one tile list (fewer idle CTAs in the last wave than one launch per GEMM).
//
// DYN: tiles are handed out at run time instead of round-robin.  `sched` then has `counter` (a zeroed word in global memory
// that the launch leaves zeroed), `total` (tiles) and `at(index, &tile)`.  The leader's producer thread draws the next
// index with an atomic add and publishes it through a four-slot ring in both CTAs' shared memory; the other roles (the
// peer's producer, the MMA thread, the eight epilogue warps) read it from there, so all of them walk the same tile list in
// the same order.  A CTA pair that starts late -- its SMs were still held by another kernel, a collective on a second
// stream for instance -- then simply takes fewer tiles, where the round-robin list would make the whole GEMM wait for it.
template <bool A_MN, bool B_MN, class Sched, class Gate, class Epi, int NSTAGES = STAGES, int NPROB = 1, bool DYN = false, int EPI_WARPS = 4>
__device__ __forceinline__ void run(const CUtensorMap* tmA, const CUtensorMap* tmB, int K, const Sched& sched,
                                    const Gate& gate, Epi& epi, uint32_t* status) {
  static_assert(NSTAGES >= 2 && NSTAGES <= STAGES, "ring length");
  static_assert(EPI_WARPS == 4 || EPI_WARPS == 8, "epilogue warps per CTA");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Barriers* bar = reinterpret_cast<Barriers*>(smem + NSTAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = tc::cluster_ctarank();
  const bool leader = cta == 0;
  const int num_kb = (K + BK - 1) / BK;
  volatile uint32_t* abort = &bar->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGES; ++s) {
      tc::mbar_init(&bar->full[s], 1);
      tc::mbar_init(&bar->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc::mbar_init(&bar->tmem_full[a], 1);
      tc::mbar_init(&bar->tmem_empty[a], 2 * EPI_WARPS);      // the epilogue warps of both CTAs of the pair
    }
    tc::mbar_init(&bar->drain, 1);
    for (int q = 0; q < SCHED_SLOTS; ++q) {
      tc::mbar_init(&bar->sched_full[q], 1);
      tc::mbar_init(&bar->sched_empty[q], 2 + 2 * EPI_WARPS);    // MMA thread + peer's producer + the epilogue warps of both CTAs
      tc::mbar_init(&bar->inbox_full[q], 1);
    }
    bar->abort = 0;
    tc::fence_barrier_init();
    for (int q = 0; q < NPROB; ++q) {
      tc::tma_prefetch_desc(tmA + q);
      tc::tma_prefetch_desc(tmB + q);
    }
  }
  __syncthreads();
  tc::cluster_sync();                 // the peer's barriers are initialised before anything signals them
  if (warp == 1) {
    tc::tmem_alloc_pair(&bar->tmem_base, TMEM_COLS);
    tc::tmem_relinquish_pair();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  epi.attach_smem(smem + NSTAGES * STAGE_BYTES + BAR_BYTES);
  if constexpr (HasPatch<Epi>::value && NSTAGES == STAGES) epi.attach_patch(smem + NSTAGES * STAGE_BYTES + BAR_BYTES);

  // Tile of iteration `it` for a role that READS the ring (every role but the leader's producer).  `warp_wide`: all lanes
  // of a warp call this together and lane 0 releases the slot.  Returns 1 (tile), 0 (end of the list) or -1 (gave up).
  auto ring_tile = [&](int it, TileCoord* t, bool warp_wide) -> int {
    if constexpr (DYN) {
      const int q = it & (SCHED_SLOTS - 1);
      if (!tc::mbar_wait(&bar->sched_full[q], (it / SCHED_SLOTS) & 1, abort)) return -1;     // published inside this CTA
      const int32_t v = *reinterpret_cast<volatile int32_t*>(&bar->sched_tile[q]);
      if (warp_wide) __syncwarp();
      // the slot goes back to the leader; the zero that is added to the address is computed from the value read (in a
      // form the compiler cannot fold), so the arrive cannot be issued before that read has returned
      if (!warp_wide || lane == 0) {
        uint32_t zero;
        asm volatile("and.b32 %0, %1, 0;" : "=r"(zero) : "r"(v));
        tc::mbar_arrive_cluster_relaxed(tc::mapa(tc::smem_u32(&bar->sched_empty[q]) + zero, 0));
      }
      if (v < 0) return 0;
      return sched.at(v, t) ? 1 : 0;
    } else {
      return sched.get(it, t) ? 1 : 0;
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (tc::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TileCoord t;
      // dynamic scheduling, leader: the index for the next iteration is drawn one iteration ahead, so the atomic's latency
      // hides behind this tile's loads.  Every producer draws exactly one index past the end; whoever draws the very last
      // one of the launch (total + pairs - 1) puts the counter back to zero for the next launch on this stream.
      uint32_t drawn = 0;
      const uint32_t n_pairs = gridDim.x >> 1;
      if constexpr (DYN) {
        if (leader) drawn = atomicAdd(sched.counter, 1u);
      }
      for (int it = 0; ok; ++it) {
        if constexpr (DYN) {
          if (leader) {
            const int q = it & (SCHED_SLOTS - 1);
            if (!tc::mbar_wait(&bar->sched_empty[q], ((it / SCHED_SLOTS) & 1) ^ 1, abort)) { ok = false; break; }   // no data comes with it
            const uint32_t cur = drawn;        // drawn one iteration ago: nothing has waited for the atomic until here
            if (cur == sched.total + n_pairs - 1) atomicExch(sched.counter, 0u);
            const int32_t v = cur < sched.total ? static_cast<int32_t>(cur) : -1;
            bar->sched_tile[q] = v;
            tc::mbar_arrive(&bar->sched_full[q]);                                          // this CTA's readers
            tc::st_shared_cluster_u32(tc::mapa(tc::smem_u32(&bar->inbox[q]), 1), static_cast<uint32_t>(v));
            tc::mbar_arrive_cluster(tc::mapa(tc::smem_u32(&bar->inbox_full[q]), 1));     // the peer's producer
            if (v < 0 || !sched.at(v, &t)) break;
            drawn = atomicAdd(sched.counter, 1u);
          } else {
            // the peer's producer: index out of the inbox (cluster-scope acquire), into this CTA's slot for its epilogue warps
            const int q = it & (SCHED_SLOTS - 1);
            if (!tc::mbar_wait_cluster(&bar->inbox_full[q], (it / SCHED_SLOTS) & 1, abort)) { ok = false; break; }
            const int32_t v = *reinterpret_cast<volatile int32_t*>(&bar->inbox[q]);
            bar->sched_tile[q] = v;
            tc::mbar_arrive(&bar->sched_full[q]);
            {                                                                                 // the inbox slot may be written again
              uint32_t zero;
              asm volatile("and.b32 %0, %1, 0;" : "=r"(zero) : "r"(v));
              tc::mbar_arrive_cluster_relaxed(tc::mapa(tc::smem_u32(&bar->sched_empty[q]) + zero, 0));
            }
            if (v < 0 || !sched.at(v, &t)) break;
          }
        } else {
          if (!sched.get(it, &t)) break;
        }
        if (!gate.wait(t, abort)) { ok = false; break; }
        const int row0 = epi.a_row0(t), col0 = epi.b_row0(t);        // already offset by this CTA's half
        const CUtensorMap* const tmA_t = NPROB > 1 ? tmA + t.extra : tmA;
        const CUtensorMap* tmB_t = NPROB > 1 ? tmB + t.extra : tmB;
        uint32_t stage_tx = 2 * STAGE_BYTES;
        if constexpr (HasVarN<Epi>::value) {
          const int sel = epi.b_box(t);
          tmB_t = tmB + sel;
          stage_tx = 2 * (A_BYTES + (B_BYTES >> sel));
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&bar->empty[stage], phase ^ 1, abort)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t full_leader = tc::mapa(tc::smem_u32(&bar->full[stage]), 0);
          if (leader) tc::mbar_arrive_expect_tx(&bar->full[stage], stage_tx);   // both CTAs' bytes
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tc::tma_load_2d_pair(sa, tmA_t, full_leader, k0, row0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tc::tma_load_2d_pair(sa + j * (64 * BK * 2), tmA_t, full_leader, row0 + j * 64, k0);
          }
          if constexpr (!B_MN) {
            tc::tma_load_2d_pair(sb, tmB_t, full_leader, k0, col0);
          } else {
#pragma unroll
            for (int j = 0; j < HALF_N / 64; ++j) tc::tma_load_2d_pair(sb + j * (64 * BK * 2), tmB_t, full_leader, col0 + j * 64, k0);
          }
          if (++stage == NSTAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok && atomicExch(const_cast<uint32_t*>(&bar->abort), 1u) == 0) dev::report(status, ST_TIMEOUT, blockIdx.x, 0, 0);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && tc::elect_one()) {
      constexpr uint32_t idesc = tc::make_idesc(1, 1, A_MN, B_MN, PAIR_M, BN);
      constexpr uint32_t A_LBO = A_MN ? 64 * BK * 2 : 16, B_LBO = B_MN ? 64 * BK * 2 : 16, SBO = 1024;
      constexpr uint32_t A_KSTEP = A_MN ? (UMMA_K / 8) * 1024 : UMMA_K * 2;
      constexpr uint32_t B_KSTEP = B_MN ? (UMMA_K / 8) * 1024 : UMMA_K * 2;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      TileCoord t;
      for (int it = 0; ok; ++it) {
        const int got = ring_tile(it, &t, false);
        if (got < 0) ok = false;
        if (got <= 0) break;
        if (!tc::mbar_wait(&bar->tmem_empty[acc], acc_phase ^ 1, abort)) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem + acc * BN;
        uint32_t idesc_t = idesc;
        if constexpr (HasVarN<Epi>::value) idesc_t = tc::make_idesc(1, 1, A_MN, B_MN, PAIR_M, static_cast<uint32_t>(epi.tile_n(t)));
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&bar->full[stage], phase, abort)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t sa = tc::smem_u32(smem + stage * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t da = tc::smem_desc_sw128(sa + k * A_KSTEP, A_LBO, SBO);
            uint64_t db = tc::smem_desc_sw128(sb + k * B_KSTEP, B_LBO, SBO);
            tc::mma_f16_pair(d_tmem, da, db, idesc_t, (kb | k) != 0);
          }
          tc::mma_commit_pair(&bar->empty[stage], 3);       // frees the stage in both CTAs
          if (++stage == NSTAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc::mma_commit_pair(&bar->tmem_full[acc], 3);       // accumulator ready in both CTAs
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok && atomicExch(const_cast<uint32_t*>(&bar->abort), 1u) == 0) dev::report(status, ST_TIMEOUT, blockIdx.x, 1, 0);
      tc::mma_commit_pair(&bar->drain, 1);
      for (uint32_t i = 0; i < (1u << 20) && !tc::mbar_try_wait(&bar->drain, 0); ++i) {}
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps, both CTAs)
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    TileCoord t;
    for (int it = 0; ok; ++it) {
      const int got = ring_tile(it, &t, true);
      if (got < 0) ok = false;
      if (got <= 0) break;
      if (!tc::mbar_wait(&bar->tmem_full[acc], acc_phase, abort)) { ok = false; break; }
      tc::tc_fence_after();
      const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      epi.tile_begin(t);
      int n_strips = BN / 32;
      if constexpr (HasVarN<Epi>::value) n_strips = (epi.tile_n(t) + 31) / 32;
      // with eight epilogue warps the two warps of a lane quarter take the lower and the upper half of the strips
      constexpr int kSplit = EPI_WARPS / 4;
      const int per = (n_strips + kSplit - 1) / kSplit;
      const int c_begin = ((warp - 2) >> 2) * per, c_end = c_begin + per < n_strips ? c_begin + per : n_strips;
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(taddr + c * 32, r);
        tc::tmem_ld_wait();
        epi.strip(t, quarter * 32 + lane, c * 32, r);
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive_cluster(tc::mapa(tc::smem_u32(&bar->tmem_empty[acc]), 0));   // on the leader's barrier
      epi.tile_done(t, abort);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (!ok && lane == 0 && atomicExch(const_cast<uint32_t*>(&bar->abort), 1u) == 0) dev::report(status, ST_TIMEOUT, blockIdx.x, 2, 0);
  }

  tc::tc_fence_before();
  __syncthreads();
  tc::cluster_sync();                 // the leader's MMAs no longer read the peer's shared memory
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc_pair(tmem, TMEM_COLS);
  }
}

// Adapters that let epilogues and gates written for 128-row tiles serve a CTA pair: the CTA with
// cluster rank c handles 128-row tile 2*m + c of pair tile m and loads rows [c*128, c*128+128) of the
// pair's 256 B rows.
__device__ __forceinline__ TileCoord half_tile(const TileCoord& t, int cta) { return TileCoord{t.m * 2 + cta, t.n, t.extra}; }

template <class Epi>
struct PairEpi {
  Epi& e;
  int cta;
  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return e.a_row0(half_tile(t, cta)); }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return e.b_row0(half_tile(t, cta)) + cta * HALF_N; }
  __device__ __forceinline__ void attach_smem(uint8_t* p) { e.attach_smem(p); }
  __device__ __forceinline__ void attach_patch(uint8_t* p) {
    if constexpr (HasPatch<Epi>::value) e.attach_patch(p);
  }
  __device__ __forceinline__ void tile_begin(const TileCoord& t) { e.tile_begin(half_tile(t, cta)); }
  __device__ __forceinline__ void tile_done(const TileCoord& t, const volatile uint32_t* abort) { e.tile_done(half_tile(t, cta), abort); }
  __device__ __forceinline__ void strip(const TileCoord& t, int row, int col, uint32_t* r) { e.strip(half_tile(t, cta), row, col, r); }
};

template <class Gate>
struct PairGate {
  const Gate& g;
  int cta;
  __device__ __forceinline__ bool wait(const TileCoord& t, const volatile uint32_t* abort) const { return g.wait(half_tile(t, cta), abort); }
};

// Launch helper: cluster of two CTAs along x, optionally cooperative (kernels whose CTAs wait on one another).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pairs(void (*kernel)(KArgs...), dim3 grid, int threads, size_t smem, cudaStream_t stream, bool cooperative,
                                Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeCooperative;
  at[1].val.cooperative = 1;
  cfg.attrs = at;
  // PCCL_NO_COOP=1 drops the co-residency check of the cooperative launch (profilers that replay a kernel
  // cannot replay cooperative launches); the kernels' waits stay bounded either way.
  static const bool no_coop = std::getenv("PCCL_NO_COOP") != nullptr && std::getenv("PCCL_NO_COOP")[0] == '1';
  cfg.numAttrs = (cooperative && !no_coop) ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace gemm2
}  // namespace pccl
