// Warp-specialised, persistent tcgen05 GEMM pipeline for sm_100a, shared by the plain GEMM and by
// the kernels that fuse a collective into it (all-gather -> GEMM, GEMM -> reduce-scatter, grouped
// expert GEMM).  D[M,N] = A[M,K] * B[N,K]^T with bf16 operands and fp32 accumulation in TMEM.
//
//   warp 0      TMA producer: one thread streams 128x64 A tiles and 256x64 B tiles (128-byte
//               swizzle) through a 4-stage shared-memory ring; `Gate` lets a fused kernel hold a
//               tile back until its rows have arrived from a peer
//   warp 1      MMA issuer: one thread issues tcgen05.mma 128x256x16 (cta_group::1), four per
//               stage, and commits the stage back to the producer; owns the TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld the 128x256 fp32 accumulator (each warp its 32-lane quarter),
//               hand 32-column strips to `Epi`; two accumulators (2 x 256 TMEM columns) let the
//               epilogue of tile i overlap the main loop of tile i+1
//
// Operands may be K-major (row-major [rows, K]) or MN-major (the transposed view of a row-major
// [K, rows] tensor); the second form feeds weight-gradient GEMMs without a transpose pass.
// No TMA load uses cluster multicast.  All waits are bounded; on a time-out the CTA flags the
// error, drains its copies, frees TMEM and returns.
#pragma once
#include <cuda_bf16.h>

#include "../base/instr.h"
#include "prims.cuh"
#include "tc05.cuh"

namespace pccl {
namespace gemm {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_BYTES = BN * BK * 2;        // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;              // two 128x256 fp32 accumulators
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int EPI_SMEM_OFFSET = STAGES * STAGE_BYTES + 256;   // epilogues that stage through shared memory start here

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort;
};

struct TileCoord {
  int m, n;       // tile indices
  int extra;      // scheduler-defined (e.g. expert id, source rank)
};

// Default scheduler: persistent CTAs walk tiles in groups of GROUP_M row-tiles so that the tiles
// in flight at one time share A and B panels in L2.
struct GroupedSched {
  int tiles_m, tiles_n, first, stride;
  static constexpr int GROUP_M = 16;
  __device__ __forceinline__ bool get(int it, TileCoord* t) const {
    long long idx = first + static_cast<long long>(it) * stride;
    if (idx >= static_cast<long long>(tiles_m) * tiles_n) return false;
    int per_group = GROUP_M * tiles_n;
    int g = static_cast<int>(idx / per_group), r = static_cast<int>(idx % per_group);
    int gm = min(GROUP_M, tiles_m - g * GROUP_M);
    t->m = g * GROUP_M + r % gm;
    t->n = r / gm;
    t->extra = 0;
    return true;
  }
};

struct NoGate {
  __device__ __forceinline__ bool wait(const TileCoord&, const volatile uint32_t*) const { return true; }
};

// The pipeline.  `tmA` / `tmB` are TMA descriptors:
//   K-major operand : dims {K, rows}, box {64, 128 (A) | 256 (B)}
//   MN-major operand: dims {rows, K}, box {64, 64}; a tile takes 2 (A) or 4 (B) boxes
// `row0_of(t)` / `col0_of(t)` map a tile to operand coordinates (lets grouped GEMMs offset rows).
template <bool A_MN, bool B_MN, class Sched, class Gate, class Epi>
__device__ __forceinline__ void run(const CUtensorMap* tmA, const CUtensorMap* tmB, int K, const Sched& sched,
                                    const Gate& gate, Epi& epi, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Barriers* bar = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;
  volatile uint32_t* abort = &bar->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&bar->full[s], 1);
      tc::mbar_init(&bar->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc::mbar_init(&bar->tmem_full[a], 1);
      tc::mbar_init(&bar->tmem_empty[a], 4);
    }
    tc::mbar_init(&bar->drain, 1);
    bar->abort = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(tmA);
    tc::tma_prefetch_desc(tmB);
  }
  if (warp == 1) {
    tc::tmem_alloc(&bar->tmem_base, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  epi.attach_smem(smem + EPI_SMEM_OFFSET);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (tc::elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0;    // bit s set: full[s] was armed with parity bit (armed_par >> s)
      uint32_t armed_par = 0;
      bool ok = true;
      TileCoord t;
      for (int it = 0; ok && sched.get(it, &t); ++it) {
        if (!gate.wait(t, abort)) { ok = false; break; }
        const int row0 = epi.a_row0(t), col0 = epi.b_row0(t);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&bar->empty[stage], phase ^ 1, abort)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          tc::mbar_arrive_expect_tx(&bar->full[stage], STAGE_BYTES);
          armed |= 1u << stage;
          armed_par = (armed_par & ~(1u << stage)) | (phase << stage);
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tc::tma_load_2d(sa, tmA, &bar->full[stage], k0, row0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tc::tma_load_2d(sa + j * (64 * BK * 2), tmA, &bar->full[stage], row0 + j * 64, k0);
          }
          if constexpr (!B_MN) {
            tc::tma_load_2d(sb, tmB, &bar->full[stage], k0, col0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tc::tma_load_2d(sb + j * (64 * BK * 2), tmB, &bar->full[stage], col0 + j * 64, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        if (atomicExch(const_cast<uint32_t*>(&bar->abort), 1u) == 0) dev::report(status, ST_TIMEOUT, blockIdx.x, 0, 0);
        // let copies already in flight land before the CTA's shared memory goes away
        for (int s = 0; s < STAGES; ++s)
          if (armed & (1u << s))
            for (uint32_t i = 0; i < (1u << 16) && !tc::mbar_try_wait(&bar->full[s], (armed_par >> s) & 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (tc::elect_one()) {
      constexpr uint32_t idesc = tc::make_idesc(1, 1, A_MN, B_MN, BM, BN);
      constexpr uint32_t A_LBO = A_MN ? 64 * BK * 2 : 16, A_SBO = 1024;
      constexpr uint32_t B_LBO = B_MN ? 64 * BK * 2 : 16, B_SBO = 1024;
      constexpr uint32_t A_KSTEP = A_MN ? (UMMA_K / 8) * 1024 : UMMA_K * 2;   // bytes per UMMA_K
      constexpr uint32_t B_KSTEP = B_MN ? (UMMA_K / 8) * 1024 : UMMA_K * 2;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      TileCoord t;
      for (int it = 0; ok && sched.get(it, &t); ++it) {
        if (!tc::mbar_wait(&bar->tmem_empty[acc], acc_phase ^ 1, abort)) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&bar->full[stage], phase, abort)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t sa = tc::smem_u32(smem + stage * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t da = tc::smem_desc_sw128(sa + k * A_KSTEP, A_LBO, A_SBO);
            uint64_t db = tc::smem_desc_sw128(sb + k * B_KSTEP, B_LBO, B_SBO);
            tc::mma_f16(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          tc::mma_commit(&bar->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc::mma_commit(&bar->tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok && atomicExch(const_cast<uint32_t*>(&bar->abort), 1u) == 0) dev::report(status, ST_TIMEOUT, blockIdx.x, 1, 0);
      // every MMA issued above must have retired before TMEM is freed
      tc::mma_commit(&bar->drain);
      for (uint32_t i = 0; i < (1u << 20) && !tc::mbar_try_wait(&bar->drain, 0); ++i) {}
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int quarter = warp & 3;          // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    TileCoord t;
    for (int it = 0; ok && sched.get(it, &t); ++it) {
      if (!tc::mbar_wait(&bar->tmem_full[acc], acc_phase, abort)) { ok = false; break; }
      tc::tc_fence_after();
      const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      epi.tile_begin(t);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(taddr + c * 32, r);
        tc::tmem_ld_wait();
        epi.strip(t, quarter * 32 + lane, c * 32, r);
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&bar->tmem_empty[acc]);
      epi.tile_done(t, abort);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (!ok && lane == 0 && atomicExch(const_cast<uint32_t*>(&bar->abort), 1u) == 0) dev::report(status, ST_TIMEOUT, blockIdx.x, 2, 0);
  }

  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace pccl
