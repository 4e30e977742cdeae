// Block-scaled fp8 (e4m3) GEMM pipeline for sm_100a: D[M,N] = sum over 128-wide K blocks kb of
//   sa[m, kb] * sb[n / 128, kb] * (A8[m, kb-block] . B8[n, kb-block])
// i.e. activations carry one fp32 scale per row and 128 values of K (1 x 128), weights one per
// 128 x 128 block.  The tensor cores cannot apply fp32 scales, so the sum is built in two levels:
//
//   warp 0       TMA producer: 128 x 128 A and 256 x 128 B fp8 tiles (128-byte swizzle; one stage is one
//                K block) through a 4-stage ring; `Gate` as in the bf16 pipeline
//   warp 1       MMA issuer: four tcgen05.mma kind::f8f6f4 128x256x32 per stage into a FRESH TMEM
//                accumulator; the two 256-column accumulators alternate per K block
//   warps 2..9   promotion + epilogue: every K block, tcgen05.ld the block's partial products and
//                fold them, times sa*sb, into 128 fp32 registers per thread (warp w and w+4 share
//                a 32-lane quarter of TMEM and split the 256 columns; packed fma.rn.f32x2); after
//                the last block the registers go to `Epi` as 32-column strips, exactly like the
//                bf16 pipeline's
//
// so the same epilogue adapters (plain store, reduce-scatter) serve both precisions.
// Cost model: the promotion reads 128 KiB of TMEM per K block through the load/store data path
// (128 B per clock and SM, ~1024 clocks) while the four MMAs of the block need ~512, so this
// exact-fp32-scale scheme tops out near half of the fp8 tensor peak -- about the bf16 peak -- and
// its gain over bf16 is the halved operand traffic (HBM, L2 and NVLink).
// All waits are bounded; on a time-out the CTA flags the error, drains its copies, frees TMEM
// and returns.  No TMA load uses cluster multicast.
//
// The reference names fp8 in its vector types only (include/plugins/cuda_executor/utils/
// vector_datatype.h:66-80) and has no GEMM.
#pragma once
#include <cuda_bf16.h>

#include "../base/instr.h"
#include "gemm_pipeline.cuh"
#include "prims.cuh"
#include "tc05.cuh"

namespace pccl {
namespace gemm8 {

using gemm::TileCoord;

constexpr int BM = 128, BN = 256, BK = 128, UMMA_K = 32;
constexpr int MAX_STAGES = 4;
constexpr int A_BYTES = BM * BK;            // 16 KiB
constexpr int B_BYTES = BN * BK;            // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;              // two 128 x 256 fp32 accumulators, alternating per K block
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;   // 320
constexpr int smem_bytes(int stages) { return stages * STAGE_BYTES + 1024 + 256; }
constexpr int SMEM_BYTES = smem_bytes(MAX_STAGES);   // epilogues that stage through shared memory start at stages * STAGE_BYTES + 256
constexpr int CW = BN / 2;                  // columns per epilogue warp

struct Barriers {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort;
};

// Scales: sa is fp32 [M, ld_sa] (ld_sa >= ceil(K/128)), sb is fp32 [ceil(N/128), ld_sb].
struct Scales {
  const float* sa;
  const float* sb;
  int ld_sa, ld_sb;
  int M, N;      // bounds for clamping the scale rows of edge tiles
};

// Two fp32 multiply-adds in one instruction (sm_100 packed fp32): acc{0,1} += r{0,1} * s.
__device__ __forceinline__ void ffma2(float& acc0, float& acc1, uint32_t r0, uint32_t r1, float s) {
  asm("{\n\t.reg .b64 a, b, c;\n\t"
      "mov.b64 a, {%2, %3};\n\t"
      "mov.b64 b, {%4, %4};\n\t"
      "mov.b64 c, {%0, %1};\n\t"
      "fma.rn.f32x2 c, a, b, c;\n\t"
      "mov.b64 {%0, %1}, c;\n\t}"
      : "+f"(acc0), "+f"(acc1)
      : "r"(r0), "r"(r1), "f"(s));
}

// STAGES (<= 4) operand stages of 48 KiB; an epilogue that needs shared memory of its own runs with three.
template <int STAGES = MAX_STAGES, class Sched, class Gate, class Epi>
__device__ __forceinline__ void run(const CUtensorMap* tmA, const CUtensorMap* tmB, int K, const Scales& sc, const Sched& sched,
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
      tc::mbar_init(&bar->tmem_empty[a], EPI_WARPS);
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
  epi.attach_smem(smem + STAGES * STAGE_BYTES + 256);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (tc::elect_one()) {
      int stage = 0;
      uint32_t phase = 0, armed = 0, armed_par = 0;
      bool ok = true;
      TileCoord t;
      for (int it = 0; ok && sched.get(it, &t); ++it) {
        if (!gate.wait(t, abort)) { ok = false; break; }
        const int row0 = epi.a_row0(t), col0 = epi.b_row0(t);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&bar->empty[stage], phase ^ 1, abort)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          tc::mbar_arrive_expect_tx(&bar->full[stage], STAGE_BYTES);
          armed |= 1u << stage;
          armed_par = (armed_par & ~(1u << stage)) | (phase << stage);
          tc::tma_load_2d(sa, tmA, &bar->full[stage], kb * BK, row0);
          tc::tma_load_2d(sa + A_BYTES, tmB, &bar->full[stage], kb * BK, col0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        if (atomicExch(const_cast<uint32_t*>(&bar->abort), 1u) == 0) dev::report(status, ST_TIMEOUT, blockIdx.x, 0, 0);
        for (int s = 0; s < STAGES; ++s)
          if (armed & (1u << s))
            for (uint32_t i = 0; i < (1u << 16) && !tc::mbar_try_wait(&bar->full[s], (armed_par >> s) & 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (tc::elect_one()) {
      constexpr uint32_t idesc = tc::make_idesc(0, 0, false, false, BM, BN);   // e4m3 x e4m3 -> f32
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      TileCoord t;
      for (int it = 0; ok && sched.get(it, &t); ++it) {
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&bar->tmem_empty[acc], acc_phase ^ 1, abort)) { ok = false; break; }
          if (!tc::mbar_wait(&bar->full[stage], phase, abort)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t d_tmem = tmem + acc * BN;
          const uint32_t sa = tc::smem_u32(smem + stage * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t da = tc::smem_desc_sw128(sa + k * UMMA_K, 16, 1024);
            uint64_t db = tc::smem_desc_sw128(sb + k * UMMA_K, 16, 1024);
            tc::mma_f8(d_tmem, da, db, idesc, k != 0);
          }
          tc::mma_commit(&bar->empty[stage]);
          tc::mma_commit(&bar->tmem_full[acc]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
      if (!ok && atomicExch(const_cast<uint32_t*>(&bar->abort), 1u) == 0) dev::report(status, ST_TIMEOUT, blockIdx.x, 1, 0);
      // every MMA issued above must have retired before TMEM is freed
      tc::mma_commit(&bar->drain);
      for (uint32_t i = 0; i < (1u << 20) && !tc::mbar_try_wait(&bar->drain, 0); ++i) {}
    }
  } else {
    // ------------------------------------------------------------------ promotion + epilogue (8 warps)
    const int quarter = warp & 3;             // TMEM lanes [32*quarter, +32) are readable by this warp
    const int half = (warp - 2) >> 2;         // columns [CW*half, +CW) of the tile
    const int row_in_tile = quarter * 32 + lane;
    const int sb_rows = (sc.N + 127) / 128;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    TileCoord t;
    for (int it = 0; ok && sched.get(it, &t); ++it) {
      float accr[CW];
#pragma unroll
      for (int i = 0; i < CW; ++i) accr[i] = 0.f;
      // A's scales arrive with its rows: a gated tile's scales may only be read once the gate has opened
      {
        int open = 1;
        if (lane == 0) open = gate.wait(t, abort) ? 1 : 0;
        if (!__shfl_sync(0xffffffffu, open, 0)) { ok = false; break; }
      }
      const int grow = min(epi.a_row0(t) + row_in_tile, sc.M - 1);
      const int gblk = min((epi.b_row0(t) + half * CW) >> 7, sb_rows - 1);
      const float* pa = sc.sa + static_cast<long long>(grow) * sc.ld_sa;
      const float* pb = sc.sb + static_cast<long long>(gblk) * sc.ld_sb;
      // raw scales travel two K blocks ahead of their use, so that no load latency is exposed
      // (A's scales may have been written by a peer during this launch: read them past L1)
      float a0 = __ldcg(pa), b0 = __ldg(pb);
      float a1 = num_kb > 1 ? __ldcg(pa + 1) : 0.f, b1 = num_kb > 1 ? __ldg(pb + 1) : 0.f;
      for (int kb = 0; kb < num_kb; ++kb) {
        const float s = a0 * b0;
        a0 = a1;
        b0 = b1;
        if (kb + 2 < num_kb) {
          a1 = __ldcg(pa + kb + 2);
          b1 = __ldg(pb + kb + 2);
        }
        if (!tc::mbar_wait(&bar->tmem_full[acc], acc_phase, abort)) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + half * CW;
#pragma unroll
        for (int c = 0; c < CW / 32; c += 2) {
          uint32_t r0[32], r1[32];
          tc::tmem_ld_32x32(taddr + c * 32, r0);
          tc::tmem_ld_32x32(taddr + (c + 1) * 32, r1);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 2) ffma2(accr[c * 32 + j], accr[c * 32 + j + 1], r0[j], r0[j + 1], s);
#pragma unroll
          for (int j = 0; j < 32; j += 2) ffma2(accr[(c + 1) * 32 + j], accr[(c + 1) * 32 + j + 1], r1[j], r1[j + 1], s);
        }
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&bar->tmem_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) break;
      epi.tile_begin(t);
      if constexpr (Epi::kRow128) {
        epi.row128(t, row_in_tile, half * CW, accr);      // the thread's 128 values are one 1 x 128 block of the output
      } else {
#pragma unroll
        for (int c = 0; c < CW / 32; ++c) {
          uint32_t r[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(accr[c * 32 + j]);
          epi.strip(t, row_in_tile, half * CW + c * 32, r);
        }
      }
      epi.tile_done(t, abort);
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

}  // namespace gemm8
}  // namespace pccl
