// fp8 (e4m3) GEMM with HARDWARE block scaling for sm_100a: tcgen05.mma kind::mxf8f6f4.block_scale.
//   D[m, n] = sum over 128-wide K blocks kb of 2^(sa[m, kb] - 127) * 2^(sb[n / 128, kb] - 127) * (A8[m, kb] . B8[n, kb])
// Scales are UE8M0 bytes (powers of two): activations one per row and 128 values of K, weights one per
// 128 x 128 block.  The tensor core applies them, so the accumulator stays in TMEM for the whole K loop
// and nothing is promoted in registers (the exact-fp32-scale kernel of gemm_fp8_pipeline.cuh pays twice
// the MMA time for that).
//
//   warp 0      TMA producer: 128 x 128 A and 224 x 128 B tiles (128-byte swizzle), 5 stages; `Gate` as in
//               the other pipelines
//   warp 1      MMA issuer: per stage four MMAs 128 x 224 x 32; every fourth stage it first copies the
//               scale images of the next 512 values of K from shared memory into TMEM (tcgen05.cp
//               32x128b.warpx4: 32 rows of 16 bytes, replicated to the four lane quarters)
//   warp 2      scale builder: writes those images.  The instruction wants, for tile row (or column)
//               r = 32 g + l, one 32-bit word at TMEM lane l, column g, whose byte j scales the j-th
//               K block of the group; the scale-id field of the instruction descriptor selects j.
//               The image in shared memory is therefore [l][g] words, 16 bytes per l.
//   warps 4..7  epilogue: tcgen05.ld the 128 x 224 fp32 accumulator in 32-column strips -> `Epi`
//
// TMEM (512 columns): accumulators at columns 0 and 256 (224 wide), the double-buffered scale words
// in the gap at 224..251.  The tile is 224 wide because two 256-wide accumulators would leave no room
// for the scales.  All waits are bounded.  No TMA load uses cluster multicast.
//
// The reference has no GEMM; its only mention of fp8 is a register-packing type
// (include/plugins/cuda_executor/utils/vector_datatype.h:66-80).
#pragma once
#include <cuda_bf16.h>

#include "../base/instr.h"
#include "gemm_pipeline.cuh"
#include "prims.cuh"
#include "tc05.cuh"

namespace pccl {
namespace gemmx {

using gemm::TileCoord;

constexpr int BM = 128, BN = 224, BK = 128, UMMA_K = 32;
constexpr int STAGES = 5;
constexpr int A_BYTES = BM * BK;            // 16 KiB
constexpr int B_BYTES = BN * BK;            // 28 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SF_BYTES = 512 + 1024;        // one scale image: A (128 rows) + B (up to 256 columns)
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 256;
constexpr int SF_IMAGES = 2;                // scale images in shared memory (five 44 KiB stages leave room for two)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SF_IMAGES * SF_BYTES + 1024 + 256;
static_assert(SF_IMAGES == 2, "image and TMEM scale buffer of a K group must share their index (see the MMA issuer)");
static_assert(SMEM_BYTES <= 232448, "shared memory budget");

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t sf_full[SF_IMAGES];
  uint64_t sf_empty[SF_IMAGES];
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort;
};

// sa: UE8M0 bytes [M, ld_sa]; sb: UE8M0 bytes [ceil(N/128), ld_sb]; one byte per 128 values of K.
struct Scales {
  const uint8_t* sa;
  const uint8_t* sb;
  int ld_sa, ld_sb;
  int M, N;
};

// Shared-memory descriptor of a 32 x 16-byte scale image for tcgen05.cp: no swizzle, K-major, 8-row core
// matrices 128 bytes apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>(128 >> 4) << 32;     // stride between core matrices along the rows
  d |= 1ull << 46;
  return d;
}
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void mma_mx8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t tsfa, uint32_t tsfb,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
// Instruction descriptor of the block-scaled kinds: [4,6) B scale id, [7,10) A format, [10,13) B format (0 = e4m3),
// [15]/[16] A/B MN-major, [17,23) N>>3, [23] scale format (1 = UE8M0), [24,29) M>>4, [29,31) A scale id.
__host__ __device__ constexpr uint32_t make_idesc_mx(uint32_t m, uint32_t n) { return ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24); }

template <class Sched, class Gate, class Epi>
__device__ __forceinline__ void run(const CUtensorMap* tmA, const CUtensorMap* tmB, int K, const Scales& sc, const Sched& sched,
                                    const Gate& gate, Epi& epi, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sf_smem = smem + STAGES * STAGE_BYTES;
  Barriers* bar = reinterpret_cast<Barriers*>(sf_smem + SF_IMAGES * SF_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;
  const int num_kg = (num_kb + 3) / 4;
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
    for (int a = 0; a < SF_IMAGES; ++a) {
      tc::mbar_init(&bar->sf_full[a], 1);
      tc::mbar_init(&bar->sf_empty[a], 1);
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
  epi.attach_smem(nullptr);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (tc::elect_one()) {
      int stage = 0;
      uint32_t phase = 0, armed = 0, armed_par = 0;
      bool ok = true;
      TileCoord t;
      for (int it = 0; ok && sched.get(it, &t); ++it) {
        if (!gate.wait(t, abort)) { ok = false; break; }
        const int row0 = t.m * BM, col0 = t.n * BN;
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
      constexpr uint32_t idesc0 = make_idesc_mx(BM, BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0, g = 0;       // g: 512-wide K groups issued so far
      bool ok = true;
      TileCoord t;
      for (int it = 0; ok && sched.get(it, &t); ++it) {
        if (!tc::mbar_wait(&bar->tmem_empty[acc], acc_phase ^ 1, abort)) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem + acc * 256;
        for (int kb = 0; kb < num_kb; ++kb) {
          // scale words of group g: TMEM buffer g & 1, shared-memory image g & 1.  The copy for group g+2 reuses the TMEM
          // words of group g; its image is only written after sf_empty of group g, i.e. after every MMA of group g has
          // finished, so the copy cannot overwrite scales that are still in use
          const uint32_t buf = g & 1, im = g % SF_IMAGES;
          const uint32_t tsfa = tmem + BN + 16 * buf, tsfb = tsfa + 4;
          if (!tc::mbar_wait(&bar->full[stage], phase, abort)) { ok = false; break; }
          if ((kb & 3) == 0) {
            if (!tc::mbar_wait(&bar->sf_full[im], (g / SF_IMAGES) & 1, abort)) { ok = false; break; }
            tc::tc_fence_after();
            const uint32_t img = tc::smem_u32(sf_smem + im * SF_BYTES);
            tmem_cp_32x128b_x4(tsfa, sf_desc(img));
            tmem_cp_32x128b_x4(tsfb, sf_desc(img + 512));
            tmem_cp_32x128b_x4(tsfb + 4, sf_desc(img + 1024));
          }
          tc::tc_fence_after();
          const uint32_t sa = tc::smem_u32(smem + stage * STAGE_BYTES), sb = sa + A_BYTES;
          const uint32_t sf = static_cast<uint32_t>(kb & 3);
          const uint32_t idesc = idesc0 | (sf << 29) | (sf << 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t da = tc::smem_desc_sw128(sa + k * UMMA_K, 16, 1024);
            uint64_t db = tc::smem_desc_sw128(sb + k * UMMA_K, 16, 1024);
            mma_mx8(d_tmem, da, db, idesc, tsfa, tsfb, (kb | k) != 0);
          }
          tc::mma_commit(&bar->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if ((kb & 3) == 3 || kb == num_kb - 1) {
            tc::mma_commit(&bar->sf_empty[im]);        // the copies that read this scale image have finished
            ++g;
          }
        }
        if (!ok) break;
        tc::mma_commit(&bar->tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok && atomicExch(const_cast<uint32_t*>(&bar->abort), 1u) == 0) dev::report(status, ST_TIMEOUT, blockIdx.x, 1, 0);
      tc::mma_commit(&bar->drain);
      for (uint32_t i = 0; i < (1u << 20) && !tc::mbar_try_wait(&bar->drain, 0); ++i) {}
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ scale builder (whole warp)
    // The words of the NEXT group (also across a tile boundary) are fetched from global memory into registers while
    // the MMAs of the current ones run; once the image buffer is free only the shared-memory writes remain.
    const int nblk = (sc.N + 127) / 128;
    const bool aligned4 = ((sc.ld_sa | sc.ld_sb) & 3) == 0 && ((reinterpret_cast<uintptr_t>(sc.sa) | reinterpret_cast<uintptr_t>(sc.sb)) & 3) == 0;
    uint32_t wa[4], wb[8];
    auto fetch = [&](const TileCoord& tt, int kg) {
      const int row0 = tt.m * BM, col0 = tt.n * BN, kb0 = kg * 4;
      const bool wide = aligned4 && kb0 + 4 <= num_kb;     // four scale bytes in one load
#pragma unroll
      for (int q = 0; q < 4; ++q) {               // A: rows 32 q + lane
        const int row = min(row0 + 32 * q + lane, sc.M - 1);
        const uint8_t* p = sc.sa + static_cast<long long>(row) * sc.ld_sa;
        uint32_t w = 0;
        if (wide) {
          w = __ldcg(reinterpret_cast<const uint32_t*>(p + kb0));     // may have been written by a peer: past L1
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (kb0 + j < num_kb) w |= static_cast<uint32_t>(__ldcg(p + kb0 + j)) << (8 * j);
        }
        wa[q] = w;
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {               // B: tile columns 32 q + lane
        const int blk = min((col0 + 32 * q + lane) >> 7, nblk - 1);
        const uint8_t* p = sc.sb + static_cast<long long>(blk) * sc.ld_sb;
        uint32_t w = 0;
        if (wide) {
          w = __ldg(reinterpret_cast<const uint32_t*>(p + kb0));
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (kb0 + j < num_kb) w |= static_cast<uint32_t>(__ldg(p + kb0 + j)) << (8 * j);
        }
        wb[q] = w;
      }
    };
    auto gate_open = [&](const TileCoord& tt) {   // A's scales arrive with its rows: read them only behind the gate
      int open = 1;
      if (lane == 0) open = gate.wait(tt, abort) ? 1 : 0;
      return __shfl_sync(0xffffffffu, open, 0) != 0;
    };
    uint32_t g = 0;
    bool ok = true;
    TileCoord t, tn;
    bool have = sched.get(0, &t);
    if (have) {
      ok = gate_open(t);
      if (ok) fetch(t, 0);
    }
    for (int it = 0; ok && have; ++it) {
      const bool have_next = sched.get(it + 1, &tn);
      for (int kg = 0; kg < num_kg; ++kg, ++g) {
        const uint32_t im = g % SF_IMAGES;
        int open = 1;
        if (lane == 0) open = tc::mbar_wait(&bar->sf_empty[im], ((g / SF_IMAGES) & 1) ^ 1, abort) ? 1 : 0;
        if (!__shfl_sync(0xffffffffu, open, 0)) { ok = false; break; }
        uint8_t* img = sf_smem + im * SF_BYTES;
#pragma unroll
        for (int q = 0; q < 4; ++q) *reinterpret_cast<uint32_t*>(img + lane * 16 + q * 4) = wa[q];
#pragma unroll
        for (int q = 0; q < 8; ++q) *reinterpret_cast<uint32_t*>(img + 512 + (q >> 2) * 512 + lane * 16 + (q & 3) * 4) = wb[q];
        tc::fence_proxy_async_smem();                // the image is read by tcgen05.cp (async proxy)
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&bar->sf_full[im]);
        if (kg + 1 < num_kg) {
          fetch(t, kg + 1);
        } else if (have_next) {
          if (!gate_open(tn)) { ok = false; break; }
          fetch(tn, 0);
        }
      }
      t = tn;
      have = have_next;
    }
    if (!ok && lane == 0 && atomicExch(const_cast<uint32_t*>(&bar->abort), 1u) == 0) dev::report(status, ST_TIMEOUT, blockIdx.x, 3, 0);
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    TileCoord t;
    for (int it = 0; ok && sched.get(it, &t); ++it) {
      if (!tc::mbar_wait(&bar->tmem_full[acc], acc_phase, abort)) { ok = false; break; }
      tc::tc_fence_after();
      const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + acc * 256;
      const TileCoord t0{t.m, 0, t.extra};           // the adapter gets absolute columns
      epi.tile_begin(t0);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(taddr + c * 32, r);
        tc::tmem_ld_wait();
        epi.strip(t0, quarter * 32 + lane, t.n * BN + c * 32, r);
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&bar->tmem_empty[acc]);
      epi.tile_done(t0, abort);
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

}  // namespace gemmx
}  // namespace pccl
