// Device parts shared by the bf16 and the fp8 kernels that fuse a collective into the tcgen05 GEMM:
// the peer barrier, the all-gather push role with its tile scheduler and gate, and the reduce-scatter
// scheduler and epilogue.  See fused_tp.cu for the protocols.
#pragma once
#include <cuda.h>

#include "fused_api.h"
#include "gemm_epilogue.cuh"
#include "gemm_pipeline.cuh"
#include "prims.cuh"
#include "tc05.cuh"

namespace pccl {
namespace fused {

using namespace gemm;

__device__ __forceinline__ uint64_t* lane_flag(const World& W, int owner, int lane, int block, int src) {
  return reinterpret_cast<uint64_t*>(W.heap[owner] + W.flag_off) +
         ((static_cast<uint64_t>(lane) * kMaxBlocksPerColl + block) * kMaxRanks + src);
}

// Barrier among CTA `block` of every rank, executed by the first `world` threads of the CTA.
__device__ __forceinline__ bool cta_peer_barrier(const World& W, int me, int lane, int block, uint64_t value, uint64_t spin_ns,
                                                 uint32_t* status) {
  __shared__ uint32_t s_bad;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  if (threadIdx.x < static_cast<uint32_t>(W.world)) {
    const int p = threadIdx.x;
    __threadfence_system();
    dev::st_release_sys(lane_flag(W, p, lane, block, me), value);
    if (!dev::wait_ge(lane_flag(W, me, lane, block, p), value, spin_ns, nullptr)) {
      s_bad = 1;
      dev::report(status, ST_TIMEOUT, block, static_cast<uint32_t>(p), 100 + static_cast<uint32_t>(value & 3));
    }
  }
  __syncthreads();
  return s_bad == 0;
}

// =================================================================================================
// all-gather -> GEMM
// =================================================================================================
// Tile order of the all-gather GEMM: the rank's own rows first (they are there), then the remote rows
// row block by row block -- block b of EVERY peer before block b+1 of any -- which is the order in which
// the senders emit them, so the data keeps ahead of the tensor cores from the first remote tile on.
// Within a row block consecutive tiles share the B panel (same n, different source rank).
// [begin, end) is the slice of that order which this group of CTAs works through (`first` + it * `stride` inside it):
// the GEMM CTAs take everything but the last `tail` tiles, the copy CTAs take the tail once their rows are sent.
struct AgSched {
  int me, world, tiles_ml, tiles_n, first, stride;
  long long begin, end;
  __device__ __forceinline__ bool get(int it, TileCoord* t) const {
    const long long idx = begin + first + static_cast<long long>(it) * stride;
    const int per_panel = tiles_ml * tiles_n;
    if (idx >= end || idx >= static_cast<long long>(world) * per_panel) return false;
    if (idx < per_panel) {
      const int r = static_cast<int>(idx);
      t->m = me * tiles_ml + r % tiles_ml;
      t->n = r / tiles_ml;
      t->extra = me;
      return true;
    }
    const long long j = idx - per_panel;
    const int per_block = (world - 1) * tiles_n;
    const int blk = static_cast<int>(j / per_block), rem = static_cast<int>(j % per_block);
    int src = me + 1 + rem % (world - 1);
    if (src >= world) src -= world;
    t->m = src * tiles_ml + blk;
    t->n = rem / (world - 1);
    t->extra = src;
    return true;
  }
};

struct AgGate {
  const uint32_t* ready;   // per 128-row chunk of the gathered X: parts written so far by the owner's copy CTAs (never reset)
  int me;
  uint32_t target;         // epoch * copy CTAs
  uint64_t spin_ns;
  unsigned long long* probe = nullptr;     // this CTA's probe words, or null
  __device__ __forceinline__ bool wait(const TileCoord& t, const volatile uint32_t* abort) const {
    if (probe) atomicAdd(probe + 7, 1ull);
    if (t.extra == me) return true;
    const uint32_t* f = ready + t.m;
    if (dev::ld_acquire_sys_u32(f) < target) {
      const uint64_t t0 = dev::global_timer_ns();
      struct Tally {
        unsigned long long* p; uint64_t t0;
        __device__ ~Tally() { if (p) atomicAdd(p, static_cast<unsigned long long>(dev::global_timer_ns() - t0)); }
      } tally{probe, t0};
      for (uint32_t i = 1;; ++i) {
        if (dev::ld_acquire_sys_u32(f) >= target) break;
        if ((i & 31) == 0) {
          if (*abort) return false;
          if (dev::global_timer_ns() - t0 > spin_ns) return false;
          __nanosleep(64);
        }
      }
    }
    tc::fence_proxy_async();   // the chunk was written by a peer's ordinary stores; TMA (async proxy) reads it next
    return true;
  }
};

// Copy CTAs send this rank's rows to every peer's gathered buffer, 128-row chunk by chunk; a chunk is
// split across the copy CTAs and each adds one to the receivers' counter for that chunk when its part
// has been written.
//   With an NVLS multicast mapping of the heap: ONE multimem.st per 16 bytes reaches all peers (the
//   switch replicates it), so a rank issues its rows once instead of world-1 times, and one
//   multimem.red bumps the chunk counter on every receiver.  A few CTAs saturate the receivers' ports.
//   Without it: plain 16-byte stores to each peer in turn (posted writes) and one counter update per peer.
template <bool MC>
__device__ __forceinline__ void push_store(char* dst, const dev::Vec16& v) {
  if constexpr (MC) dev::multimem_st(dst, v);
  else dev::st16(dst, v);
}

// Copies 16-byte vectors [lo, hi) of src to dst with the whole CTA; the loads of batch b+1 are issued
// before the stores of batch b, so that a thread keeps 8 to 16 vectors in flight.
template <bool MC>
__device__ __forceinline__ void push_vecs(const char* src, char* dst, long long lo, long long hi) {
  const long long nt = blockDim.x;
  long long i = lo + threadIdx.x;
  if (i + 7 * nt < hi) {
    dev::Vec16 cur[8], nxt[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) cur[u] = dev::ld16(src + ((i + u * nt) << 4));
    for (;;) {
      const long long j = i + 8 * nt;
      const bool more = j + 7 * nt < hi;
      if (more) {
#pragma unroll
        for (int u = 0; u < 8; ++u) nxt[u] = dev::ld16(src + ((j + u * nt) << 4));
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) push_store<MC>(dst + ((i + u * nt) << 4), cur[u]);
      i = j;
      if (!more) break;
#pragma unroll
      for (int u = 0; u < 8; ++u) cur[u] = nxt[u];
    }
  }
  for (; i < hi; i += nt) push_store<MC>(dst + (i << 4), dev::ld16(src + (i << 4)));
}

__device__ __forceinline__ void ag_push_role(const AgGemmArgs& A, const AgGemmRank& R) {
  const int me = R.rank, world = A.w.world, j = blockIdx.x;
  const uint64_t push_t0 = A.probe ? dev::global_timer_ns() : 0;
  struct PushTally {
    unsigned long long* p; uint64_t t0;
    __device__ ~PushTally() { if (p && threadIdx.x == 0) p[6] = dev::global_timer_ns() - t0; }
  } push_tally{A.probe ? A.probe + static_cast<long long>(blockIdx.y * gridDim.x + blockIdx.x) * kProbeWords : nullptr, push_t0};
  if (!cta_peer_barrier(A.w, me, A.flag_lane, j, 4 * A.bar_epoch + 1, A.spin_ns, R.status)) return;
  const int chunks = A.M_local / BM;
  const long long row_bytes = static_cast<long long>(A.K) * (A.elem_bytes ? A.elem_bytes : 2);
  const long long nvec = (static_cast<long long>(BM) * row_bytes) >> 4;
  const long long per = (nvec + A.n_copy - 1) / A.n_copy;
  const long long lo = min(nvec, per * j), hi = min(nvec, per * (j + 1));
  // block-scaled operands: the 1 x 128 scales of a chunk (fp32 [128, K/128]) travel with it
  const int sbytes = A.scale_bytes ? A.scale_bytes : 4;
  const long long svec = A.xs_off ? (static_cast<long long>(BM) * (A.K / 128) * sbytes) >> 4 : 0;
  const long long sper = (svec + A.n_copy - 1) / A.n_copy;
  const long long slo = min(svec, sper * j), shi = min(svec, sper * (j + 1));
  const bool mc = A.w.mc_heap != nullptr && A.nvirt <= 1;
  for (int c = 0; c < chunks; ++c) {
    const long long row0 = static_cast<long long>(me) * A.M_local + static_cast<long long>(c) * BM;
    const long long off = static_cast<long long>(A.x_off) + row0 * row_bytes;
    const long long soff = static_cast<long long>(A.xs_off) + row0 * (A.K / 128) * sbytes;
    const long long cnt_off = static_cast<long long>(A.ready_off) + static_cast<long long>(me * chunks + c) * 4;
    if (mc) {
      push_vecs<true>(A.w.heap[me] + off, A.w.mc_heap + off, lo, hi);
      if (svec) push_vecs<true>(A.w.heap[me] + soff, A.w.mc_heap + soff, slo, shi);
      __syncthreads();                        // every thread's stores of this chunk part are issued
      if (threadIdx.x == 0) {
        __threadfence_system();
        asm volatile("multimem.red.release.sys.global.add.u32 [%0], 1;" ::"l"(A.w.mc_heap + cnt_off) : "memory");
      }
    } else {
      for (int k = 1; k < world; ++k) {
        int p = me - k;
        if (p < 0) p += world;
        push_vecs<false>(A.w.heap[me] + off, A.w.heap[p] + off, lo, hi);
        if (svec) push_vecs<false>(A.w.heap[me] + soff, A.w.heap[p] + soff, slo, shi);
      }
      __syncthreads();
      if (threadIdx.x >= 1 && threadIdx.x < static_cast<uint32_t>(world)) {
        int p = me - static_cast<int>(threadIdx.x);
        if (p < 0) p += world;
        __threadfence_system();
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(A.w.heap[p] + cnt_off) : "memory");
      }
    }
  }
}

// =================================================================================================
// GEMM -> reduce-scatter
// =================================================================================================
struct RsSched {
  int me, world, tiles_ml, tiles_n, first, stride;
  __device__ __forceinline__ bool get(int it, TileCoord* t) const {
    const long long idx = first + static_cast<long long>(it) * stride;
    const int per_panel = tiles_ml * tiles_n;
    if (idx >= static_cast<long long>(world) * per_panel) return false;
    const int panel = static_cast<int>(idx / per_panel), r = static_cast<int>(idx % per_panel);
    int owner = me + 1 + panel;          // peers first, own rows last
    if (owner >= world) owner -= world;
    t->m = owner * tiles_ml + r % tiles_ml;
    t->n = r / tiles_ml;
    t->extra = owner;
    return true;
  }
};

constexpr int kRsPitch = 144;                       // bytes per staged row: 64 bf16 + 16 pad (bank-conflict free)
constexpr int kRsStageBytes = 4 * 32 * kRsPitch;    // four epilogue warps
constexpr int RS_SMEM_BYTES = SMEM_BYTES + kRsStageBytes;

// EW epilogue warps (warps 2 .. 2+EW of the CTA) take part.
template <int EW>
struct RsEpiT {
  static constexpr bool kRow128 = false;
  const GemmRsArgs* A;
  const GemmRsRank* R;
  uint8_t* stage;      // this warp's 32 x 144 B staging rows
  int me, tiles_ml, tiles_n;
  unsigned long long* probe = nullptr;     // this CTA's probe words, or null

  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return t.m * BM; }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return t.n * BN; }
  __device__ __forceinline__ void attach_smem(uint8_t* p) { stage = p + ((static_cast<int>(threadIdx.x >> 5) - 2) & (EW - 1)) * (32 * kRsPitch); }

  __device__ __forceinline__ long long tile_local_index(const TileCoord& t) const {
    return static_cast<long long>(t.m - t.extra * tiles_ml) * tiles_n + t.n;
  }
  __device__ __forceinline__ uint64_t* tile_flag(int owner, int src, long long tile_local) const {
    return reinterpret_cast<uint64_t*>(A->w.heap[owner] + A->flag_off2) + static_cast<long long>(src) * tiles_ml * tiles_n + tile_local;
  }

  __device__ __forceinline__ void tile_begin(const TileCoord& t) {
    if (t.extra != me) return;
    // our own rows: the peers' partials of this tile must be in our staging slots
    const int lane = threadIdx.x & 31;
    const uint64_t t0 = probe ? dev::global_timer_ns() : 0;
    if (lane < A->w.world && lane != me) {
      if (!dev::wait_ge(tile_flag(me, lane, tile_local_index(t)), A->epoch, A->spin_ns, nullptr))
        dev::report(R->status, ST_TIMEOUT, blockIdx.x, 4, static_cast<uint32_t>(lane));
    }
    __syncwarp();
    if (probe && lane == 0 && (threadIdx.x >> 5) == 2) atomicAdd(probe + 1, static_cast<unsigned long long>(dev::global_timer_ns() - t0));
  }

  __device__ __forceinline__ void strip(const TileCoord& t, int row_in_tile, int col_in_tile, uint32_t* r) {
    const int lane = threadIdx.x & 31;
    const int owner = t.extra;
    const long long row_local = static_cast<long long>(t.m - owner * tiles_ml) * BM + row_in_tile;   // row inside the owner's block
    const long long col = static_cast<long long>(t.n) * BN + col_in_tile;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    if (owner != me) {
      uint8_t* srow = stage + lane * kRsPitch + (col_in_tile & 32) * 2;
#pragma unroll
      for (int i = 0; i < 32; i += 8) *reinterpret_cast<dev::Vec16*>(srow + i * 2) = dev::pack<DT_BF16>(v + i);
      if (col_in_tile & 32) {
        // 64 columns staged: one 128-byte bulk copy per row into the owner's slot for this rank
        tc::fence_proxy_async_smem();
        __syncwarp();
        char* dst = A->w.heap[owner] + A->stage_off +
                    ((static_cast<long long>(me) * A->M_local + row_local) * A->N + (col - 32)) * 2;
        tc::bulk_store_s2g(dst, stage + lane * kRsPitch, 128);
        tc::bulk_commit();
        const uint64_t t0 = probe ? dev::global_timer_ns() : 0;
        tc::bulk_wait_read<0>();      // the staging row may be overwritten by the next strip
        if (probe && lane == 0 && (threadIdx.x >> 5) == 2) atomicAdd(probe + 2, static_cast<unsigned long long>(dev::global_timer_ns() - t0));
      }
      return;
    }
    // own rows: add the peers' bf16 partials (local memory) to the fp32 accumulator and store the result
    const char* base = A->w.heap[me] + A->stage_off;
    for (int s = 0; s < A->w.world; ++s) {
      if (s == me) continue;
      const char* p = base + ((static_cast<long long>(s) * A->M_local + row_local) * A->N + col) * 2;
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        float f[8];
        dev::unpack<DT_BF16>(dev::ld16(p + i * 2), f);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[i + k] += f[k];
      }
    }
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(R->out) + row_local * R->ldo + col;
#pragma unroll
    for (int i = 0; i < 32; i += 8) dev::st16(out + i, dev::pack<DT_BF16>(v + i));
  }

  __device__ __forceinline__ void tile_done(const TileCoord& t, const volatile uint32_t*) {
    if (t.extra == me) return;
    const uint64_t t0 = probe ? dev::global_timer_ns() : 0;
    tc::bulk_wait<0>();                  // this lane's rows have been written to the owner
    tc::fence_proxy_async();
    asm volatile("bar.sync 1, %0;" ::"n"(EW * 32) : "memory");   // the epilogue warps
    if ((threadIdx.x >> 5) == 2 && (threadIdx.x & 31) == 0) {
      __threadfence_system();
      dev::st_release_sys(tile_flag(t.extra, me, tile_local_index(t)), A->epoch);
      if (probe) {
        atomicAdd(probe + 3, static_cast<unsigned long long>(dev::global_timer_ns() - t0));
        atomicAdd(probe + 7, 1ull);
      }
    }
  }
};
using RsEpi = RsEpiT<4>;

// The same protocol with whole rows staged: a warp keeps 32 rows x 256 columns (512 bytes per row) of a peer-owned tile
// in shared memory and sends each row with ONE 512-byte bulk copy when the tile's last strip is packed, instead of a
// 128-byte copy and a full drain after every 64 columns.  Four times fewer, four times larger writes on NVLink, and the
// epilogue never waits inside a tile.  Needs 64 KiB of staging, which the CTA-pair kernel makes room for by running a
// five-stage operand ring (gemm2::run<..., 5>).
constexpr int kRsRowBytes = BN * 2;                          // 512
constexpr int kRsRowStageBytes = 4 * 32 * kRsRowBytes;       // four epilogue warps: 64 KiB
struct RsEpiRow : RsEpiT<4> {
  __device__ __forceinline__ void attach_smem(uint8_t* p) { stage = p + ((static_cast<int>(threadIdx.x >> 5) - 2) & 3) * (32 * kRsRowBytes); }

  __device__ __forceinline__ void strip(const TileCoord& t, int row_in_tile, int col_in_tile, uint32_t* r) {
    if (t.extra == me) {
      RsEpiT<4>::strip(t, row_in_tile, col_in_tile, r);
      return;
    }
    const int lane = threadIdx.x & 31;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    uint8_t* srow = stage + lane * kRsRowBytes;
#pragma unroll
    for (int i = 0; i < 32; i += 8) *reinterpret_cast<dev::Vec16*>(srow + (col_in_tile + i) * 2) = dev::pack<DT_BF16>(v + i);
    if (col_in_tile == BN - 32) {
      const int owner = t.extra;
      const long long row_local = static_cast<long long>(t.m - owner * tiles_ml) * BM + row_in_tile;
      char* dst = A->w.heap[owner] + A->stage_off +
                  ((static_cast<long long>(me) * A->M_local + row_local) * A->N + static_cast<long long>(t.n) * BN) * 2;
      tc::fence_proxy_async_smem();       // this lane's own stores to its row, before the bulk copy reads them
      tc::bulk_store_s2g(dst, srow, kRsRowBytes);
      tc::bulk_commit();
    }
  }
  // tile_done (inherited) waits for the copies, so the rows are free again before the next tile's first strip
};

}  // namespace fused
}  // namespace pccl
