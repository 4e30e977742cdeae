// Tensor/sequence-parallel MLP halves with the collective fused into the GEMM kernel, tile by tile.
//
//   all-gather -> GEMM   Y[M,N] = gather_rows(X)[M,K] * W1[N,K]^T.  Every rank keeps its own row
//       block of X inside a symmetric [M,K] buffer.  A few CTAs of the kernel pull the peers' row
//       blocks over NVLink with bulk async copies (peer global -> shared -> local global, ~190 KB in
//       flight per CTA) in 128-row chunks and raise a local flag per chunk; the other CTAs run the
//       tcgen05 pipeline, starting with the local rows and taking the remote panels in arrival
//       order; a tile's TMA loads are issued once its chunk's flag is up.  TMA only ever reads
//       local memory and nothing uses cluster multicast.
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
#include "gemm_epilogue.cuh"
#include "gemm_pipeline.cuh"
#include "tensormap.h"

namespace pccl {

namespace {

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
struct AgSched {
  int me, world, tiles_ml, tiles_n, first, stride;
  __device__ __forceinline__ bool get(int it, TileCoord* t) const {
    const long long idx = first + static_cast<long long>(it) * stride;
    const int per_panel = tiles_ml * tiles_n;
    if (idx >= static_cast<long long>(world) * per_panel) return false;
    const int panel = static_cast<int>(idx / per_panel), r = static_cast<int>(idx % per_panel);
    int src = me + panel;
    if (src >= world) src -= world;
    t->m = src * tiles_ml + r % tiles_ml;
    t->n = r / tiles_ml;
    t->extra = src;
    return true;
  }
};

struct AgGate {
  const uint32_t* ready;   // per 128-row chunk of the gathered X: pieces copied so far (never reset)
  int me;
  uint32_t target;         // epoch * pieces per chunk
  uint64_t spin_ns;
  __device__ __forceinline__ bool wait(const TileCoord& t, const volatile uint32_t* abort) const {
    if (t.extra == me) return true;
    const uint32_t* f = ready + t.m;
    if (dev::ld_acquire_gpu_u32(f) < target) {
      const uint64_t t0 = dev::global_timer_ns();
      for (uint32_t i = 1;; ++i) {
        if (dev::ld_acquire_gpu_u32(f) >= target) break;
        if ((i & 31) == 0) {
          if (*abort) return false;
          if (dev::global_timer_ns() - t0 > spin_ns) return false;
          __nanosleep(64);
        }
      }
    }
    tc::fence_proxy_async();   // the chunk was written through the async proxy of other CTAs; TMA reads it next
    return true;
  }
};

constexpr int kCopyPiece = 32 * 1024;
constexpr int kCopyBufs = 6;

// One thread per copy CTA drives a ring of bulk copies: peer global -> shared -> local global.
__device__ void ag_copy_role(const AgGemmArgs& A, const AgGemmRank& R, uint8_t* smem) {
  const int me = R.rank, world = A.w.world, j = blockIdx.x;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kCopyBufs * kCopyPiece);
  __shared__ uint32_t s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int b = 0; b < kCopyBufs; ++b) tc::mbar_init(&bars[b], 1);
    tc::fence_barrier_init();
  }
  __syncthreads();
  bool ok = cta_peer_barrier(A.w, me, A.flag_lane, j, 4 * A.bar_epoch + 1, A.spin_ns, R.status);
  if (ok && threadIdx.x == 0) {
    const int chunks = A.M_local / BM;
    const long long chunk_bytes = static_cast<long long>(BM) * A.K * 2;
    const int pieces = static_cast<int>(chunk_bytes / kCopyPiece);      // host checks divisibility
    // All pieces of all remote chunks form one list in the order the GEMM consumes them (panel
    // me+1 first); CTA j takes pieces j, j+n_copy, ... so every chunk is pulled by all copy CTAs
    // together and the first chunks are complete almost at once.
    const long long all = static_cast<long long>(world - 1) * chunks * pieces;
    const long long total = j < all ? (all - j + A.n_copy - 1) / A.n_copy : 0;
    auto locate = [&](long long q, const char** src, char** dst, int* m_tile) {
      const long long g = j + q * A.n_copy;
      const int it = static_cast<int>(g / pieces), pc = static_cast<int>(g % pieces);
      const int panel = 1 + it / chunks, c = it % chunks;
      int s = me + panel;
      if (s >= world) s -= world;
      const long long off = static_cast<long long>(A.x_off) +
                            (static_cast<long long>(s) * A.M_local + static_cast<long long>(c) * BM) * A.K * 2 +
                            static_cast<long long>(pc) * kCopyPiece;
      *src = A.w.heap[s] + off;
      *dst = A.w.heap[me] + off;
      *m_tile = s * chunks + c;
    };
    auto signal_piece = [&](long long q) {
      const char* s; char* d; int mt;
      locate(q, &s, &d, &mt);
      tc::fence_proxy_async();
      __threadfence();
      asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(R.ready + mt) : "memory");
    };
    long long issued = 0;
    uint32_t phase_bits = 0;     // wait parity per buffer
    for (; issued < total && issued < kCopyBufs; ++issued) {
      const char* s; char* d; int mt;
      locate(issued, &s, &d, &mt);
      tc::mbar_arrive_expect_tx(&bars[issued], kCopyPiece);
      tc::bulk_load_g2s(smem + issued * kCopyPiece, s, kCopyPiece, &bars[issued]);
    }
    long long done = 0;          // pieces whose store has been issued
    for (long long q = 0; q < total; ++q) {
      const int b = static_cast<int>(q % kCopyBufs);
      const char* s; char* d; int mt;
      locate(q, &s, &d, &mt);
      if (!tc::mbar_wait(&bars[b], (phase_bits >> b) & 1, &s_abort)) {
        dev::report(R.status, ST_TIMEOUT, j, 3, static_cast<uint32_t>(q));
        ok = false;
        break;
      }
      phase_bits ^= 1u << b;
      tc::fence_proxy_async_smem();
      tc::bulk_store_s2g(d, smem + b * kCopyPiece, kCopyPiece);
      tc::bulk_commit();
      done = q + 1;
      if (q >= 1) {
        tc::bulk_wait<1>();            // the store of piece q-1 has landed in local memory
        signal_piece(q - 1);
        if (issued < total) {          // its buffer is free again
          const int fb = static_cast<int>((q - 1) % kCopyBufs);
          const char* s2; char* d2; int mt2;
          locate(issued, &s2, &d2, &mt2);
          tc::mbar_arrive_expect_tx(&bars[fb], kCopyPiece);
          tc::bulk_load_g2s(smem + fb * kCopyPiece, s2, kCopyPiece, &bars[fb]);
          ++issued;
        }
      }
    }
    tc::bulk_wait<0>();
    if (done >= 1 && ok) signal_piece(done - 1);
    if (!ok) {
      // loads still in flight must land before this CTA's shared memory is released
      for (long long q = done; q < issued; ++q) {
        const int b = static_cast<int>(q % kCopyBufs);
        for (uint32_t i = 0; i < (1u << 16) && !tc::mbar_try_wait(&bars[b], (phase_bits >> b) & 1); ++i) {}
      }
    }
  }
  __syncthreads();
  // peers may still be pulling our rows: nobody leaves (and lets the next kernel overwrite X) before all are done
  cta_peer_barrier(A.w, me, A.flag_lane, j, 4 * A.bar_epoch + 2, A.spin_ns, R.status);
}

template <bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1) ag_gemm_kernel(const __grid_constant__ AgGemmArgs A) {
  const AgGemmRank& R = A.r[blockIdx.y];
  if (static_cast<int>(blockIdx.x) < A.n_copy) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    if (A.w.world > 1) ag_copy_role(A, R, smem);
    return;
  }
  const int tiles_ml = A.M_local / BM, tiles_n = (A.N + BN - 1) / BN;
  AgSched sched{R.rank, A.w.world, tiles_ml, tiles_n, static_cast<int>(blockIdx.x) - A.n_copy, static_cast<int>(gridDim.x) - A.n_copy};
  AgGate gate{R.ready, R.rank, static_cast<uint32_t>(A.epoch) * static_cast<uint32_t>((static_cast<long long>(BM) * A.K * 2) / kCopyPiece), A.spin_ns};
  StoreEpi epi{R.D, nullptr, static_cast<const __nv_bfloat16*>(R.bias), R.ldd, A.M, A.N, A.flags};
  run<false, B_MN>(&R.tmA, &R.tmB, A.K, sched, gate, epi, R.status);
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

struct RsEpi {
  const GemmRsArgs* A;
  const GemmRsRank* R;
  uint8_t* stage;      // this warp's 32 x 144 B staging rows
  int me, tiles_ml, tiles_n;

  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return t.m * BM; }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return t.n * BN; }
  __device__ __forceinline__ void attach_smem(uint8_t* p) { stage = p + ((threadIdx.x >> 5) & 3) * (32 * kRsPitch); }

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
    if (lane < A->w.world && lane != me) {
      if (!dev::wait_ge(tile_flag(me, lane, tile_local_index(t)), A->epoch, A->spin_ns, nullptr))
        dev::report(R->status, ST_TIMEOUT, blockIdx.x, 4, static_cast<uint32_t>(lane));
    }
    __syncwarp();
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
        tc::bulk_wait_read<0>();      // the staging row may be overwritten by the next strip
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
    tc::bulk_wait<0>();                  // this lane's rows have been written to the owner
    tc::fence_proxy_async();
    asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
    if ((threadIdx.x >> 5) == 2 && (threadIdx.x & 31) == 0) {
      __threadfence_system();
      dev::st_release_sys(tile_flag(t.extra, me, tile_local_index(t)), A->epoch);
    }
  }
};

template <bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_rs_kernel(const __grid_constant__ GemmRsArgs A) {
  const GemmRsRank& R = A.r[blockIdx.y];
  const int tiles_ml = A.M_local / BM, tiles_n = A.N / BN;
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
  if (A.M_local % BM || A.M != A.M_local * A.w.world || A.K % 8 || (static_cast<long long>(BM) * A.K * 2) % kCopyPiece) {
    g_err = "ag_gemm: rows per rank must be a multiple of 128 and 128*K*2 a multiple of 32 KiB";
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
  void* kern = host[0].b_mn ? reinterpret_cast<void*>(ag_gemm_kernel<true>) : reinterpret_cast<void*>(ag_gemm_kernel<false>);
  static bool set[2] = {false, false};
  if (!set[host[0].b_mn]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    set[host[0].b_mn] = true;
  }
  dim3 grid(ctas, nv), block(NUM_THREADS);
  void* args[] = {&A};
  return static_cast<int>(cudaLaunchCooperativeKernel(kern, grid, block, args, SMEM_BYTES, stream));
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
  void* kern = host[0].b_mn ? reinterpret_cast<void*>(gemm_rs_kernel<true>) : reinterpret_cast<void*>(gemm_rs_kernel<false>);
  static bool set[2] = {false, false};
  if (!set[host[0].b_mn]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, RS_SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    set[host[0].b_mn] = true;
  }
  dim3 grid(ctas, nv), block(NUM_THREADS);
  void* args[] = {&A};
  return static_cast<int>(cudaLaunchCooperativeKernel(kern, grid, block, args, RS_SMEM_BYTES, stream));
}

}  // namespace pccl
