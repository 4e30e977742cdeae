// Host entry points of the kernels that fuse a collective into the tcgen05 GEMM (fused_tp.cu).
// ("communication-computation overlap" is a feature bullet of the reference, README.md:1-9, with no code behind it.)
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "api.h"

namespace pccl {

constexpr int kMaxVirt = 4;   // ranks that one launch can emulate on a single GPU (tests)

// Opt-in time attribution of the fused kernels.  With a probe buffer set (device memory, kProbeWords u64 per CTA of the
// largest grid, zeroed by the caller), every CTA adds up where it waited, in nanoseconds of %globaltimer:
//   [0] all-gather GEMM: waiting for a remote chunk's counter before a tile's loads (AgGate)
//   [1] GEMM reduce-scatter: waiting for the peers' partial tiles before an own tile (tile_begin)
//   [2] GEMM reduce-scatter: waiting for staged rows to leave shared memory (per strip / per tile)
//   [3] GEMM reduce-scatter: waiting for a peer tile's writes to complete before its flag is released (tile_done)
//   [4] %globaltimer when the CTA started, [5] when it ended, [6] duration of the copy role, [7] tiles computed
// The probes cost a few timer reads per tile; they are for attribution runs, not for timed ones.
constexpr int kProbeWords = 8;
void setFusedProbe(unsigned long long* device_buffer);

struct AgGemmRank {
  CUtensorMap tmA, tmB;       // filled by launchAgGemm
  void* D;                    // [M, N] bf16 output (local)
  long long ldd;
  const void* bias;           // bf16 [N] or null
  uint32_t* status;
  int rank;
  int pad;
  // block-scaled fp8 only
  const float* w_scale;       // fp32 [N/128, ld_ws]: 128 x 128 scales of the W shard (UE8M0 bytes when scale_bytes is 1)
  int ld_ws;
  int pad2;
  void* Dq;                   // when set, the output is quantised instead: e4m3 [M, ldq] ...
  float* Ds;                  // ... with fp32 1 x 128 scales [M, N/128]
  long long ldq;
};

struct AgGemmArgs {
  World w;
  int nvirt;                  // 1, or the emulated world size
  int M, N, K, M_local;       // M = M_local * world
  uint64_t x_off;             // heap offset of the symmetric gathered-X buffer [M, K] bf16; rows
                              // [rank*M_local, (rank+1)*M_local) hold the rank's own activations
  uint64_t ready_off;         // heap offset of the symmetric chunk counters: uint32 [M / 128], zeroed once
  uint64_t epoch;             // 1, 2, 3, ... per launch on these buffers (chunk counters)
  uint64_t bar_epoch;         // strictly increasing per launch on `flag_lane` (peer barriers)
  int n_copy;                 // CTAs that pull peer rows (the rest compute)
  int flag_lane;
  uint64_t spin_ns;
  uint32_t flags;             // GEMM_BIAS, GEMM_GELU_INPLACE (fp8 path)
  int elem_bytes;             // 2 (bf16 X) or 1 (e4m3 X with scales at xs_off); 0 is read as 2
  uint64_t xs_off;            // fp8: heap offset of the symmetric gathered scales [M, K/128]: fp32, or UE8M0 bytes (scale_bytes 1)
  int scale_bytes;            // 4 (fp32 scales; 0 is read as 4) or 1 (UE8M0 bytes, hardware block scaling)
  int tail_tiles;             // tiles at the end of the tile order that the copy CTAs compute once their rows are sent
  unsigned long long* probe;  // null, or kProbeWords x u64 per CTA (see setFusedProbe)
  AgGemmRank r[kMaxVirt];
};

// W shard per (virtual) rank: [N, K] bf16 row-major, or, with b_mn, stored [K, N] (the transposed view feeds
// backward passes without a transpose)
struct AgGemmHost { const void* W; long long ldw; bool b_mn; };

struct GemmRsRank {
  CUtensorMap tmA, tmB;
  void* out;                  // [M_local, N] bf16 (local)
  long long ldo;
  uint32_t* status;
  int rank;
  int pad;
  // block-scaled fp8 only
  const float* y_scale;       // fp32 [M, ld_ys]
  const float* w_scale;       // fp32 [N/128, ld_ws]
  int ld_ys, ld_ws;
};

struct GemmRsArgs {
  World w;
  int nvirt;
  int M, N, K, M_local;
  uint64_t stage_off;         // heap offset of the symmetric staging buffer [world][M_local][N] bf16
  uint64_t flag_off2;         // heap offset of the symmetric tile flags uint64 [world][M_local/128 * N/256], zeroed once
  uint64_t epoch;
  uint64_t spin_ns;
  unsigned long long* probe;  // null, or kProbeWords x u64 per CTA (see setFusedProbe)
  GemmRsRank r[kMaxVirt];
};

struct GemmRsHost { const void* Y; long long ldy; const void* W; long long ldw; bool b_mn; };   // Y [M, K]; W [N, K], or [K, N] with b_mn

int launchAgGemm(AgGemmArgs& args, const AgGemmHost* host, int ctas, cudaStream_t stream);
int launchGemmRs(GemmRsArgs& args, const GemmRsHost* host, int ctas, cudaStream_t stream);
// Block-scaled fp8 forms (fused_tp_fp8.cu): X / Y and W are e4m3 bytes, K-major, K a multiple of 128, N a multiple of
// 256; the scale fields of the argument structs must be filled.  Single-CTA tiles.
int launchAgGemmFp8(AgGemmArgs& args, const AgGemmHost* host, int ctas, cudaStream_t stream);
int launchGemmRsFp8(GemmRsArgs& args, const GemmRsHost* host, int ctas, cudaStream_t stream);
// all-gather -> GEMM on the hardware block-scaled pipeline (UE8M0 scale bytes; N a multiple of 32; bf16 output)
int launchAgGemmMx8(AgGemmArgs& args, const AgGemmHost* host, int ctas, cudaStream_t stream);
const char* fusedLastError();

}  // namespace pccl
