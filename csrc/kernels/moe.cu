// Expert-parallel MoE data movement fused with its arithmetic, plus the fp8 block quantisers.
//
//   dispatch   one pass per token: bf16 row -> e4m3 with one fp32 scale per 128 values (amax / 448),
//              staged in shared memory, then stored straight into the receive buffers of the ranks
//              that own the token's top-k experts (NVLink stores, 16 bytes per thread per target)
//   dequant    fp8 rows + scales -> bf16 rows for the grouped expert GEMM
//   combine    one pass per token: pull the top-k expert outputs from their ranks (up to 32
//              independent 16-byte NVLink loads in flight per thread), weight by the gate
//              probability, accumulate in fp32, write bf16
// Both communication kernels are persistent (one CTA per SM at most), open and close with a bounded
// peer barrier on per-CTA flags in the symmetric heap, and can emulate all ranks in one launch.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "gemm_api.h"
#include "gemm_epilogue.cuh"
#include "gemm_pipeline.cuh"
#include "gemm_pipeline2.cuh"
#include "moe_api.h"
#include "prims.cuh"
#include "tensormap.h"

namespace pccl {

namespace {

using namespace dev;

__device__ __forceinline__ uint64_t* moe_flag(const World& W, int owner, int lane, int block, int src) {
  return reinterpret_cast<uint64_t*>(W.heap[owner] + W.flag_off) +
         ((static_cast<uint64_t>(lane) * kMaxBlocksPerColl + block) * kMaxRanks + src);
}

__device__ __forceinline__ bool moe_barrier(const MoeArgs& A, int me, uint64_t value, uint32_t* s_fail) {
  __syncthreads();
  if (threadIdx.x < static_cast<uint32_t>(A.w.world)) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(moe_flag(A.w, p, A.flag_lane, blockIdx.x, me), value);
    if (!wait_ge(moe_flag(A.w, me, A.flag_lane, blockIdx.x, p), value, A.spin_ns, nullptr)) {
      *s_fail = 1;
      report(A.status[A.nvirt > 1 ? me : 0], ST_TIMEOUT, blockIdx.x, static_cast<uint32_t>(p), static_cast<uint32_t>(value & 3));
    }
  }
  __syncthreads();
  return *s_fail == 0;
}

// Quantises 8 bf16 values with a given inverse scale into 8 e4m3 bytes.
__device__ __forceinline__ uint2 quant8(const float* f, float inv) {
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * h] * inv, f[4 * h + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * h + 2] * inv, f[4 * h + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    w[h] = (lo & 0xffffu) | (hi << 16);
  }
  return make_uint2(w[0], w[1]);
}

// Quantise one row held in global memory into shared memory (q: hidden bytes, s: hidden/128 floats).
// 16 consecutive lanes own one 128-value block, so the block amax is a half-warp shuffle reduction.
__device__ __forceinline__ void quant_row_to_smem(const __nv_bfloat16* x, int hidden, uint8_t* q, float* s, int tid = threadIdx.x,
                                                  int nthreads = blockDim.x) {
  const int nvec = hidden >> 3;
  for (int v = tid; v < ((nvec + 31) & ~31); v += nthreads) {     // warp-uniform trip count for the shuffles
    float f[8];
    float amax = 0.f;
    if (v < nvec) {
      unpack<DT_BF16>(ld16(x + v * 8), f);
#pragma unroll
      for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(f[k]));
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
    if (v < nvec) {
      *reinterpret_cast<uint2*>(q + v * 8) = quant8(f, 1.0f / scale);
      if ((v & 15) == 0) s[v >> 4] = scale;
    }
  }
}

// A token is a chain of dependent steps (load the row, block maxima, quantise, store), a few microseconds long whatever the
// bandwidth; one token at a time per SM leaves both HBM and NVLink idle most of the time.  So a CTA is kDispatchSubs groups
// of 256 threads, each with its own staging row and its own named barrier, working on different tokens.
constexpr int kDispatchSubs = 3, kCombineSubs = 2;
__device__ __forceinline__ void sub_sync(int sub) { asm volatile("bar.sync %0, 256;" ::"r"(sub + 1) : "memory"); }
__host__ __device__ inline size_t dispatch_stage_bytes(int hidden) { return (static_cast<size_t>(hidden) + (hidden >> 7) * 4 + 15) / 16 * 16; }

__global__ void __launch_bounds__(256 * kDispatchSubs) moe_dispatch_kernel(const __grid_constant__ MoeArgs A) {
  extern __shared__ __align__(16) uint8_t dsm[];
  __shared__ uint32_t s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const int me = A.nvirt > 1 ? static_cast<int>(blockIdx.y) : A.rank;
  const int slot = A.nvirt > 1 ? me : 0;
  const int H = A.hidden, G = H >> 7;
  const int sub = threadIdx.x >> 8, tid = threadIdx.x & 255;
  uint8_t* q = dsm + sub * dispatch_stage_bytes(H);
  float* s = reinterpret_cast<float*>(q + H);
  if (!moe_barrier(A, me, 4 * A.epoch + 1, &s_fail)) return;
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(A.x[slot]);
  const int qvec = H >> 4, svec = (G + 3) >> 2;       // 16-byte vectors of payload / of scales
  for (int t = blockIdx.x * kDispatchSubs + sub; t < A.tokens; t += gridDim.x * kDispatchSubs) {
    sub_sync(sub);                                      // the previous token's stores have read the staging row
    quant_row_to_smem(x + static_cast<long long>(t) * H, H, q, s, tid, 256);
    sub_sync(sub);
    // destination rank and row of every assignment; with de-duplication, the primary of each (first k to that rank)
    int dest[8], prim[8];
    long long rowk[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      dest[k] = -1; prim[k] = k; rowk[k] = -1;
      if (k < A.topk) {
        const int e = A.expert_ids[slot][t * A.topk + k];
        rowk[k] = A.dst_rows[slot][t * A.topk + k];
        if (e >= 0 && rowk[k] >= 0) dest[k] = e / A.experts_per_rank;
      }
    }
    const bool dedupe = A.dedupe && A.alias_off && !A.probs[slot];      // scaled payloads differ per destination
    if (dedupe) {
#pragma unroll
      for (int k = 1; k < 8; ++k)
#pragma unroll
        for (int j = k - 1; j >= 0; --j)
          if (dest[k] >= 0 && dest[j] == dest[k]) prim[k] = prim[j];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (dest[k] < 0) continue;                        // dropped assignment (receive buffer full), or k >= topk
      const long long row = rowk[k];
      char* base = A.w.heap[dest[k]];
      if (A.alias_off && tid == 0) reinterpret_cast<int*>(base + A.alias_off)[row] = static_cast<int>(rowk[prim[k]]);
      if (prim[k] != k) continue;                       // the payload is already on its way to that rank
      if (dedupe && A.group_off && tid < 16) {
        // group record of this primary: the token's rows on that rank and their gate weights
        const int j = tid & 7;
        const bool member = dest[j] == dest[k] && prim[j] == k;
        uint32_t word;
        if (tid < 8) word = member ? static_cast<uint32_t>(rowk[j]) : 0xffffffffu;
        else word = __float_as_uint(member && A.gate[slot] ? A.gate[slot][t * A.topk + j] : 0.f);
        reinterpret_cast<uint32_t*>(base + A.group_off + row * 64)[tid] = word;
      }
      char* dq = base + A.recv_q_off + row * H;
      char* ds = base + A.recv_s_off + row * G * 4;
      for (int v = tid; v < qvec; v += 256) st16(dq + v * 16, *reinterpret_cast<const Vec16*>(q + v * 16));
      // With gate weights attached, destination k receives p[t,k] * x[t] (the gradient of an expert's output row in
      // the backward pass): the e4m3 payload is the same for every destination, only the block scales are multiplied.
      const float pk = A.probs[slot] ? A.probs[slot][t * A.topk + k] : 1.0f;
      if (tid < svec) {
        if ((G & 3) == 0 && !A.probs[slot]) st16(ds + tid * 16, *reinterpret_cast<const Vec16*>(reinterpret_cast<uint8_t*>(s) + tid * 16));
        else for (int i = tid * 4; i < min(G, tid * 4 + 4); ++i) reinterpret_cast<float*>(ds)[i] = s[i] * pk;
      }
    }
  }
  moe_barrier(A, me, 4 * A.epoch + 2, &s_fail);
}

// Two groups of 256 threads per CTA, each pulling a different token's rows: twice the loads in flight per SM (the register
// budget of 16 vectors in flight per thread allows no more).
__global__ void __launch_bounds__(256 * kCombineSubs) moe_combine_kernel(const __grid_constant__ MoeArgs A) {
  __shared__ uint32_t s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const int me = A.nvirt > 1 ? static_cast<int>(blockIdx.y) : A.rank;
  const int slot = A.nvirt > 1 ? me : 0;
  const int H = A.hidden, nvec = H >> 3;
  const int sub = threadIdx.x >> 8, tid = threadIdx.x & 255;
  if (!moe_barrier(A, me, 4 * A.epoch + 1, &s_fail)) return;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(A.out[slot]);
  for (int t = blockIdx.x * kCombineSubs + sub; t < A.tokens; t += gridDim.x * kCombineSubs) {
    const char* src[8];
    float p[8];
    int dest[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      src[k] = nullptr;
      p[k] = 0.f;
      dest[k] = -1;
      if (k < A.topk) {
        const int e = A.expert_ids[slot][t * A.topk + k];
        const long long row = A.dst_rows[slot][t * A.topk + k];
        if (e >= 0 && row >= 0) {
          dest[k] = e / A.experts_per_rank;
          src[k] = A.w.heap[dest[k]] + A.y_off + row * H * 2;
          p[k] = A.probs[slot][t * A.topk + k];
        }
      }
    }
    if (A.dedupe && A.z_off) {
      // one row per (token, rank): the first assignment to a rank stands for the token's whole group there; a group of two
      // or more has been summed (with its weights) into z on that rank, a group of one is still the plain expert output
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (dest[k] < 0) continue;
        bool first = true;
        int size = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (dest[j] == dest[k]) {
            ++size;
            if (j < k) first = false;
          }
        }
        if (!first) src[k] = nullptr;
        else if (size > 1) {
          src[k] = src[k] - A.y_off + A.z_off;
          p[k] = 1.0f;
        }
      }
    }
    for (int v0 = tid; v0 < nvec; v0 += 2 * 256) {
      const int v1 = v0 + 256;
      Vec16 a[8], b[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {        // all loads first: up to 16 NVLink loads in flight per thread
        if (src[k]) {
          a[k] = ld16(src[k] + v0 * 16);
          if (v1 < nvec) b[k] = ld16(src[k] + v1 * 16);
        }
      }
      float acc0[8] = {0, 0, 0, 0, 0, 0, 0, 0}, acc1[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (src[k]) {
          float f[8];
          unpack<DT_BF16>(a[k], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc0[j] += p[k] * f[j];
          if (v1 < nvec) {
            unpack<DT_BF16>(b[k], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc1[j] += p[k] * f[j];
          }
        }
      }
      st16(out + static_cast<long long>(t) * H + v0 * 8, pack<DT_BF16>(acc0));
      if (v1 < nvec) st16(out + static_cast<long long>(t) * H + v1 * 8, pack<DT_BF16>(acc1));
    }
  }
  moe_barrier(A, me, 4 * A.epoch + 2, &s_fail);
}

// dot[t,k] = <g[t], y[rank of expert (t,k)][dst_rows[t,k]]>: the gradient of the gate weight of an assignment, which is
// the upstream gradient of the token times the expert's output row.  The rows are pulled like in the combine.
__global__ void __launch_bounds__(256) moe_combine_dot_kernel(const __grid_constant__ MoeArgs A) {
  __shared__ uint32_t s_fail;
  __shared__ float part[8][8];
  if (threadIdx.x == 0) s_fail = 0;
  const int me = A.nvirt > 1 ? static_cast<int>(blockIdx.y) : A.rank;
  const int slot = A.nvirt > 1 ? me : 0;
  const int H = A.hidden, nvec = H >> 3;
  if (!moe_barrier(A, me, 4 * A.epoch + 1, &s_fail)) return;
  const __nv_bfloat16* g = static_cast<const __nv_bfloat16*>(A.x[slot]);
  float* dot = static_cast<float*>(A.out[slot]);
  for (int t = blockIdx.x; t < A.tokens; t += gridDim.x) {
    const char* src[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      src[k] = nullptr;
      if (k < A.topk) {
        const int e = A.expert_ids[slot][t * A.topk + k];
        const long long row = A.dst_rows[slot][t * A.topk + k];
        if (e >= 0 && row >= 0) src[k] = A.w.heap[e / A.experts_per_rank] + A.y_off + row * H * 2;
      }
    }
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      Vec16 a[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (src[k]) a[k] = ld16(src[k] + v * 16);
      float gf[8];
      unpack<DT_BF16>(ld16(g + static_cast<long long>(t) * H + v * 8), gf);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (src[k]) {
          float f[8];
          unpack<DT_BF16>(a[k], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[k] += gf[j] * f[j];
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], o);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
      for (int k = 0; k < 8; ++k) part[threadIdx.x >> 5][k] = acc[k];
    }
    __syncthreads();
    if (threadIdx.x < static_cast<uint32_t>(A.topk)) {
      float sum = 0.f;
      for (int w = 0; w < 8; ++w) sum += part[w][threadIdx.x];
      dot[t * A.topk + threadIdx.x] = sum;
    }
  }
  moe_barrier(A, me, 4 * A.epoch + 2, &s_fail);
}

__global__ void __launch_bounds__(256) moe_dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales,
                                                          __nv_bfloat16* __restrict__ out, const int* __restrict__ n_rows,
                                                          int max_rows, int hidden, const int* __restrict__ alias) {
  const int rows = min(*n_rows, max_rows);
  const int nvec = hidden >> 4, G = hidden >> 7;      // 16 fp8 values per 16-byte vector
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    long long from = r;
    if (alias) {                                        // a de-duplicated row: its payload sits in the token's primary row
      const int a = alias[r];
      if (a >= 0 && a < max_rows) from = a;
    }
    const uint8_t* qr = q + from * hidden;
    const float* sr = scales + from * G;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[16];
      unpack<DT_FP8_E4M3>(ld16(qr + v * 16), f);
      const float sc = sr[v >> 3];
#pragma unroll
      for (int k = 0; k < 16; ++k) f[k] *= sc;
      st16(out + r * hidden + v * 16, pack<DT_BF16>(f));
      st16(out + r * hidden + v * 16 + 8, pack<DT_BF16>(f + 8));
    }
  }
}

// z[r] = sum_j weight_j * y[row_j] over the group record of primary row r, for groups of two or more (a group of one stays in y
// and gets its weight in the combine).  Element-wise over the row, accumulated in fp32.
__global__ void __launch_bounds__(256) moe_reduce_groups_kernel(const __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ z,
                                                                const int* __restrict__ alias, const uint32_t* __restrict__ groups,
                                                                const int* __restrict__ n_rows, int max_rows, int hidden) {
  const int rows = min(*n_rows, max_rows);
  const int nvec = hidden >> 3;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    if (alias[r] != static_cast<int>(r)) continue;
    const uint32_t* g = groups + r * 16;
    int member[8];
    float w[8];
    int size = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int m = static_cast<int>(g[j]);
      member[j] = (m >= 0 && m < max_rows) ? m : -1;
      w[j] = __uint_as_float(g[8 + j]);
      size += member[j] >= 0;
    }
    if (size < 2) continue;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      Vec16 a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (member[j] >= 0) a[j] = ld16(y + static_cast<long long>(member[j]) * hidden + v * 8);
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (member[j] >= 0) {
          float f[8];
          unpack<DT_BF16>(a[j], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += w[j] * f[i];
        }
      }
      st16(z + r * hidden + v * 8, pack<DT_BF16>(acc));
    }
  }
}

__global__ void __launch_bounds__(256) quant_rows_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                         float* __restrict__ scales, long long rows, int hidden) {
  extern __shared__ __align__(16) uint8_t qsm[];
  uint8_t* sq = qsm;
  float* ss = reinterpret_cast<float*>(qsm + hidden);
  const int G = hidden >> 7;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    __syncthreads();
    quant_row_to_smem(x + r * hidden, hidden, sq, ss);
    __syncthreads();
    for (int v = threadIdx.x; v < (hidden >> 4); v += blockDim.x) st16(q + r * hidden + v * 16, *reinterpret_cast<const Vec16*>(sq + v * 16));
    for (int g = threadIdx.x; g < G; g += blockDim.x) scales[r * G + g] = ss[g];
  }
}

// one CTA per 128 x 128 block of a weight matrix
__global__ void __launch_bounds__(256) quant_blocks_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                                                           float* __restrict__ scales, int rows, int cols) {
  __shared__ float red[8];
  const int bc = blockIdx.x, br = blockIdx.y;
  const __nv_bfloat16* base = w + static_cast<long long>(br) * 128 * cols + bc * 128;
  float f[8][8];
  float amax = 0.f;
  // 128 x 128 values = 2048 vectors of 8; 256 threads take 8 each: thread -> (row group, vector in row)
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = threadIdx.x + i * 256, r = idx >> 4, v = idx & 15;
    unpack<DT_BF16>(ld16(base + static_cast<long long>(r) * cols + v * 8), f[i]);
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(f[i][k]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float scale = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
  if (threadIdx.x == 0) scales[br * (cols >> 7) + bc] = scale;
  const float inv = 1.0f / scale;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = threadIdx.x + i * 256, r = idx >> 4, v = idx & 15;
    *reinterpret_cast<uint2*>(q + (static_cast<long long>(br) * 128 + r) * cols + bc * 128 + v * 8) = quant8(f[i], inv);
  }
}

// ---------------------------------------------------------------------------------------------
// grouped GEMM on the tcgen05 pipeline
// ---------------------------------------------------------------------------------------------
using namespace gemm;

// Both schedulers walk the concatenated per-group tile lists.  A role asks for its tiles in increasing order, so each keeps a
// cursor (group, tiles before it) instead of scanning the groups from the start for every tile: the scan is a chain of
// dependent loads, and the MMA warp's share of it would sit between two tiles with the tensor cores idle.
struct GroupedSched {
  const int* row_off;    // groups + 1
  int groups, tiles_n, first, stride;
  int tile_rows;         // 128 (single CTA) or 256 (CTA pair)
  mutable int cur_g = 0;
  mutable long long cur_base = 0;
  // Tile `idx` of the concatenated per-group tile lists -> (group, m-tile inside group, n-tile).
  __device__ __forceinline__ bool get(int it, TileCoord* t) const {
    const long long idx = first + static_cast<long long>(it) * stride;
    while (cur_g < groups) {
      const int rows = row_off[cur_g + 1] - row_off[cur_g];
      const int tm = (rows + tile_rows - 1) / tile_rows;
      const long long tiles = static_cast<long long>(tm) * tiles_n;
      if (idx - cur_base < tiles) {
        const int local = static_cast<int>(idx - cur_base);
        t->m = local % tm;
        t->n = local / tm;
        t->extra = cur_g;
        return true;
      }
      cur_base += tiles;
      ++cur_g;
    }
    return false;
  }
};

struct GroupedEpi {
  __nv_bfloat16* D;
  long long ldd;
  const int* row_off;
  int N;
  uint32_t flags;
  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return row_off[t.extra] + t.m * BM; }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return t.extra * N + t.n * BN; }
  __device__ __forceinline__ void attach_smem(uint8_t*) {}
  __device__ __forceinline__ void tile_begin(const TileCoord&) {}
  __device__ __forceinline__ void tile_done(const TileCoord&, const volatile uint32_t*) {}
  __device__ __forceinline__ void strip(const TileCoord& t, int row_in_tile, int col_in_tile, uint32_t* r) {
    const int row = row_off[t.extra] + t.m * BM + row_in_tile;
    const int col = t.n * BN + col_in_tile;
    if (row >= row_off[t.extra + 1] || col >= N) return;     // rows past the group's end belong to the next group
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    if (flags & GEMM_GELU_INPLACE) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
    }
    __nv_bfloat16* d = D + static_cast<long long>(row) * ldd + col;
    if (col + 32 <= N) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) st16(d + i, pack<DT_BF16>(v + i));
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col + i < N) d[i] = __float2bfloat16_rn(v[i]);
    }
  }
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GroupedEpi epi, int groups, int K,
                    uint32_t* status) {
  GroupedSched sched{epi.row_off, groups, (epi.N + BN - 1) / BN, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), BM};
  NoGate gate;
  run<false, false>(&tmA, &tmB, K, sched, gate, epi, status);
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_grouped_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GroupedEpi epi, int groups, int K,
                         uint32_t* status) {
  GroupedSched sched{epi.row_off, groups, (epi.N + BN - 1) / BN, static_cast<int>(blockIdx.x >> 1), static_cast<int>(gridDim.x >> 1), 2 * BM};
  NoGate gate;
  const int cta = static_cast<int>(tc::cluster_ctarank());
  gemm2::PairEpi<GroupedEpi> pe{epi, cta};
  gemm2::PairGate<NoGate> pg{gate, cta};
  gemm2::run<false, false>(&tmA, &tmB, K, sched, pg, pe, status);
}

// The same product with the operands exchanged: the weights of a group are the M side of the tile (whole 256-row tiles, their
// count is a multiple of 256) and the group's rows are the N side, whose extent the MMA instruction takes per tile in steps
// of 16.  A group of 520 rows then costs 2 + 8/256 tiles of tensor time per weight tile, where the row-major form above pays
// for 3: with a few hundred rows per expert that is a fifth of the whole product.  The accumulator arrives transposed (lane =
// output feature, column = row of the group), so a warp stores 32 consecutive features of one row per instruction.
struct RaggedSched {
  const int* row_off;
  int groups, tiles_f, first, stride;        // tiles_f = N / 256 weight tiles per group
  mutable int cur_g = 0;
  mutable long long cur_base = 0;
  __device__ __forceinline__ bool get(int it, TileCoord* t) const {
    const long long idx = first + static_cast<long long>(it) * stride;
    while (cur_g < groups) {
      const int rows = row_off[cur_g + 1] - row_off[cur_g];
      const int tr = (rows + 255) / 256;
      const long long tiles = static_cast<long long>(tr) * tiles_f;
      if (idx - cur_base < tiles) {
        const int local = static_cast<int>(idx - cur_base);
        t->m = local / tr;                     // weight tile; the row tiles of one weight tile are neighbours in the list
        t->n = local % tr;
        t->extra = cur_g;
        return true;
      }
      cur_base += tiles;
      ++cur_g;
    }
    return false;
  }
};

struct RaggedEpi {
  static constexpr bool kVarN = true;
  __nv_bfloat16* D;
  long long ldd;
  const int* row_off;
  int N;             // output features per group
  uint32_t flags;
  int cta;
  __device__ __forceinline__ int tile_n(const TileCoord& t) const {
    const int left = row_off[t.extra + 1] - row_off[t.extra] - t.n * 256;
    return left >= 256 ? 256 : ((left + 15) & ~15);
  }
  // A operand: this CTA's 128 weight rows; B operand: this CTA's half of the tile's rows
  // descriptor whose box holds 128 >> b_box rows: the smallest that covers this CTA's tile_n / 2 rows
  __device__ __forceinline__ int b_box(const TileCoord& t) const {
    const int half = tile_n(t) >> 1;
    return half > 64 ? 0 : half > 32 ? 1 : half > 16 ? 2 : half > 8 ? 3 : 4;
  }
  __device__ __forceinline__ int a_row0(const TileCoord& t) const { return t.extra * N + t.m * 256 + cta * 128; }
  __device__ __forceinline__ int b_row0(const TileCoord& t) const { return row_off[t.extra] + t.n * 256 + cta * (tile_n(t) >> 1); }
  __device__ __forceinline__ void attach_smem(uint8_t*) {}
  __device__ __forceinline__ void tile_begin(const TileCoord&) {}
  __device__ __forceinline__ void tile_done(const TileCoord&, const volatile uint32_t*) {}
  // The lane holds 32 rows of ONE feature; its neighbours hold the next features of the same rows.  Two exchange steps
  // (lane ^ 1, lane ^ 2) regroup that into 4 consecutive features of one row per lane, so a strip leaves as 8 stores of 8 bytes
  // per lane instead of 32 of 2: lanes 4q..4q+3 then cover rows 4j+0..3 of features 4q..4q+3.
  __device__ __forceinline__ void strip(const TileCoord& t, int feat_in_cta, int col0, uint32_t* r) {
    const int lane = feat_in_cta & 31;
    const int feat4 = t.m * 256 + cta * 128 + (feat_in_cta & ~3);
    const int row0 = row_off[t.extra] + t.n * 256 + col0;
    const int n_valid = row_off[t.extra + 1] - row0;          // rows of this strip that belong to the group (may exceed 32)
    const bool gelu = flags & GEMM_GELU_INPLACE;
    const bool odd1 = lane & 1, odd2 = lane & 2;
    uint32_t p[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float a = __uint_as_float(r[2 * j]), b = __uint_as_float(r[2 * j + 1]);
      if (gelu) { a = gelu_tanh(a); b = gelu_tanh(b); }
      const float got = __shfl_xor_sync(0xffffffffu, odd1 ? a : b, 1);
      // even lane: row 2j, features (f, f+1) = (own a, neighbour's a); odd lane: row 2j+1, features (f-1, f) = (neighbour's b, own b)
      const __nv_bfloat162 v = odd1 ? __floats2bfloat162_rn(got, b) : __floats2bfloat162_rn(a, got);
      p[j] = *reinterpret_cast<const uint32_t*>(&v);
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      const uint32_t got = __shfl_xor_sync(0xffffffffu, odd2 ? p[2 * m] : p[2 * m + 1], 2);
      // bit 1 clear: keeps pair-row 2m, features +0..1 own, +2..3 from lane ^ 2; bit 1 set: keeps pair-row 2m+1
      const uint2 out = odd2 ? make_uint2(got, p[2 * m + 1]) : make_uint2(p[2 * m], got);
      const int row = 2 * (2 * m + (odd2 ? 1 : 0)) + (odd1 ? 1 : 0);
      if (row < n_valid)
        *reinterpret_cast<uint2*>(D + static_cast<long long>(row0 + row) * ldd + feat4) = out;
    }
  }
};

struct RaggedMaps { CUtensorMap x[5]; };     // boxes of 128, 64, 32, 16, 8 rows

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_grouped_ragged_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ RaggedMaps tmX, RaggedEpi epi, int groups, int K,
                           uint32_t* status) {
  RaggedSched sched{epi.row_off, groups, epi.N / 256, static_cast<int>(blockIdx.x >> 1), static_cast<int>(gridDim.x >> 1)};
  NoGate gate;
  epi.cta = static_cast<int>(tc::cluster_ctarank());
  gemm2::run<false, false>(&tmW, tmX.x, K, sched, gate, epi, status);
}

// ---------------------------------------------------------------------------------------------
// routing and placement
// ---------------------------------------------------------------------------------------------
template <int PER_LANE>
__global__ void __launch_bounds__(256) moe_route_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ probs,
                                                        int* __restrict__ pos, int* __restrict__ counts, int tokens, int experts, int topk) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  float v[PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = j * 32 + lane;
    v[j] = e < experts ? logits[static_cast<long long>(t) * experts + e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    v[j] = __expf(v[j] - mx);
    sum += v[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  for (int k = 0; k < topk; ++k) {
    float best = -1.f;
    int bi = 0;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j)
      if (v[j] > best) { best = v[j]; bi = j * 32 + lane; }
    // warp arg-max; ties go to the lower expert id (what a stable top-k returns)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int j = 0; j < PER_LANE; ++j)
        if (j == (bi >> 5)) v[j] = -2.f;       // taken
      ids[t * topk + k] = bi;
      probs[t * topk + k] = best * inv;
      pos[t * topk + k] = atomicAdd(counts + bi, 1);
    }
  }
}

__global__ void __launch_bounds__(256) moe_plan_kernel(const int* __restrict__ counts_all, const int* __restrict__ ids, const int* __restrict__ pos,
                                                       int* __restrict__ rows, int* __restrict__ row_off, int world, int rank, int experts,
                                                       int tokens, int topk, int cap) {
  extern __shared__ int base[];            // experts entries: first row of (this rank's assignments to e) on e's rank
  const int epr = experts / world;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int owner = e / epr;
    int before = 0;                        // rows of the owner's earlier experts
    for (int e2 = owner * epr; e2 < e; ++e2)
      for (int r = 0; r < world; ++r) before += counts_all[r * experts + e2];
    for (int r = 0; r < rank; ++r) before += counts_all[r * experts + e];     // lower ranks inside the expert's segment
    base[e] = before;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i <= epr; i += blockDim.x) {
      int acc = 0;
      for (int e2 = rank * epr; e2 < rank * epr + i; ++e2)
        for (int r = 0; r < world; ++r) acc += counts_all[r * experts + e2];
      row_off[i] = min(acc, cap);
    }
  }
  const int total = tokens * topk;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int row = base[ids[i]] + pos[i];
    rows[i] = row < cap ? row : -1;
  }
}

template <typename K>
int coop(K kernel, const MoeArgs& a, int blocks, size_t smem, cudaStream_t stream, int threads = 256) {
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocksPerColl) blocks = kMaxBlocksPerColl;
  if (a.topk > 8 || a.hidden % 128 || a.flag_lane < 0 || a.flag_lane >= 8) return static_cast<int>(cudaErrorInvalidValue);
  dim3 grid(blocks, a.nvirt > 1 ? a.nvirt : 1), block(threads);
  void* args[] = {const_cast<MoeArgs*>(&a)};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), grid, block, args, smem, stream));
}

}  // namespace

int launchMoeDispatch(const MoeArgs& a, int blocks, cudaStream_t stream) {
  const size_t smem = kDispatchSubs * dispatch_stage_bytes(a.hidden);
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(moe_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    smem_set = smem;
  }
  return coop(moe_dispatch_kernel, a, blocks, smem, stream, 256 * kDispatchSubs);
}

int launchMoeCombine(const MoeArgs& a, int blocks, cudaStream_t stream) {
  return coop(moe_combine_kernel, a, blocks, 0, stream, 256 * kCombineSubs);
}
int launchMoeCombineDot(const MoeArgs& a, int blocks, cudaStream_t stream) { return coop(moe_combine_dot_kernel, a, blocks, 0, stream); }

int launchMoeDequant(const void* q, const float* scales, void* out, const int* n_rows, int max_rows, int hidden, const int* alias,
                     cudaStream_t stream) {
  if (hidden % 128) return static_cast<int>(cudaErrorInvalidValue);
  moe_dequant_kernel<<<148 * 8, 256, 0, stream>>>(static_cast<const uint8_t*>(q), scales, static_cast<__nv_bfloat16*>(out), n_rows, max_rows, hidden,
                                                  alias);
  return static_cast<int>(cudaGetLastError());
}

int launchMoeReduceGroups(const void* y, void* z, const int* alias, const void* groups, const int* n_rows, int max_rows, int hidden,
                          cudaStream_t stream) {
  if (hidden % 8 || !alias || !groups) return static_cast<int>(cudaErrorInvalidValue);
  moe_reduce_groups_kernel<<<148 * 8, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(z), alias,
                                                        static_cast<const uint32_t*>(groups), n_rows, max_rows, hidden);
  return static_cast<int>(cudaGetLastError());
}

int launchQuantFp8Rows(const void* x, void* q, float* scales, long long rows, int hidden, cudaStream_t stream) {
  if (hidden % 128 || rows <= 0) return static_cast<int>(cudaErrorInvalidValue);
  long long blocks = rows < 148 * 8 ? rows : 148 * 8;
  quant_rows_kernel<<<static_cast<int>(blocks), 256, static_cast<size_t>(hidden) + (hidden >> 7) * 4 + 16, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scales, rows, hidden);
  return static_cast<int>(cudaGetLastError());
}

int launchQuantFp8Blocks(const void* w, void* q, float* scales, int rows, int cols, cudaStream_t stream) {
  if (rows % 128 || cols % 128 || rows <= 0 || cols <= 0) return static_cast<int>(cudaErrorInvalidValue);
  dim3 grid(cols / 128, rows / 128);
  quant_blocks_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q), scales, rows, cols);
  return static_cast<int>(cudaGetLastError());
}

int launchMoeRoute(const float* logits, int* ids, float* probs, int* pos, int* counts, int tokens, int experts, int topk,
                   cudaStream_t stream) {
  if (experts < 1 || experts > 1024 || topk > experts || tokens <= 0) return static_cast<int>(cudaErrorInvalidValue);
  const int grid = (tokens + 7) / 8;
  const int per = (experts + 31) / 32;
  if (per <= 4) moe_route_kernel<4><<<grid, 256, 0, stream>>>(logits, ids, probs, pos, counts, tokens, experts, topk);
  else if (per <= 8) moe_route_kernel<8><<<grid, 256, 0, stream>>>(logits, ids, probs, pos, counts, tokens, experts, topk);
  else if (per <= 16) moe_route_kernel<16><<<grid, 256, 0, stream>>>(logits, ids, probs, pos, counts, tokens, experts, topk);
  else moe_route_kernel<32><<<grid, 256, 0, stream>>>(logits, ids, probs, pos, counts, tokens, experts, topk);
  return static_cast<int>(cudaGetLastError());
}

int launchMoePlan(const int* counts_all, const int* ids, const int* pos, int* rows, int* row_off, int world, int rank, int experts,
                  int tokens, int topk, int cap, cudaStream_t stream) {
  if (experts % world || tokens <= 0) return static_cast<int>(cudaErrorInvalidValue);
  int grid = (tokens * topk + 255) / 256;
  if (grid > 148) grid = 148;
  moe_plan_kernel<<<grid, 256, experts * sizeof(int), stream>>>(counts_all, ids, pos, rows, row_off, world, rank, experts, tokens, topk, cap);
  return static_cast<int>(cudaGetLastError());
}

int gemmGroupedBf16(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, const int* row_off,
                    int groups, int max_rows, int N, int K, uint32_t flags, int sms, uint32_t* status, cudaStream_t stream) {
  if (groups <= 0 || max_rows <= 0) return 0;
  if ((lda | ldb | ldd) % 8) return static_cast<int>(cudaErrorInvalidValue);
  CUtensorMap ta, tb;
  std::string err;
  if (!makeTensorMap2D(&ta, A, TM_BF16, K, max_rows, lda, BK, BM, &err)) return static_cast<int>(cudaErrorInvalidValue);
  int n_sm = deviceSmCount();
  if (sms > 0 && sms < n_sm) n_sm = sms;
  GroupedEpi epi{static_cast<__nv_bfloat16*>(D), ldd, row_off, N, flags};
  static const bool ragged_on = !(std::getenv("PCCL_GROUPED_RAGGED") && std::getenv("PCCL_GROUPED_RAGGED")[0] == '0');
  if (N % 256 == 0 && n_sm >= 2 && ragged_on) {
    // operands exchanged: weights on the M side, the groups' rows on an N side that is cut to the rows there are
    CUtensorMap tw;
    RaggedMaps tx;
    if (!makeTensorMap2D(&tw, B, TM_BF16, K, static_cast<uint64_t>(groups) * N, ldb, BK, 128, &err)) return static_cast<int>(cudaErrorInvalidValue);
    for (int i = 0; i < 5; ++i)
      if (!makeTensorMap2D(&tx.x[i], A, TM_BF16, K, max_rows, lda, BK, 128 >> i, &err)) return static_cast<int>(cudaErrorInvalidValue);
    static bool set3 = false;
    if (!set3) {
      cudaError_t e = cudaFuncSetAttribute(gemm_grouped_ragged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm2::SMEM_BYTES);
      if (e != cudaSuccess) return static_cast<int>(e);
      set3 = true;
    }
    RaggedEpi repi{static_cast<__nv_bfloat16*>(D), ldd, row_off, N, flags, 0};
    return static_cast<int>(gemm2::launch_pairs(gemm_grouped_ragged_kernel, dim3(n_sm & ~1), NUM_THREADS, gemm2::SMEM_BYTES, stream, false, tw, tx,
                                                repi, groups, K, status));
  }
  if (N % 256 == 0 && n_sm >= 2) {       // CTA pairs: each CTA loads 128 of the 256 B rows of a tile
    if (!makeTensorMap2D(&tb, B, TM_BF16, K, static_cast<uint64_t>(groups) * N, ldb, BK, 128, &err)) return static_cast<int>(cudaErrorInvalidValue);
    static bool set2 = false;
    if (!set2) {
      cudaError_t e = cudaFuncSetAttribute(gemm_grouped_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm2::SMEM_BYTES);
      if (e != cudaSuccess) return static_cast<int>(e);
      set2 = true;
    }
    return static_cast<int>(gemm2::launch_pairs(gemm_grouped_pair_kernel, dim3(n_sm & ~1), NUM_THREADS, gemm2::SMEM_BYTES, stream, false, ta, tb,
                                                epi, groups, K, status));
  }
  if (!makeTensorMap2D(&tb, B, TM_BF16, K, static_cast<uint64_t>(groups) * N, ldb, BK, BN, &err)) return static_cast<int>(cudaErrorInvalidValue);
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    set = true;
  }
  gemm_grouped_kernel<<<n_sm, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, epi, groups, K, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace pccl
