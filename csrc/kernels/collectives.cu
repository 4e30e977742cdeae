// Hand-written collectives over the symmetric heap: all-reduce, reduce-scatter (+ scale/cast
// epilogue for gradient buckets), all-gather, all-to-all; P2P (ld/st over NVLink) and NVLS
// (multimem through the switch) forms.
//
// The reference has only the three multimem wrappers and no kernel that uses them
// (include/plugins/cuda_executor/utils/multimem.h:12-127).  These kernels are what its README
// bullets ("NVLS", "CUDA IPC") stand for, built for NVSwitch: every GPU reaches every peer at full
// port bandwidth, so each collective is one hop -- a rank pull-reduces (or ld_reduce's) its own
// slice from all peers and pushes (or multicast-stores) results -- instead of a ring.
//
// Synchronisation: CTA b of every rank shares one row of flags with CTA b of every other rank
// (flags[lane][b][source rank], uint64, in the symmetric heap).  A launch with epoch e uses values
// 4e+1 (entry) and 4e+2 (exit); values only grow, so nothing is ever cleared and a late flag
// from an old launch cannot release a newer wait.  Waits are bounded (see prims.cuh).
#include "api.h"
#include "prims.cuh"

namespace pccl {

using namespace dev;

namespace {

__device__ __forceinline__ uint64_t* flag_ptr(const World& W, int owner, int lane, int block, int src) {
  return reinterpret_cast<uint64_t*>(W.heap[owner] + W.flag_off) +
         ((static_cast<uint64_t>(lane) * kMaxBlocksPerColl + block) * kMaxRanks + src);
}

// Returns false (after recording ST_TIMEOUT) if some peer did not arrive in time.
__device__ __forceinline__ bool peer_barrier(const CollArgs& A, int me, uint64_t value, uint32_t* s_fail) {
  __syncthreads();
  if (threadIdx.x < static_cast<uint32_t>(A.w.world)) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(flag_ptr(A.w, p, A.flag_lane, blockIdx.x, me), value);
    if (!wait_ge(flag_ptr(A.w, me, A.flag_lane, blockIdx.x, p), value, A.spin_limit, nullptr)) {
      *s_fail = 1;
      report(A.status[A.nvirt > 1 ? me : 0], ST_TIMEOUT, blockIdx.x, static_cast<uint32_t>(p), static_cast<uint32_t>(value & 3));
    }
  }
  __syncthreads();
  return *s_fail == 0;
}

__device__ __forceinline__ int my_rank(const CollArgs& A) { return A.nvirt > 1 ? static_cast<int>(blockIdx.y) : A.rank; }

// Sum/max/min of vector i (16 bytes) of every rank's `in` at heap offset `off`, accumulated in fp32.
template <uint32_t DT, uint32_t OP>
__device__ __forceinline__ void pull_reduce(const CollArgs& A, int me, uint64_t off, float* acc) {
  constexpr int N = Lanes<DT>::n;
  const int n = A.w.world;
  // Peers are visited eight at a time with the loads fully unrolled and predicated, so the
  // vectors stay in registers and up to eight 16-byte NVLink loads are in flight per thread.
  for (int g = 0; g < n; g += 8) {
    Vec16 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (g + k < n) {
        int p = me + g + k;
        if (p >= n) p -= n;
        v[k] = ld16(A.w.heap[p] + off);
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (g + k < n) {
        if (g + k == 0) {
          unpack<DT>(v[0], acc);
        } else {
          float f[N];
          unpack<DT>(v[k], f);
#pragma unroll
          for (int j = 0; j < N; ++j) acc[j] = red1<OP>(acc[j], f[j]);
        }
      }
    }
  }
}

template <uint32_t DT, uint32_t OP>
__device__ __forceinline__ float pull_reduce1(const CollArgs& A, int me, uint64_t off) {
  float acc = load1<DT>(A.w.heap[me] + off);
  for (int k = 1; k < A.w.world; ++k) acc = red1<OP>(acc, load1<DT>(A.w.heap[(me + k) % A.w.world] + off));
  return acc;
}

// ---------------------------------------------------------------------------------------------
// all-reduce: two-shot (slice r is reduced by rank r and written to every rank's output)
// ---------------------------------------------------------------------------------------------
template <uint32_t DT, uint32_t OP, bool NVLS>
__global__ void __launch_bounds__(512) allreduce_kernel(const __grid_constant__ CollArgs A) {
  constexpr int N = Lanes<DT>::n;
  constexpr int ES = 16 / N;
  __shared__ uint32_t s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const int me = my_rank(A), n = A.w.world;
  if (!peer_barrier(A, me, 4 * A.epoch + 1, &s_fail)) return;

  const uint64_t bytes = A.count * ES;
  const uint64_t nvec = bytes >> 4;
  // A long vector is taken in 128 MiB segments, each split over the ranks: the slices that the ranks work on at
  // one time then lie within one segment instead of a whole vector apart (measured: above 256 MiB the all-at-once
  // split lost a fifth of its bandwidth on eight GPUs).  No synchronisation between segments is needed.
  const uint64_t seg = (128ull << 20) >> 4;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t s0 = 0; s0 < nvec; s0 += seg) {
    const uint64_t ns = min(seg, nvec - s0);
    const uint64_t per = (ns + n - 1) / n;
    const uint64_t lo = s0 + min(per * me, ns), hi = s0 + min(per * (me + 1), ns);
    uint64_t i = lo + static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if constexpr (NVLS && MultimemSupported<DT, OP>::value) {
      // four in-switch reductions in flight per thread before the first multicast store
      for (; i + 3 * stride < hi; i += 4 * stride) {
        Vec16 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) r[u] = multimem_ld_reduce<DT, OP>(A.w.mc_heap + A.in_off + ((i + u * stride) << 4));
#pragma unroll
        for (int u = 0; u < 4; ++u) multimem_st(A.w.mc_heap + A.out_off + ((i + u * stride) << 4), r[u]);
      }
      for (; i < hi; i += stride) multimem_st(A.w.mc_heap + A.out_off + (i << 4), multimem_ld_reduce<DT, OP>(A.w.mc_heap + A.in_off + (i << 4)));
    } else {
      for (; i + stride < hi; i += 2 * stride) {     // two vectors = up to 16 peer loads in flight per thread
        float acc0[N], acc1[N];
        pull_reduce<DT, OP>(A, me, A.in_off + (i << 4), acc0);
        pull_reduce<DT, OP>(A, me, A.in_off + ((i + stride) << 4), acc1);
        Vec16 r0 = pack<DT>(acc0), r1 = pack<DT>(acc1);
        for (int k = 0; k < n; ++k) {
          int p = me + k;
          if (p >= n) p -= n;
          st16(A.w.heap[p] + A.out_off + (i << 4), r0);
          st16(A.w.heap[p] + A.out_off + ((i + stride) << 4), r1);
        }
      }
      for (; i < hi; i += stride) {
        float acc[N];
        pull_reduce<DT, OP>(A, me, A.in_off + (i << 4), acc);
        Vec16 r = pack<DT>(acc);
        for (int k = 0; k < n; ++k) {
          int p = me + k;
          if (p >= n) p -= n;
          st16(A.w.heap[p] + A.out_off + (i << 4), r);
        }
      }
    }
  }
  // ragged tail (bytes not a multiple of 16): the last rank handles it element by element
  if (me == n - 1 && blockIdx.x == 0) {
    for (uint64_t b = (nvec << 4) + static_cast<uint64_t>(threadIdx.x) * ES; b + ES <= bytes; b += static_cast<uint64_t>(blockDim.x) * ES) {
      float r = pull_reduce1<DT, OP>(A, me, A.in_off + b);
      for (int p = 0; p < n; ++p) store1<DT>(A.w.heap[p] + A.out_off + b, r);
    }
  }
  peer_barrier(A, me, 4 * A.epoch + 2, &s_fail);
}

// one-shot: every rank reduces everything into its own output (out must not alias in)
template <uint32_t DT, uint32_t OP, bool NVLS>
__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const __grid_constant__ CollArgs A) {
  constexpr int N = Lanes<DT>::n;
  constexpr int ES = 16 / N;
  __shared__ uint32_t s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const int me = my_rank(A);
  if (!peer_barrier(A, me, 4 * A.epoch + 1, &s_fail)) return;
  const uint64_t bytes = A.count * ES;
  const uint64_t nvec = bytes >> 4;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  char* out = A.w.heap[me] + A.out_off;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const uint64_t o = i << 4;
    if constexpr (NVLS && MultimemSupported<DT, OP>::value) {
      st16(out + o, multimem_ld_reduce<DT, OP>(A.w.mc_heap + A.in_off + o));
    } else {
      float acc[N];
      pull_reduce<DT, OP>(A, me, A.in_off + o, acc);
      st16(out + o, pack<DT>(acc));
    }
  }
  if (blockIdx.x == 0)
    for (uint64_t b = (nvec << 4) + static_cast<uint64_t>(threadIdx.x) * ES; b + ES <= bytes; b += static_cast<uint64_t>(blockDim.x) * ES)
      store1<DT>(out + b, pull_reduce1<DT, OP>(A, me, A.in_off + b));
  peer_barrier(A, me, 4 * A.epoch + 2, &s_fail);
}

// ---------------------------------------------------------------------------------------------
// low-latency all-reduce (flag in the data): <= kLlMaxBytes, a multiple of 4 bytes; input and output may be any local
// tensors (also the same one); no barrier, one kernel, every wait bounded
// ---------------------------------------------------------------------------------------------
template <uint32_t DT, uint32_t OP>
__device__ __forceinline__ uint32_t ll_reduce_word(uint32_t a, uint32_t b) {
  if constexpr (DT == DT_F32) {
    return __float_as_uint(red1<OP>(__uint_as_float(a), __uint_as_float(b)));
  } else {
    // two 16-bit values per word: reduce in fp32, round once per step (the sum of at most 16 ranks)
    float a0 = load1<DT>(reinterpret_cast<const char*>(&a)), a1 = load1<DT>(reinterpret_cast<const char*>(&a) + 2);
    float b0 = load1<DT>(reinterpret_cast<const char*>(&b)), b1 = load1<DT>(reinterpret_cast<const char*>(&b) + 2);
    uint32_t r;
    store1<DT>(reinterpret_cast<char*>(&r), red1<OP>(a0, b0));
    store1<DT>(reinterpret_cast<char*>(&r) + 2, red1<OP>(a1, b1));
    return r;
  }
}

template <uint32_t DT, uint32_t OP>
__global__ void __launch_bounds__(512) allreduce_ll_kernel(const __grid_constant__ CollArgs A) {
  const int me = my_rank(A), n = A.w.world;
  const int slot = A.nvirt > 1 ? me : 0;
  const uint32_t words = static_cast<uint32_t>(A.count * (DT == DT_F32 ? 4 : 2) / 4);
  const uint32_t flag = static_cast<uint32_t>(A.epoch);                   // never 0: epochs start at 1
  const uint64_t area = A.ll_off + (A.epoch & 1) * (static_cast<uint64_t>(kMaxRanks) * kLlSlotBytes);
  const uint32_t* in = reinterpret_cast<const uint32_t*>(A.local_in[slot] ? A.local_in[slot] : A.w.heap[me] + A.in_off);
  uint32_t* out = reinterpret_cast<uint32_t*>(A.local_out[slot] ? static_cast<char*>(A.local_out[slot]) : A.w.heap[me] + A.out_off);
  const uint32_t stride = gridDim.x * blockDim.x, first = blockIdx.x * blockDim.x + threadIdx.x;
  // 1. every word to every peer's slot for this rank, flag attached (8-byte stores are single transactions)
  for (uint32_t w = first; w < words; w += stride) {
    const uint64_t pkt = (static_cast<uint64_t>(flag) << 32) | in[w];
    for (int k = 1; k < n; ++k) {
      int p = me + k;
      if (p >= n) p -= n;
      uint64_t* dst = reinterpret_cast<uint64_t*>(A.w.heap[p] + area + static_cast<uint64_t>(me) * kLlSlotBytes) + w;
      asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(pkt) : "memory");
    }
  }
  // 2. own word plus the peers' packets as they arrive
  bool failed = false;
  for (uint32_t w = first; w < words && !failed; w += stride) {
    uint32_t acc = in[w];
    for (int k = 1; k < n; ++k) {
      int p = me - k;
      if (p < 0) p += n;
      const uint64_t* src = reinterpret_cast<const uint64_t*>(A.w.heap[me] + area + static_cast<uint64_t>(p) * kLlSlotBytes) + w;
      uint64_t pkt = ld_relaxed_sys(src);
      if (static_cast<uint32_t>(pkt >> 32) != flag) {
        const uint64_t t0 = global_timer_ns();
        for (uint32_t i = 1;; ++i) {
          pkt = ld_relaxed_sys(src);
          if (static_cast<uint32_t>(pkt >> 32) == flag) break;
          if ((i & 63) == 0 && global_timer_ns() - t0 > A.spin_limit) { failed = true; break; }
        }
        if (failed) {
          report(A.status[slot], ST_TIMEOUT, blockIdx.x, static_cast<uint32_t>(p), 0x11u);
          break;
        }
      }
      acc = ll_reduce_word<DT, OP>(acc, static_cast<uint32_t>(pkt));
    }
    if (!failed) out[w] = acc;
  }
}

// ---------------------------------------------------------------------------------------------
// reduce-scatter with epilogue: out_r[i] = cast(scale * reduce_p in_p[r*count + i])
// ---------------------------------------------------------------------------------------------
template <uint32_t DT, uint32_t OP, bool NVLS, bool OUT_F32>
__global__ void __launch_bounds__(512) reduce_scatter_kernel(const __grid_constant__ CollArgs A) {
  constexpr int N = Lanes<DT>::n;
  constexpr int ES = 16 / N;
  __shared__ uint32_t s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const int me = my_rank(A);
  const int slot = A.nvirt > 1 ? me : 0;
  if (!peer_barrier(A, me, 4 * A.epoch + 1, &s_fail)) return;
  const uint64_t bytes = A.count * ES;
  const uint64_t nvec = bytes >> 4;
  const uint64_t base = A.in_off + static_cast<uint64_t>(me) * bytes;
  char* out = A.local_out[slot] ? static_cast<char*>(A.local_out[slot]) : A.w.heap[me] + A.out_off;
  const bool aligned = ((base | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const float scale = A.scale;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  const uint64_t gtid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  uint64_t done = 0;
  if (aligned) {
    auto finish = [&](uint64_t i, float* acc) {
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] *= scale;
      if constexpr (OUT_F32 && DT != DT_F32) {
        float* of = reinterpret_cast<float*>(out) + i * N;
#pragma unroll
        for (int j = 0; j < N; j += 4) {
          Vec16 r;
          r.w[0] = __float_as_uint(acc[j]); r.w[1] = __float_as_uint(acc[j + 1]);
          r.w[2] = __float_as_uint(acc[j + 2]); r.w[3] = __float_as_uint(acc[j + 3]);
          st16(of + j, r);
        }
      } else {
        st16(out + (i << 4), pack<DT>(acc));
      }
    };
    uint64_t i = gtid;
    if constexpr (NVLS && MultimemSupported<DT, OP>::value) {
      for (; i + 3 * stride < nvec; i += 4 * stride) {
        Vec16 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) r[u] = multimem_ld_reduce<DT, OP>(A.w.mc_heap + base + ((i + u * stride) << 4));
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float acc[N];
          unpack<DT>(r[u], acc);
          finish(i + u * stride, acc);
        }
      }
      for (; i < nvec; i += stride) {
        float acc[N];
        unpack<DT>(multimem_ld_reduce<DT, OP>(A.w.mc_heap + base + (i << 4)), acc);
        finish(i, acc);
      }
    } else {
      for (; i + stride < nvec; i += 2 * stride) {
        float acc0[N], acc1[N];
        pull_reduce<DT, OP>(A, me, base + (i << 4), acc0);
        pull_reduce<DT, OP>(A, me, base + ((i + stride) << 4), acc1);
        finish(i, acc0);
        finish(i + stride, acc1);
      }
      for (; i < nvec; i += stride) {
        float acc[N];
        pull_reduce<DT, OP>(A, me, base + (i << 4), acc);
        finish(i, acc);
      }
    }
    done = nvec << 4;
  }
  for (uint64_t b = done + gtid * ES; b + ES <= bytes; b += stride * ES) {
    float r = pull_reduce1<DT, OP>(A, me, base + b) * scale;
    if constexpr (OUT_F32 && DT != DT_F32) reinterpret_cast<float*>(out)[b / ES] = r;
    else store1<DT>(out + b, r);
  }
  peer_barrier(A, me, 4 * A.epoch + 2, &s_fail);
}

// ---------------------------------------------------------------------------------------------
// all-gather (push) and all-to-all (push); `count` is in bytes here
// ---------------------------------------------------------------------------------------------
template <bool NVLS>
__global__ void __launch_bounds__(1024) allgather_kernel(const __grid_constant__ CollArgs A) {
  __shared__ uint32_t s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const int me = my_rank(A), n = A.w.world;
  const int slot = A.nvirt > 1 ? me : 0;
  if (!peer_barrier(A, me, 4 * A.epoch + 1, &s_fail)) return;
  const uint64_t bytes = A.count;
  const char* in = A.local_in[slot] ? static_cast<const char*>(A.local_in[slot]) : A.w.heap[me] + A.in_off;
  const uint64_t dst = A.out_off + static_cast<uint64_t>(me) * bytes;
  const bool aligned = ((reinterpret_cast<uintptr_t>(in) | dst) & 15) == 0;
  const uint64_t nvec = aligned ? bytes >> 4 : 0;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  const uint64_t gtid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  {
    uint64_t i = gtid;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      Vec16 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = ld16(in + ((i + u * stride) << 4));
      if constexpr (NVLS) {
#pragma unroll
        for (int u = 0; u < 4; ++u) multimem_st(A.w.mc_heap + dst + ((i + u * stride) << 4), v[u]);
      } else {
        for (int k = 0; k < n; ++k) {
          int p = me + k;
          if (p >= n) p -= n;
#pragma unroll
          for (int u = 0; u < 4; ++u) st16(A.w.heap[p] + dst + ((i + u * stride) << 4), v[u]);
        }
      }
    }
    for (; i < nvec; i += stride) {
      Vec16 v = ld16(in + (i << 4));
      if constexpr (NVLS) {
        multimem_st(A.w.mc_heap + dst + (i << 4), v);
      } else {
        for (int k = 0; k < n; ++k) {
          int p = me + k;
          if (p >= n) p -= n;
          st16(A.w.heap[p] + dst + (i << 4), v);
        }
      }
    }
  }
  for (uint64_t b = (nvec << 4) + gtid; b < bytes; b += stride) {
    char c = in[b];
    for (int p = 0; p < n; ++p) A.w.heap[p][dst + b] = c;
  }
  peer_barrier(A, me, 4 * A.epoch + 2, &s_fail);
}

__global__ void __launch_bounds__(1024) alltoall_kernel(const __grid_constant__ CollArgs A) {
  __shared__ uint32_t s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const int me = my_rank(A), n = A.w.world;
  const int slot = A.nvirt > 1 ? me : 0;
  if (!peer_barrier(A, me, 4 * A.epoch + 1, &s_fail)) return;
  const uint64_t bytes = A.count;
  const char* in = A.local_in[slot] ? static_cast<const char*>(A.local_in[slot]) : A.w.heap[me] + A.in_off;
  const uint64_t dst = A.out_off + static_cast<uint64_t>(me) * bytes;
  const bool aligned = ((reinterpret_cast<uintptr_t>(in) | dst | bytes) & 15) == 0;
  const uint64_t nvec = aligned ? bytes >> 4 : 0;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  const uint64_t gtid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (int k = 0; k < n; ++k) {
    int p = me + k;
    if (p >= n) p -= n;
    const char* src = in + static_cast<uint64_t>(p) * bytes;
    char* out = A.w.heap[p] + dst;
    for (uint64_t i = gtid; i < nvec; i += stride) st16(out + (i << 4), ld16(src + (i << 4)));
    for (uint64_t b = (nvec << 4) + gtid; b < bytes; b += stride) out[b] = src[b];
  }
  peer_barrier(A, me, 4 * A.epoch + 2, &s_fail);
}

// ---------------------------------------------------------------------------------------------
// reduce-scatter + AdamW (bf16 gradients; count % 8 == 0; shard 16-byte aligned)
// ---------------------------------------------------------------------------------------------
template <bool NVLS>
__global__ void __launch_bounds__(512) reduce_scatter_adamw_kernel(const __grid_constant__ CollArgs A, const AdamArgs O) {
  __shared__ uint32_t s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const int me = A.rank;
  if (!peer_barrier(A, me, 4 * A.epoch + 1, &s_fail)) return;
  const uint64_t nvec = (A.count * 2) >> 4;
  const uint64_t base = A.in_off + static_cast<uint64_t>(me) * A.count * 2;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  const float scale = A.scale, one_m_b1 = 1.f - O.b1, one_m_b2 = 1.f - O.b2, decay = 1.f - O.lr * O.wd;
  __nv_bfloat16* pb = static_cast<__nv_bfloat16*>(O.p_bf16);
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float g[8];
    if constexpr (NVLS) unpack<DT_BF16>(multimem_ld_reduce<DT_BF16, RED_SUM>(A.w.mc_heap + base + (i << 4)), g);
    else pull_reduce<DT_BF16, RED_SUM>(A, me, base + (i << 4), g);
    float P[8], M[8], V[8];
    unpack<DT_F32>(ld16(O.p + i * 8), P); unpack<DT_F32>(ld16(O.p + i * 8 + 4), P + 4);
    unpack<DT_F32>(ld16(O.m + i * 8), M); unpack<DT_F32>(ld16(O.m + i * 8 + 4), M + 4);
    unpack<DT_F32>(ld16(O.v + i * 8), V); unpack<DT_F32>(ld16(O.v + i * 8 + 4), V + 4);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = g[k] * scale;
      M[k] = O.b1 * M[k] + one_m_b1 * gk;
      V[k] = O.b2 * V[k] + one_m_b2 * gk * gk;
      P[k] = P[k] * decay - O.lr * (M[k] * O.inv_bc1) / (sqrtf(V[k]) * O.inv_sqrt_bc2 + O.eps);
    }
    st16(O.p + i * 8, pack<DT_F32>(P)); st16(O.p + i * 8 + 4, pack<DT_F32>(P + 4));
    st16(O.m + i * 8, pack<DT_F32>(M)); st16(O.m + i * 8 + 4, pack<DT_F32>(M + 4));
    st16(O.v + i * 8, pack<DT_F32>(V)); st16(O.v + i * 8 + 4, pack<DT_F32>(V + 4));
    st16(pb + i * 8, pack<DT_BF16>(P));
  }
  peer_barrier(A, me, 4 * A.epoch + 2, &s_fail);
}

template <typename K>
int launchCoop(K kernel, const CollArgs& a, int blocks, int threads, cudaStream_t stream) {
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocksPerColl) blocks = kMaxBlocksPerColl;
  if (a.flag_lane < 0 || a.flag_lane >= 8) return static_cast<int>(cudaErrorInvalidValue);
  if (a.algo == ALGO_NVLS && (!a.w.mc_heap || a.nvirt > 1)) return static_cast<int>(cudaErrorInvalidValue);
  dim3 grid(blocks, a.nvirt > 1 ? a.nvirt : 1), block(threads);
  void* args[] = {const_cast<CollArgs*>(&a)};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), grid, block, args, 0, stream));
}

#define PCCL_DISPATCH_DT_OP(CALL)                                                    \
  switch (a.dtype) {                                                                 \
    case DT_F32:                                                                     \
      switch (a.redop) { case RED_SUM: CALL(DT_F32, RED_SUM) case RED_MAX: CALL(DT_F32, RED_MAX) case RED_MIN: CALL(DT_F32, RED_MIN) default: break; } break; \
    case DT_BF16:                                                                    \
      switch (a.redop) { case RED_SUM: CALL(DT_BF16, RED_SUM) case RED_MAX: CALL(DT_BF16, RED_MAX) case RED_MIN: CALL(DT_BF16, RED_MIN) default: break; } break; \
    case DT_F16:                                                                     \
      switch (a.redop) { case RED_SUM: CALL(DT_F16, RED_SUM) case RED_MAX: CALL(DT_F16, RED_MAX) case RED_MIN: CALL(DT_F16, RED_MIN) default: break; } break; \
    case DT_FP8_E4M3:                                                                \
      switch (a.redop) { case RED_SUM: CALL(DT_FP8_E4M3, RED_SUM) case RED_MAX: CALL(DT_FP8_E4M3, RED_MAX) default: break; } break; \
    default: break;                                                                  \
  }

}  // namespace

int launchAllReduce(const CollArgs& a, int blocks, int threads, cudaStream_t stream) {
  const bool nvls = a.algo == ALGO_NVLS;
  const uint64_t bytes = a.count * dtypeSize(a.dtype);
  // Up to 64 KiB: flag-in-data packets, no barrier at all (needs the low-latency area and whole 4-byte words).
  if (a.ll_off && bytes <= kLlMaxBytes && bytes % 4 == 0 && a.w.world > 1 && a.w.world <= kMaxRanks &&
      (a.dtype == DT_F32 || a.dtype == DT_BF16 || a.dtype == DT_F16) && (a.redop == RED_SUM || a.redop == RED_MAX || a.redop == RED_MIN)) {
    const int words = static_cast<int>(bytes / 4);
    int ll_blocks = (words + threads - 1) / threads;
    if (ll_blocks > 32) ll_blocks = 32;
    // One rank per launch: at most 32 CTAs, which wait only on other GPUs, so a plain launch will do (it costs less on
    // the host than a cooperative one, and this path is about latency).  Emulated ranks share a GPU: cooperative.
#define PCCL_LL(DT_, OP_)                                                            \
    if (a.nvirt <= 1) {                                                              \
      allreduce_ll_kernel<DT_, OP_><<<ll_blocks, threads, 0, stream>>>(a);           \
      return static_cast<int>(cudaGetLastError());                                   \
    }                                                                                \
    return launchCoop(allreduce_ll_kernel<DT_, OP_>, a, ll_blocks, threads, stream);
    switch (a.dtype) {
      case DT_F32: switch (a.redop) { case RED_SUM: PCCL_LL(DT_F32, RED_SUM) case RED_MAX: PCCL_LL(DT_F32, RED_MAX) default: PCCL_LL(DT_F32, RED_MIN) }
      case DT_BF16: switch (a.redop) { case RED_SUM: PCCL_LL(DT_BF16, RED_SUM) case RED_MAX: PCCL_LL(DT_BF16, RED_MAX) default: PCCL_LL(DT_BF16, RED_MIN) }
      default: switch (a.redop) { case RED_SUM: PCCL_LL(DT_F16, RED_SUM) case RED_MAX: PCCL_LL(DT_F16, RED_MAX) default: PCCL_LL(DT_F16, RED_MIN) }
    }
#undef PCCL_LL
  }
  // One-shot below 256 KiB when the output does not alias the input: one barrier pair, no second hop.  Through the switch
  // only up to 64 KiB: every rank then asks the switch to reduce the WHOLE message, and on four GPUs that took 23 us at
  // 128 KiB and 72 us at 256 KiB where the two-hop kernel needs under 20.
  const bool oneshot = bytes <= (nvls ? (64u << 10) : (256u << 10)) && a.in_off != a.out_off;
#define PCCL_AR(DT_, OP_)                                                                              \
  return oneshot ? (nvls ? launchCoop(allreduce_oneshot_kernel<DT_, OP_, true>, a, blocks, threads, stream)  \
                         : launchCoop(allreduce_oneshot_kernel<DT_, OP_, false>, a, blocks, threads, stream)) \
                 : (nvls ? launchCoop(allreduce_kernel<DT_, OP_, true>, a, blocks, threads, stream)           \
                         : launchCoop(allreduce_kernel<DT_, OP_, false>, a, blocks, threads, stream));
  PCCL_DISPATCH_DT_OP(PCCL_AR)
#undef PCCL_AR
  return static_cast<int>(cudaErrorNotSupported);
}

int launchReduceScatter(const CollArgs& a, int blocks, int threads, cudaStream_t stream) {
  const bool nvls = a.algo == ALGO_NVLS;
  const bool f32out = a.out_dtype == DT_F32 && a.dtype != DT_F32;
#define PCCL_RS(DT_, OP_)                                                                                       \
  return f32out ? (nvls ? launchCoop(reduce_scatter_kernel<DT_, OP_, true, true>, a, blocks, threads, stream)   \
                        : launchCoop(reduce_scatter_kernel<DT_, OP_, false, true>, a, blocks, threads, stream)) \
                : (nvls ? launchCoop(reduce_scatter_kernel<DT_, OP_, true, false>, a, blocks, threads, stream)  \
                        : launchCoop(reduce_scatter_kernel<DT_, OP_, false, false>, a, blocks, threads, stream));
  PCCL_DISPATCH_DT_OP(PCCL_RS)
#undef PCCL_RS
  return static_cast<int>(cudaErrorNotSupported);
}

int launchReduceScatterAdamW(const CollArgs& a, const AdamArgs& o, int blocks, int threads, cudaStream_t stream) {
  if (a.dtype != DT_BF16 || a.nvirt > 1 || a.count % 8 || a.flag_lane < 0 || a.flag_lane >= 8) return static_cast<int>(cudaErrorInvalidValue);
  if (a.algo == ALGO_NVLS && !a.w.mc_heap) return static_cast<int>(cudaErrorInvalidValue);
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocksPerColl) blocks = kMaxBlocksPerColl;
  void* args[] = {const_cast<CollArgs*>(&a), const_cast<AdamArgs*>(&o)};
  void* kern = a.algo == ALGO_NVLS ? reinterpret_cast<void*>(reduce_scatter_adamw_kernel<true>)
                                   : reinterpret_cast<void*>(reduce_scatter_adamw_kernel<false>);
  return static_cast<int>(cudaLaunchCooperativeKernel(kern, dim3(blocks), dim3(threads), args, 0, stream));
}

// ---------------------------------------------------------------------------------------------
// block-scaled fp8 all-reduce / reduce-scatter: dequantise -> fp32 accumulate -> requantise, per 128-value block
// ---------------------------------------------------------------------------------------------
// 16 consecutive lanes own one block (8 bytes each); the block's scale is read by all of them (one broadcast load).
template <bool ALL, uint32_t OP>
__global__ void __launch_bounds__(512) reduce_fp8_kernel(const __grid_constant__ CollArgs A) {
  __shared__ uint32_t s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const int me = my_rank(A), n = A.w.world;
  if (!peer_barrier(A, me, 4 * A.epoch + 1, &s_fail)) return;
  const uint64_t nb = A.count >> 7;                       // blocks of the vector (AR) or of one shard (RS)
  uint64_t lo, hi;                                        // input blocks this rank reduces
  if (ALL) {
    const uint64_t per = (nb + n - 1) / n;
    lo = min(per * me, nb);
    hi = min(per * (me + 1), nb);
  } else {
    lo = nb * me;
    hi = nb * (me + 1);
  }
  const int sub = threadIdx.x & 15;
  const uint64_t hw = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const uint64_t nhw = (static_cast<uint64_t>(gridDim.x) * blockDim.x) >> 4;
  const int slot = A.nvirt > 1 ? me : 0;
  // every half-warp of a warp runs the same number of iterations (the shuffles below are warp-wide)
  const uint64_t span = hi - lo;
  const uint64_t iters = (span + nhw - 1) / nhw;
  for (uint64_t it = 0; it < iters; ++it) {
    const uint64_t b = lo + it * nhw + hw;
    const bool live = b < hi;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = OP == RED_SUM ? 0.f : (OP == RED_MAX ? -INFINITY : INFINITY);
    if (live) {
      for (int g = 0; g < n; g += 8) {
        uint2 q[8];
        float sc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (g + k < n) {
            int p = me + g + k;
            if (p >= n) p -= n;
            q[k] = *reinterpret_cast<const uint2*>(A.w.heap[p] + A.in_off + (b << 7) + sub * 8);
            sc[k] = *reinterpret_cast<const float*>(A.w.heap[p] + A.s_in_off + (b << 2));
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (g + k < n) {
            const uint32_t w[2] = {q[k].x, q[k].y};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((w[h] >> (16 * j)) & 0xffffu), __NV_E4M3);
                const float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
                const float v0 = f.x * sc[k], v1 = f.y * sc[k];
                float& a0 = acc[4 * h + 2 * j];
                float& a1 = acc[4 * h + 2 * j + 1];
                if (OP == RED_SUM) { a0 += v0; a1 += v1; }
                else if (OP == RED_MAX) { a0 = fmaxf(a0, v0); a1 = fmaxf(a1, v1); }
                else { a0 = fminf(a0, v0); a1 = fminf(a1, v1); }
              }
            }
          }
        }
      }
    }
    float amax = 0.f;
    if (live) {
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(acc[i]));
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!live) continue;
    const float scale = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
    const float inv = 1.0f / scale;
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t l = __nv_cvt_float2_to_fp8x2(make_float2(acc[4 * h] * inv, acc[4 * h + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      uint32_t u = __nv_cvt_float2_to_fp8x2(make_float2(acc[4 * h + 2] * inv, acc[4 * h + 3] * inv), __NV_SATFINITE, __NV_E4M3);
      w[h] = (l & 0xffffu) | (u << 16);
    }
    const uint2 out = make_uint2(w[0], w[1]);
    if (ALL) {
      for (int k = 0; k < n; ++k) {
        int p = me + k;
        if (p >= n) p -= n;
        *reinterpret_cast<uint2*>(A.w.heap[p] + A.out_off + (b << 7) + sub * 8) = out;
        if (sub == 0) *reinterpret_cast<float*>(A.w.heap[p] + A.s_out_off + (b << 2)) = scale;
      }
    } else {
      const uint64_t ob = b - lo;
      char* oq = A.local_out[slot] ? static_cast<char*>(A.local_out[slot]) : A.w.heap[me] + A.out_off;
      *reinterpret_cast<uint2*>(oq + (ob << 7) + sub * 8) = out;
      if (sub == 0) *reinterpret_cast<float*>(A.w.heap[me] + A.s_out_off + (ob << 2)) = scale;
    }
  }
  peer_barrier(A, me, 4 * A.epoch + 2, &s_fail);
}

template <bool ALL>
int launchReduceFp8(const CollArgs& a, int blocks, int threads, cudaStream_t stream) {
  if (a.count % 128 || a.dtype != DT_FP8_E4M3) return static_cast<int>(cudaErrorInvalidValue);
  if (a.redop == RED_SUM) return launchCoop(reduce_fp8_kernel<ALL, RED_SUM>, a, blocks, threads, stream);
  if (a.redop == RED_MAX) return launchCoop(reduce_fp8_kernel<ALL, RED_MAX>, a, blocks, threads, stream);
  if (a.redop == RED_MIN) return launchCoop(reduce_fp8_kernel<ALL, RED_MIN>, a, blocks, threads, stream);
  return static_cast<int>(cudaErrorNotSupported);
}

int launchAllReduceFp8(const CollArgs& a, int blocks, int threads, cudaStream_t stream) { return launchReduceFp8<true>(a, blocks, threads, stream); }
int launchReduceScatterFp8(const CollArgs& a, int blocks, int threads, cudaStream_t stream) { return launchReduceFp8<false>(a, blocks, threads, stream); }

int launchAllGather(const CollArgs& a, int blocks, int threads, cudaStream_t stream) {
  return a.algo == ALGO_NVLS ? launchCoop(allgather_kernel<true>, a, blocks, threads, stream)
                             : launchCoop(allgather_kernel<false>, a, blocks, threads, stream);
}

int launchAllToAll(const CollArgs& a, int blocks, int threads, cudaStream_t stream) {
  CollArgs b = a;
  b.algo = ALGO_P2P;
  return launchCoop(alltoall_kernel, b, blocks, threads, stream);
}

}  // namespace pccl
