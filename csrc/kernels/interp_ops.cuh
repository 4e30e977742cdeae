// The data-movement loops of the collective instruction set: COPY, REDUCE (two-operand and n-ary), the in-switch
// MM_LD_REDUCE / MM_ST and their fusion.  Shared by the interpreter kernel (interpreter.cu) and by kernels that are
// generated and compiled at run time for one registered program (pccl_b200/jit.py), so both run the same loops.
#pragma once
#include "prims.cuh"

namespace pccl {
namespace iops {

using namespace dev;

__device__ __forceinline__ void copy_range(char* dst, const char* src, uint64_t bytes) {
  const uint32_t tid = threadIdx.x, nt = blockDim.x;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
    const uint64_t nvec = bytes >> 4;
    uint64_t i = tid;
    // four independent 16-byte loads in flight per thread
    for (; i + 3ull * nt < nvec; i += 4ull * nt) {
      Vec16 a = ld16(src + (i << 4)), b = ld16(src + ((i + nt) << 4));
      Vec16 c = ld16(src + ((i + 2ull * nt) << 4)), d = ld16(src + ((i + 3ull * nt) << 4));
      st16(dst + (i << 4), a);
      st16(dst + ((i + nt) << 4), b);
      st16(dst + ((i + 2ull * nt) << 4), c);
      st16(dst + ((i + 3ull * nt) << 4), d);
    }
    for (; i < nvec; i += nt) st16(dst + (i << 4), ld16(src + (i << 4)));
    for (uint64_t b = (nvec << 4) + tid; b < bytes; b += nt) dst[b] = src[b];
  } else {
    for (uint64_t b = tid; b < bytes; b += nt) dst[b] = src[b];
  }
}

template <uint32_t DT, uint32_t OP>
__device__ __forceinline__ void reduce_range_f(char* dst, const char* src, uint64_t bytes) {
  constexpr int N = Lanes<DT>::n;
  constexpr int ES = 16 / N;
  const uint32_t tid = threadIdx.x, nt = blockDim.x;
  uint64_t done = 0;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
    const uint64_t nvec = bytes >> 4;
    for (uint64_t i = tid; i < nvec; i += nt) {
      Vec16 a = ld16(dst + (i << 4)), b = ld16(src + (i << 4));
      float fa[N], fb[N];
      unpack<DT>(a, fa);
      unpack<DT>(b, fb);
#pragma unroll
      for (int k = 0; k < N; ++k) fa[k] = red1<OP>(fa[k], fb[k]);
      st16(dst + (i << 4), pack<DT>(fa));
    }
    done = nvec << 4;
  }
  for (uint64_t b = done + static_cast<uint64_t>(tid) * ES; b + ES <= bytes; b += static_cast<uint64_t>(nt) * ES)
    store1<DT>(dst + b, red1<OP>(load1<DT>(dst + b), load1<DT>(src + b)));
}

// dst = dst (op) src[0] (op) ... (op) src[k-1] in ONE pass: the destination is read and written once and the loads of
// all sources of a vector are in flight together (a chain of two-operand reduces makes a pass per source).
constexpr int kMaxFused = 8;
template <uint32_t DT, uint32_t OP>
__device__ __forceinline__ void reduce_n_range_f(char* dst, char* const* src, int k, uint64_t bytes) {
  constexpr int N = Lanes<DT>::n;
  const uint32_t tid = threadIdx.x, nt = blockDim.x;
  const uint64_t nvec = bytes >> 4;
  for (uint64_t i = tid; i < nvec; i += nt) {
    Vec16 v[kMaxFused + 1];
    v[0] = ld16(dst + (i << 4));
#pragma unroll
    for (int s = 0; s < kMaxFused; ++s)
      if (s < k) v[s + 1] = ld16(src[s] + (i << 4));
    float acc[N];
    unpack<DT>(v[0], acc);
#pragma unroll
    for (int s = 0; s < kMaxFused; ++s) {
      if (s < k) {
        float f[N];
        unpack<DT>(v[s + 1], f);
#pragma unroll
        for (int e = 0; e < N; ++e) acc[e] = red1<OP>(acc[e], f[e]);
      }
    }
    st16(dst + (i << 4), pack<DT>(acc));
  }
}

// dst = src[0] (op) src[1] ... (op) src[k-1] without reading dst: "COPY a -> d; REDUCE b -> d; REDUCE c -> d" as one pass.
// 16-byte aligned ranges, 2 <= k <= kMaxFused.
template <uint32_t DT, uint32_t OP>
__device__ __forceinline__ void reduce_n_from_f(char* dst, char* const* src, int k, uint64_t bytes) {
  constexpr int N = Lanes<DT>::n;
  const uint32_t tid = threadIdx.x, nt = blockDim.x;
  const uint64_t nvec = bytes >> 4;
  uint64_t i = tid;
  if (k <= 4) {
    // few sources (a small world): two vectors per source in flight, or the peers' links are not kept busy
    for (; i + nt < nvec; i += 2ull * nt) {
      Vec16 v[4], w[4];
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        if (s < k) {
          v[s] = ld16(src[s] + (i << 4));
          w[s] = ld16(src[s] + ((i + nt) << 4));
        }
      }
      float acc[N], bcc[N];
      unpack<DT>(v[0], acc);
      unpack<DT>(w[0], bcc);
#pragma unroll
      for (int s = 1; s < 4; ++s) {
        if (s < k) {
          float f[N], g[N];
          unpack<DT>(v[s], f);
          unpack<DT>(w[s], g);
#pragma unroll
          for (int e = 0; e < N; ++e) {
            acc[e] = red1<OP>(acc[e], f[e]);
            bcc[e] = red1<OP>(bcc[e], g[e]);
          }
        }
      }
      st16(dst + (i << 4), pack<DT>(acc));
      st16(dst + ((i + nt) << 4), pack<DT>(bcc));
    }
  }
  for (; i < nvec; i += nt) {
    Vec16 v[kMaxFused];
#pragma unroll
    for (int s = 0; s < kMaxFused; ++s)
      if (s < k) v[s] = ld16(src[s] + (i << 4));
    float acc[N];
    unpack<DT>(v[0], acc);
#pragma unroll
    for (int s = 1; s < kMaxFused; ++s) {
      if (s < k) {
        float f[N];
        unpack<DT>(v[s], f);
#pragma unroll
        for (int e = 0; e < N; ++e) acc[e] = red1<OP>(acc[e], f[e]);
      }
    }
    st16(dst + (i << 4), pack<DT>(acc));
  }
}

template <uint32_t OP>
__device__ __forceinline__ bool reduce_n_from_dispatch(uint32_t dt, char* dst, char* const* src, int k, uint64_t bytes) {
  switch (dt) {
    case DT_F32: reduce_n_from_f<DT_F32, OP>(dst, src, k, bytes); return true;
    case DT_BF16: reduce_n_from_f<DT_BF16, OP>(dst, src, k, bytes); return true;
    case DT_F16: reduce_n_from_f<DT_F16, OP>(dst, src, k, bytes); return true;
    default: return false;
  }
}

// One source, n destinations ("COPY a -> d0; COPY a -> d1; ..."): the source is read once, four vectors in flight.
// 16-byte aligned ranges.
__device__ __forceinline__ void copy_fan_range(char* const* dst, int n, const char* src, uint64_t bytes) {
  const uint32_t tid = threadIdx.x, nt = blockDim.x;
  const uint64_t nvec = bytes >> 4;
  uint64_t i = tid;
  for (; i + 3ull * nt < nvec; i += 4ull * nt) {
    const Vec16 a = ld16(src + (i << 4)), b = ld16(src + ((i + nt) << 4));
    const Vec16 c = ld16(src + ((i + 2ull * nt) << 4)), d = ld16(src + ((i + 3ull * nt) << 4));
#pragma unroll
    for (int q = 0; q < kMaxFused; ++q) {
      if (q < n) {
        st16(dst[q] + (i << 4), a);
        st16(dst[q] + ((i + nt) << 4), b);
        st16(dst[q] + ((i + 2ull * nt) << 4), c);
        st16(dst[q] + ((i + 3ull * nt) << 4), d);
      }
    }
  }
  for (; i < nvec; i += nt) {
    const Vec16 a = ld16(src + (i << 4));
#pragma unroll
    for (int q = 0; q < kMaxFused; ++q)
      if (q < n) st16(dst[q] + (i << 4), a);
  }
  for (uint64_t b = (nvec << 4) + tid; b < bytes; b += nt)
    for (int q = 0; q < n; ++q) dst[q][b] = src[b];
}

template <uint32_t OP>
__device__ __forceinline__ bool reduce_n_dispatch(uint32_t dt, char* dst, char* const* src, int k, uint64_t bytes) {
  switch (dt) {
    case DT_F32: reduce_n_range_f<DT_F32, OP>(dst, src, k, bytes); return true;
    case DT_BF16: reduce_n_range_f<DT_BF16, OP>(dst, src, k, bytes); return true;
    case DT_F16: reduce_n_range_f<DT_F16, OP>(dst, src, k, bytes); return true;
    default: return false;
  }
}

template <typename T, uint32_t OP>
__device__ __forceinline__ void reduce_range_i(char* dst, const char* src, uint64_t bytes) {
  T* d = reinterpret_cast<T*>(dst);
  const T* s = reinterpret_cast<const T*>(src);
  for (uint64_t i = threadIdx.x; i < bytes / sizeof(T); i += blockDim.x) {
    T a = d[i], b = s[i];
    if constexpr (OP == RED_SUM) d[i] = a + b;
    else if constexpr (OP == RED_MAX) d[i] = a > b ? a : b;
    else if constexpr (OP == RED_MIN) d[i] = a < b ? a : b;
    else d[i] = a * b;
  }
}

template <uint32_t OP>
__device__ __forceinline__ bool reduce_dispatch(uint32_t dt, char* dst, const char* src, uint64_t bytes) {
  switch (dt) {
    case DT_F32: reduce_range_f<DT_F32, OP>(dst, src, bytes); return true;
    case DT_BF16: reduce_range_f<DT_BF16, OP>(dst, src, bytes); return true;
    case DT_F16: reduce_range_f<DT_F16, OP>(dst, src, bytes); return true;
    case DT_FP8_E4M3: reduce_range_f<DT_FP8_E4M3, OP>(dst, src, bytes); return true;
    case DT_I32: reduce_range_i<int32_t, OP>(dst, src, bytes); return true;
    case DT_I64: reduce_range_i<long long, OP>(dst, src, bytes); return true;
    case DT_F64: reduce_range_i<double, OP>(dst, src, bytes); return true;
    case DT_U8: reduce_range_i<uint8_t, OP>(dst, src, bytes); return true;
    default: return false;
  }
}

template <uint32_t DT, uint32_t OP>
__device__ __forceinline__ void mm_ld_reduce_range(char* dst, const char* mc_src, uint64_t bytes) {
  const uint64_t nvec = bytes >> 4, nt = blockDim.x;
  uint64_t i = threadIdx.x;
  for (; i + 3 * nt < nvec; i += 4 * nt) {       // four in-switch reductions in flight per thread
    const Vec16 a = multimem_ld_reduce<DT, OP>(mc_src + (i << 4)), b = multimem_ld_reduce<DT, OP>(mc_src + ((i + nt) << 4));
    const Vec16 c = multimem_ld_reduce<DT, OP>(mc_src + ((i + 2 * nt) << 4)), d = multimem_ld_reduce<DT, OP>(mc_src + ((i + 3 * nt) << 4));
    st16(dst + (i << 4), a);
    st16(dst + ((i + nt) << 4), b);
    st16(dst + ((i + 2 * nt) << 4), c);
    st16(dst + ((i + 3 * nt) << 4), d);
  }
  for (; i < nvec; i += nt) st16(dst + (i << 4), multimem_ld_reduce<DT, OP>(mc_src + (i << 4)));
}

// in-switch reduction handed straight to a multicast store: the reduced vector never visits local memory on its way
template <uint32_t DT, uint32_t OP>
__device__ __forceinline__ void mm_reduce_bcast_range(char* mc_dst, const char* mc_src, uint64_t bytes) {
  const uint64_t nvec = bytes >> 4, nt = blockDim.x;
  uint64_t i = threadIdx.x;
  for (; i + 3 * nt < nvec; i += 4 * nt) {
    const Vec16 a = multimem_ld_reduce<DT, OP>(mc_src + (i << 4)), b = multimem_ld_reduce<DT, OP>(mc_src + ((i + nt) << 4));
    const Vec16 c = multimem_ld_reduce<DT, OP>(mc_src + ((i + 2 * nt) << 4)), d = multimem_ld_reduce<DT, OP>(mc_src + ((i + 3 * nt) << 4));
    multimem_st(mc_dst + (i << 4), a);
    multimem_st(mc_dst + ((i + nt) << 4), b);
    multimem_st(mc_dst + ((i + 2 * nt) << 4), c);
    multimem_st(mc_dst + ((i + 3 * nt) << 4), d);
  }
  for (; i < nvec; i += nt) multimem_st(mc_dst + (i << 4), multimem_ld_reduce<DT, OP>(mc_src + (i << 4)));
}

__device__ __forceinline__ bool mm_reduce_bcast_dispatch(uint32_t dt, uint32_t op, char* mc_dst, const char* mc_src, uint64_t bytes) {
#define PCCL_MM(DT_, OP_) if (dt == DT_ && op == OP_) { mm_reduce_bcast_range<DT_, OP_>(mc_dst, mc_src, bytes); return true; }
  PCCL_MM(DT_F32, RED_SUM)
  PCCL_MM(DT_BF16, RED_SUM) PCCL_MM(DT_BF16, RED_MAX) PCCL_MM(DT_BF16, RED_MIN)
  PCCL_MM(DT_F16, RED_SUM) PCCL_MM(DT_F16, RED_MAX) PCCL_MM(DT_F16, RED_MIN)
#undef PCCL_MM
  return false;
}

__device__ __forceinline__ bool mm_ld_reduce_dispatch(uint32_t dt, uint32_t op, char* dst, const char* mc, uint64_t bytes) {
#define PCCL_MM(DT_, OP_) if (dt == DT_ && op == OP_) { mm_ld_reduce_range<DT_, OP_>(dst, mc, bytes); return true; }
  PCCL_MM(DT_F32, RED_SUM)
  PCCL_MM(DT_BF16, RED_SUM) PCCL_MM(DT_BF16, RED_MAX) PCCL_MM(DT_BF16, RED_MIN)
  PCCL_MM(DT_F16, RED_SUM) PCCL_MM(DT_F16, RED_MAX) PCCL_MM(DT_F16, RED_MIN)
#undef PCCL_MM
  return false;
}

__device__ __forceinline__ void mm_st_range(char* mc_dst, const char* src, uint64_t bytes) {
  const uint64_t nvec = bytes >> 4, nt = blockDim.x;
  uint64_t i = threadIdx.x;
  for (; i + 3 * nt < nvec; i += 4 * nt) {
    const Vec16 a = ld16(src + (i << 4)), b = ld16(src + ((i + nt) << 4));
    const Vec16 c = ld16(src + ((i + 2 * nt) << 4)), d = ld16(src + ((i + 3 * nt) << 4));
    multimem_st(mc_dst + (i << 4), a);
    multimem_st(mc_dst + ((i + nt) << 4), b);
    multimem_st(mc_dst + ((i + 2 * nt) << 4), c);
    multimem_st(mc_dst + ((i + 3 * nt) << 4), d);
  }
  for (; i < nvec; i += nt) multimem_st(mc_dst + (i << 4), ld16(src + (i << 4)));
}

}  // namespace iops
}  // namespace pccl
