// Device-side building blocks for the communication kernels (sm_100a).
//
// Covers what the reference's two device headers were for —
//   include/plugins/cuda_executor/utils/multimem.h:12-127 (multimem.ld_reduce / .st / .red wrappers,
//   add only; its ld_reduce never returns the loaded value and the scalar .red forms are malformed)
//   include/plugins/cuda_executor/utils/vector_datatype.h:21-80 (packed register types)
// — and adds what a kernel that talks to peers needs: system-scope release/acquire flag accesses,
// waits that give up after a time limit instead of hanging, min/max in-switch reductions for the
// 16-bit types, fp32 accumulation for 16-bit in-switch sums, and typed 16-byte reduce helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdint>

#include "../base/instr.h"

namespace pccl {
namespace dev {

// ---------------------------------------------------------------------------------------------
// flags: system-scope release / acquire
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ld_relaxed_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Polls until *p >= target.  Gives up after `limit_ns` nanoseconds of waiting, or as soon as
// *abort_word != 0 (another worker of this rank already failed).  Returns true on success.
// Never traps, never spins forever.
__device__ __forceinline__ bool wait_ge(const uint64_t* p, uint64_t target, uint64_t limit_ns,
                                        const uint32_t* abort_word) {
  if (ld_acquire_sys(p) >= target) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if (ld_acquire_sys(p) >= target) return true;
    if ((i & 63) == 0) {
      if (abort_word && ld_volatile_u32(abort_word) != 0) return false;
      if (global_timer_ns() - t0 > limit_ns) return false;
      __nanosleep(32);
    }
  }
}

// First failure wins; later ones keep the first record.
__device__ __forceinline__ void report(uint32_t* status, uint32_t code, uint32_t a, uint32_t b, uint32_t c) {
  if (atomicCAS(status, 0u, code) == 0u) {
    status[1] = a;
    status[2] = b;
    status[3] = c;
    __threadfence_system();
  }
}

// ---------------------------------------------------------------------------------------------
// 16-byte vectors
// ---------------------------------------------------------------------------------------------
struct alignas(16) Vec16 {
  uint32_t w[4];
};

__device__ __forceinline__ Vec16 ld16(const void* p) {
  Vec16 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st16(void* p, const Vec16& v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]) : "memory");
}

// ---------------------------------------------------------------------------------------------
// multimem (NVLS): the address must be inside a multicast mapping, 16-byte aligned for .v4
// ---------------------------------------------------------------------------------------------
template <uint32_t DT, uint32_t OP>
struct MultimemSupported {
  static constexpr bool value = (DT == DT_F32 && OP == RED_SUM) || ((DT == DT_BF16 || DT == DT_F16) && OP != RED_PROD);
};

template <uint32_t DT, uint32_t OP>
__device__ __forceinline__ Vec16 multimem_ld_reduce(const void* mc) {
  Vec16 v = {};
  if constexpr (DT == DT_F32 && OP == RED_SUM) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(mc) : "memory");
  } else if constexpr (DT == DT_BF16 && OP == RED_SUM) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(mc) : "memory");
  } else if constexpr (DT == DT_BF16 && OP == RED_MAX) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(mc) : "memory");
  } else if constexpr (DT == DT_BF16 && OP == RED_MIN) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(mc) : "memory");
  } else if constexpr (DT == DT_F16 && OP == RED_SUM) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(mc) : "memory");
  } else if constexpr (DT == DT_F16 && OP == RED_MAX) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(mc) : "memory");
  } else if constexpr (DT == DT_F16 && OP == RED_MIN) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(mc) : "memory");
  }
  return v;
}

// Store to every replica (type-agnostic 16 bytes).
__device__ __forceinline__ void multimem_st(void* mc, const Vec16& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.w[0]), "r"(v.w[1]),
               "r"(v.w[2]), "r"(v.w[3]) : "memory");
}

// Fire-and-forget add into every replica.
template <uint32_t DT>
__device__ __forceinline__ void multimem_red_add(void* mc, const Vec16& v) {
  if constexpr (DT == DT_F32) {
    asm volatile("multimem.red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.w[0]), "r"(v.w[1]),
                 "r"(v.w[2]), "r"(v.w[3]) : "memory");
  } else if constexpr (DT == DT_BF16) {
    asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.w[0]), "r"(v.w[1]),
                 "r"(v.w[2]), "r"(v.w[3]) : "memory");
  } else if constexpr (DT == DT_F16) {
    asm volatile("multimem.red.relaxed.sys.global.add.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.w[0]), "r"(v.w[1]),
                 "r"(v.w[2]), "r"(v.w[3]) : "memory");
  }
}

__device__ __forceinline__ void multimem_red_add_u64(uint64_t* mc, uint64_t v) {
  asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(mc), "l"(v) : "memory");
}

// ---------------------------------------------------------------------------------------------
// typed element access and reduction in fp32
// ---------------------------------------------------------------------------------------------
template <uint32_t OP>
__device__ __forceinline__ float red1(float a, float b) {
  if constexpr (OP == RED_SUM) return a + b;
  else if constexpr (OP == RED_MAX) return fmaxf(a, b);
  else if constexpr (OP == RED_MIN) return fminf(a, b);
  else return a * b;
}

// Number of elements in 16 bytes and unpack/pack to fp32 lanes.
template <uint32_t DT> struct Lanes { static constexpr int n = 16 / 4; };
template <> struct Lanes<DT_BF16> { static constexpr int n = 8; };
template <> struct Lanes<DT_F16> { static constexpr int n = 8; };
template <> struct Lanes<DT_FP8_E4M3> { static constexpr int n = 16; };

template <uint32_t DT>
__device__ __forceinline__ void unpack(const Vec16& v, float* f) {
  if constexpr (DT == DT_F32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(v.w[i]);
  } else if constexpr (DT == DT_BF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(v.w[i] << 16);
      f[2 * i + 1] = __uint_as_float(v.w[i] & 0xffff0000u);
    }
  } else if constexpr (DT == DT_F16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&v.w[i]);
      float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  } else if constexpr (DT == DT_FP8_E4M3) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        __nv_fp8x2_storage_t pr = static_cast<__nv_fp8x2_storage_t>((v.w[i] >> (16 * j)) & 0xffffu);
        __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pr, __NV_E4M3);
        float2 t = __half22float2(*reinterpret_cast<__half2*>(&hr));
        f[4 * i + 2 * j] = t.x;
        f[4 * i + 2 * j + 1] = t.y;
      }
    }
  }
}

template <uint32_t DT>
__device__ __forceinline__ Vec16 pack(const float* f) {
  Vec16 v;
  if constexpr (DT == DT_F32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v.w[i] = __float_as_uint(f[i]);
  } else if constexpr (DT == DT_BF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 b = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      v.w[i] = *reinterpret_cast<uint32_t*>(&b);
    }
  } else if constexpr (DT == DT_F16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      v.w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
  } else if constexpr (DT == DT_FP8_E4M3) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i], f[4 * i + 1]), __NV_SATFINITE, __NV_E4M3);
      uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i + 2], f[4 * i + 3]), __NV_SATFINITE, __NV_E4M3);
      v.w[i] = (lo & 0xffffu) | (hi << 16);
    }
  }
  return v;
}

// scalar element <-> float, for ragged edges
template <uint32_t DT>
__device__ __forceinline__ float load1(const void* p) {
  if constexpr (DT == DT_F32) return *static_cast<const float*>(p);
  else if constexpr (DT == DT_BF16) return __bfloat162float(*static_cast<const __nv_bfloat16*>(p));
  else if constexpr (DT == DT_F16) return __half2float(*static_cast<const __half*>(p));
  else {
    __half_raw hr = __nv_cvt_fp8_to_halfraw(*static_cast<const __nv_fp8_storage_t*>(p), __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&hr));
  }
}
template <uint32_t DT>
__device__ __forceinline__ void store1(void* p, float f) {
  if constexpr (DT == DT_F32) *static_cast<float*>(p) = f;
  else if constexpr (DT == DT_BF16) *static_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn(f);
  else if constexpr (DT == DT_F16) *static_cast<__half*>(p) = __float2half_rn(f);
  else *static_cast<__nv_fp8_storage_t*>(p) = __nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3);
}

}  // namespace dev
}  // namespace pccl
