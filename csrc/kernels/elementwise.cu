// Memory-bound training kernels that sit next to the GEMMs: fused AdamW on a flat fp32 shard with
// the bf16 parameter write-back, and softmax cross-entropy forward+backward in one pass over the
// logits (the row is staged in shared memory: read once, gradient written once, in place).
#include <atomic>
#include <cuda_bf16.h>

#include "elementwise_api.h"
#include "prims.cuh"

namespace pccl {

namespace {

// ---------------------------------------------------------------------------------------------
// AdamW: p, m, v fp32 (sharded); g fp32; writes the updated parameter also as bf16
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                                    const float* __restrict__ g, __nv_bfloat16* __restrict__ p_bf16,
                                                    long long n, float lr, float b1, float b2, float eps, float wd,
                                                    float inv_bc1, float inv_sqrt_bc2, float grad_scale) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 pp = *reinterpret_cast<const float4*>(p + i), mm = *reinterpret_cast<const float4*>(m + i);
      float4 vv = *reinterpret_cast<const float4*>(v + i), gg = *reinterpret_cast<const float4*>(g + i);
      float P[4] = {pp.x, pp.y, pp.z, pp.w}, M[4] = {mm.x, mm.y, mm.z, mm.w}, V[4] = {vv.x, vv.y, vv.z, vv.w};
      float G[4] = {gg.x * grad_scale, gg.y * grad_scale, gg.z * grad_scale, gg.w * grad_scale};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        M[k] = b1 * M[k] + (1.f - b1) * G[k];
        V[k] = b2 * V[k] + (1.f - b2) * G[k] * G[k];
        float denom = sqrtf(V[k]) * inv_sqrt_bc2 + eps;
        P[k] = P[k] * (1.f - lr * wd) - lr * (M[k] * inv_bc1) / denom;
      }
      *reinterpret_cast<float4*>(p + i) = make_float4(P[0], P[1], P[2], P[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(M[0], M[1], M[2], M[3]);
      *reinterpret_cast<float4*>(v + i) = make_float4(V[0], V[1], V[2], V[3]);
      __nv_bfloat162 lo = __floats2bfloat162_rn(P[0], P[1]), hi = __floats2bfloat162_rn(P[2], P[3]);
      uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      *reinterpret_cast<uint2*>(p_bf16 + i) = packed;
    } else {
      for (long long j = i; j < n; ++j) {
        float G = g[j] * grad_scale;
        float M = b1 * m[j] + (1.f - b1) * G, V = b2 * v[j] + (1.f - b2) * G * G;
        float P = p[j] * (1.f - lr * wd) - lr * (M * inv_bc1) / (sqrtf(V) * inv_sqrt_bc2 + eps);
        p[j] = P; m[j] = M; v[j] = V;
        p_bf16[j] = __float2bfloat16_rn(P);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// cross entropy: one CTA per row; logits bf16 [rows, ld]; writes loss[row] and, in place,
// dlogits = (softmax - onehot) * grad_scale
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_reduce(float v, float* scratch, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
  for (int w = 1; w < nw; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
  return r;
}

__global__ void __launch_bounds__(512) cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                                                            float* __restrict__ loss, int vocab, long long ld, float grad_scale,
                                                            long long ignore_index, uint32_t* __restrict__ status) {
  extern __shared__ __align__(16) uint8_t ce_smem[];
  __nv_bfloat16* row_s = reinterpret_cast<__nv_bfloat16*>(ce_smem);
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  __nv_bfloat16* g = logits + row * ld;
  const long long tgt = targets[row];
  // stage the row: 16-byte vectors when the row start is aligned (ld % 8 == 0 and base aligned)
  const int nvec = vocab / 8;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    dev::Vec16 v = dev::ld16(g + i * 8);
    *reinterpret_cast<dev::Vec16*>(row_s + i * 8) = v;
    float f[8];
    dev::unpack<DT_BF16>(v, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) mx = fmaxf(mx, f[k]);
  }
  for (int i = nvec * 8 + threadIdx.x; i < vocab; i += blockDim.x) {
    row_s[i] = g[i];
    mx = fmaxf(mx, __bfloat162float(row_s[i]));
  }
  mx = block_reduce(mx, scratch, true);
  float sum = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) sum += __expf(__bfloat162float(row_s[i]) - mx);
  sum = block_reduce(sum, scratch, false);
  const float lse = mx + __logf(sum);
  // A target outside [0, vocab) never indexes the staged row: the row is handled like an ignored one (loss 0,
  // zero gradient), and unless it is the ignore value itself the first such row is recorded in the status words.
  const bool valid = tgt >= 0 && tgt < static_cast<long long>(vocab);
  const bool ignored = tgt == ignore_index || !valid;
  if (threadIdx.x == 0) {
    loss[row] = ignored ? 0.f : lse - __bfloat162float(row_s[tgt]);
    if (!valid && tgt != ignore_index && status && atomicCAS(status, 0u, static_cast<uint32_t>(ST_BOUNDS)) == 0u) {
      status[1] = static_cast<uint32_t>(row);
      status[2] = static_cast<uint32_t>(tgt);
      status[3] = 0xCEu;          // detail: cross-entropy target out of range
    }
  }
  const float scale = ignored ? 0.f : grad_scale;
  const float inv = 1.f / sum;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    dev::unpack<DT_BF16>(*reinterpret_cast<dev::Vec16*>(row_s + i * 8), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float p = __expf(f[k] - mx) * inv;
      f[k] = (p - ((i * 8 + k) == tgt ? 1.f : 0.f)) * scale;
    }
    dev::st16(g + i * 8, dev::pack<DT_BF16>(f));
  }
  for (int i = nvec * 8 + threadIdx.x; i < vocab; i += blockDim.x) {
    float p = __expf(__bfloat162float(row_s[i]) - mx) * inv;
    g[i] = __float2bfloat16_rn((p - (i == tgt ? 1.f : 0.f)) * scale);
  }
}

}  // namespace

int launchAdamW(float* p, float* m, float* v, const float* g, void* p_bf16, long long n, float lr, float b1, float b2,
                float eps, float wd, int step, float grad_scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  float bc1 = 1.f - powf(b1, static_cast<float>(step)), bc2 = 1.f - powf(b2, static_cast<float>(step));
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  adamw_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(p, m, v, g, static_cast<__nv_bfloat16*>(p_bf16), n, lr, b1, b2, eps, wd,
                                                             1.f / bc1, 1.f / sqrtf(bc2), grad_scale);
  return static_cast<int>(cudaGetLastError());
}

namespace {
constexpr int kMaxDevices = 64;
// The shared-memory opt-in of cross_entropy_kernel is a per-device function attribute.
std::atomic<bool> g_ce_attr[kMaxDevices];

cudaError_t ensureCrossEntropyAttr() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (g_ce_attr[dev].load(std::memory_order_acquire)) return cudaSuccess;
  e = cudaFuncSetAttribute(cross_entropy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  if (e == cudaSuccess) g_ce_attr[dev].store(true, std::memory_order_release);
  return e;
}
}  // namespace

int launchCrossEntropy(void* logits, const long long* targets, float* loss, long long rows, int vocab, long long ld,
                       float grad_scale, long long ignore_index, uint32_t* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  size_t smem = (static_cast<size_t>(vocab) * 2 + 15) / 16 * 16;
  if (smem > 200 * 1024 || ld % 8 || reinterpret_cast<uintptr_t>(logits) % 16) return static_cast<int>(cudaErrorInvalidValue);
  cudaError_t e = ensureCrossEntropyAttr();
  if (e != cudaSuccess) return static_cast<int>(e);
  cross_entropy_kernel<<<static_cast<unsigned>(rows), 512, smem, stream>>>(static_cast<__nv_bfloat16*>(logits), targets, loss, vocab, ld,
                                                                          grad_scale, ignore_index, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace pccl

// =================================================================================================
// Allocation-free mean cross-entropy (declared in no_alloc_api.h)
// =================================================================================================
#include "no_alloc_api.h"

namespace pccl {
namespace {

// Per-row losses of the call in flight.  In host code this name is only a handle for
// cudaGetSymbolAddress; kernels below name it directly.
static __device__ __align__(256) float g_noalloc_row_loss[PCCL_NOALLOC_MAX_ROWS];

__global__ void __launch_bounds__(1024) noalloc_mean_kernel(float* __restrict__ out, long long rows, float scale) {
  __shared__ float part[32];
  float s = 0.f;
  for (long long i = threadIdx.x; i < rows; i += blockDim.x) s += g_noalloc_row_loss[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) out[0] = s * scale;
  }
}

// Written without a lock: two host threads that make the FIRST call on one device at the same time both resolve
// and store the same address, which is harmless.
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
int g_noalloc_cuda_error = 0;

}  // namespace
}  // namespace pccl

extern "C" int pccl_noalloc_last_cuda_error(void) { return pccl::g_noalloc_cuda_error; }

extern "C" int pccl_cross_entropy_mean_noalloc(void* logits, const long long* targets, float* mean_loss, long long rows, int vocab,
                                               long long ld, cudaStream_t stream) {
  using namespace pccl;
  if (!logits || !targets || !mean_loss || rows <= 0 || vocab <= 0) return PCCL_NOALLOC_BAD_ARGUMENT;
  if (rows > PCCL_NOALLOC_MAX_ROWS) return PCCL_NOALLOC_TOO_LARGE;
  const size_t smem = (static_cast<size_t>(vocab) * 2 + 15) / 16 * 16;
  if (smem > 200 * 1024 || ld % 8 || ld < vocab || reinterpret_cast<uintptr_t>(logits) % 16) return PCCL_NOALLOC_BAD_ARGUMENT;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) { g_noalloc_cuda_error = static_cast<int>(e); return PCCL_NOALLOC_CUDA_ERROR; }
  if (!g_noalloc_ptr[dev]) {
    // once per device, with that device current: the device address of the static array
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_row_loss);
    if (e != cudaSuccess || !p) { g_noalloc_cuda_error = static_cast<int>(e); return PCCL_NOALLOC_CUDA_ERROR; }
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  e = ensureCrossEntropyAttr();
  if (e != cudaSuccess) { g_noalloc_cuda_error = static_cast<int>(e); return PCCL_NOALLOC_CUDA_ERROR; }
  const float scale = 1.0f / static_cast<float>(rows);
  // no ignore value of its own: every target outside [0, vocab) (the customary -100 included) makes an ignored row
  cross_entropy_kernel<<<static_cast<unsigned>(rows), 512, smem, stream>>>(static_cast<__nv_bfloat16*>(logits), targets,
                                                                          g_noalloc_ptr[dev], vocab, ld, scale, -(1ll << 62), nullptr);
  noalloc_mean_kernel<<<1, 1024, 0, stream>>>(mean_loss, rows, scale);
  e = cudaGetLastError();
  if (e != cudaSuccess) { g_noalloc_cuda_error = static_cast<int>(e); return PCCL_NOALLOC_CUDA_ERROR; }
  return PCCL_NOALLOC_OK;
}
