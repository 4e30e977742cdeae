// LayerNorm forward and backward for bf16 activations (fp32 statistics).  One CTA per row; every
// thread keeps its 8-element vectors of the row in registers, so x is read once in forward and x, dy
// once in backward.  The backward kernel is persistent: each CTA walks rows with a stride, keeps its
// share of dgamma / dbeta in registers across all of its rows and writes one partial row at the end;
// a second small kernel adds the partial rows.  (PyTorch's stock backward takes two kernels and ~230 us
// per call at 16384 x 2048; this takes ~60 us.)
#include <cuda_bf16.h>

#include "elementwise_api.h"
#include "prims.cuh"

namespace pccl {

namespace {

using namespace dev;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = 0.f;
  for (int w = 0; w < nw; ++w) r += scratch[w];
  return r;
}

__device__ __forceinline__ void block_sum2(float a, float b, float* scratch, float* ra, float* rb) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { scratch[warp] = a; scratch[8 + warp] = b; }
  __syncthreads();
  float x = 0.f, y = 0.f;
  for (int w = 0; w < nw; ++w) { x += scratch[w]; y += scratch[8 + w]; }
  *ra = x;
  *rb = y;
}

template <int MAXV>
__global__ void __launch_bounds__(256) ln_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                                                     const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                                                     float* __restrict__ mean, float* __restrict__ rstd, int D, float eps) {
  __shared__ float scratch[8];
  const long long row = blockIdx.x;
  const int nvec = D >> 3;
  float f[MAXV][8];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int v = threadIdx.x + j * 256;
    if (v < nvec) {
      unpack<DT_BF16>(ld16(x + row * D + v * 8), f[j]);
#pragma unroll
      for (int k = 0; k < 8; ++k) s += f[j][k];
    }
  }
  const float mu = block_sum(s, scratch) / D;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int v = threadIdx.x + j * 256;
    if (v < nvec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) { const float d = f[j][k] - mu; q += d * d; }
    }
  }
  const float rs = rsqrtf(block_sum(q, scratch) / D + eps);
  if (threadIdx.x == 0) { mean[row] = mu; rstd[row] = rs; }
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int v = threadIdx.x + j * 256;
    if (v < nvec) {
      float g[8], b[8], o[8];
      unpack<DT_BF16>(ld16(gamma + v * 8), g);
      unpack<DT_BF16>(ld16(beta + v * 8), b);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = (f[j][k] - mu) * rs * g[k] + b[k];
      st16(y + row * D + v * 8, pack<DT_BF16>(o));
    }
  }
}

template <int MAXV>
__global__ void __launch_bounds__(256) ln_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                     const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean,
                                                     const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                                                     float* __restrict__ part_g, float* __restrict__ part_b, long long rows, int D) {
  __shared__ float scratch[16];
  const int nvec = D >> 3;
  float g[MAXV][8], ag[MAXV][8], ab[MAXV][8];
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int v = threadIdx.x + j * 256;
#pragma unroll
    for (int k = 0; k < 8; ++k) { ag[j][k] = 0.f; ab[j][k] = 0.f; g[j][k] = 0.f; }
    if (v < nvec) unpack<DT_BF16>(ld16(gamma + v * 8), g[j]);
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mu = mean[row], rs = rstd[row];
    float xh[MAXV][8], dg[MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int v = threadIdx.x + j * 256;
      if (v < nvec) {
        float d[8];
        unpack<DT_BF16>(ld16(x + row * D + v * 8), xh[j]);
        unpack<DT_BF16>(ld16(dy + row * D + v * 8), d);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[j][k] = (xh[j][k] - mu) * rs;
          dg[j][k] = d[k] * g[j][k];
          s1 += dg[j][k];
          s2 += dg[j][k] * xh[j][k];
          ag[j][k] += d[k] * xh[j][k];
          ab[j][k] += d[k];
        }
      }
    }
    float m1, m2;
    block_sum2(s1, s2, scratch, &m1, &m2);
    m1 /= D;
    m2 /= D;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int v = threadIdx.x + j * 256;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rs * (dg[j][k] - m1 - xh[j][k] * m2);
        st16(dx + row * D + v * 8, pack<DT_BF16>(o));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int v = threadIdx.x + j * 256;
    if (v < nvec) {
      float* pg = part_g + static_cast<long long>(blockIdx.x) * D + v * 8;
      float* pb = part_b + static_cast<long long>(blockIdx.x) * D + v * 8;
      st16(pg, pack<DT_F32>(ag[j])); st16(pg + 4, pack<DT_F32>(ag[j] + 4));
      st16(pb, pack<DT_F32>(ab[j])); st16(pb + 4, pack<DT_F32>(ab[j] + 4));
    }
  }
}

// 32 columns x 8 partial-row lanes per CTA: the partial rows are summed eight at a time in parallel
__global__ void __launch_bounds__(256) ln_bwd_reduce_kernel(const float* __restrict__ part_g, const float* __restrict__ part_b,
                                                            __nv_bfloat16* __restrict__ dgamma, __nv_bfloat16* __restrict__ dbeta,
                                                            int nparts, int D) {
  __shared__ float sg[8][33], sb[8][33];
  const int col = blockIdx.x * 32 + (threadIdx.x & 31), lane8 = threadIdx.x >> 5;
  float g = 0.f, b = 0.f;
  if (col < D) {
    for (int p = lane8; p < nparts; p += 8) {
      g += part_g[static_cast<long long>(p) * D + col];
      b += part_b[static_cast<long long>(p) * D + col];
    }
  }
  sg[lane8][threadIdx.x & 31] = g;
  sb[lane8][threadIdx.x & 31] = b;
  __syncthreads();
  if (lane8 == 0 && col < D) {
#pragma unroll
    for (int k = 1; k < 8; ++k) { g += sg[k][threadIdx.x]; b += sb[k][threadIdx.x]; }
    dgamma[col] = __float2bfloat16_rn(g);
    dbeta[col] = __float2bfloat16_rn(b);
  }
}

}  // namespace

int launchLayerNormFwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, long long rows, int D,
                       float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 8 || D > 8192) return static_cast<int>(cudaErrorInvalidValue);
  auto X = static_cast<const __nv_bfloat16*>(x); auto G = static_cast<const __nv_bfloat16*>(gamma);
  auto B = static_cast<const __nv_bfloat16*>(beta); auto Y = static_cast<__nv_bfloat16*>(y);
  const unsigned grid = static_cast<unsigned>(rows);
  if (D <= 2048) ln_fwd_kernel<1><<<grid, 256, 0, stream>>>(X, G, B, Y, mean, rstd, D, eps);
  else if (D <= 4096) ln_fwd_kernel<2><<<grid, 256, 0, stream>>>(X, G, B, Y, mean, rstd, D, eps);
  else ln_fwd_kernel<4><<<grid, 256, 0, stream>>>(X, G, B, Y, mean, rstd, D, eps);
  return static_cast<int>(cudaGetLastError());
}

int layerNormBwdParts(long long rows) { return static_cast<int>(rows < 148 * 8 ? rows : 148 * 8); }

int launchLayerNormBwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx, void* dgamma,
                       void* dbeta, float* partials, long long rows, int D, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 8 || D > 8192) return static_cast<int>(cudaErrorInvalidValue);
  const int parts = layerNormBwdParts(rows);
  float* pg = partials;
  float* pb = partials + static_cast<long long>(parts) * D;
  auto DY = static_cast<const __nv_bfloat16*>(dy); auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const __nv_bfloat16*>(gamma); auto DX = static_cast<__nv_bfloat16*>(dx);
  if (D <= 2048) ln_bwd_kernel<1><<<parts, 256, 0, stream>>>(DY, X, G, mean, rstd, DX, pg, pb, rows, D);
  else if (D <= 4096) ln_bwd_kernel<2><<<parts, 256, 0, stream>>>(DY, X, G, mean, rstd, DX, pg, pb, rows, D);
  else ln_bwd_kernel<4><<<parts, 256, 0, stream>>>(DY, X, G, mean, rstd, DX, pg, pb, rows, D);
  ln_bwd_reduce_kernel<<<(D + 31) / 32, 256, 0, stream>>>(pg, pb, static_cast<__nv_bfloat16*>(dgamma), static_cast<__nv_bfloat16*>(dbeta), parts, D);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace pccl
