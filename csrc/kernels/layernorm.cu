// LayerNorm forward and backward for bf16 activations (fp32 statistics).  One CTA per row; every
// thread keeps its 8-element vectors of the row in registers, so x is read once in forward and x, dy
// once in backward.  The backward kernel is persistent: each CTA walks rows with a stride, keeps its
// share of dgamma / dbeta in registers across all of its rows and writes one partial row at the end;
// a second small kernel adds the partial rows.  (PyTorch's stock backward takes two kernels and ~230 us
// per call at 16384 x 2048; this takes ~60 us.)
//
// Both directions can carry the residual connection that surrounds the norm in a pre-norm transformer block:
// forward takes `delta` and computes s = x + delta (stored, it is the next residual stream) and y = LN(s) in one
// pass; backward adds the gradient that arrives on the residual stream (`dres`) to the norm's input gradient, and
// can emit the column sums of that total -- the bias gradient of the linear layer that produced `delta` -- next
// to dgamma / dbeta.  That removes the separate element-wise add kernels and one pass per bias gradient.
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
__global__ void __launch_bounds__(256) ln_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                                                     __nv_bfloat16* __restrict__ sum_out, const __nv_bfloat16* __restrict__ gamma,
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
      if (delta) {
        // the norm sees the sum as it is stored (rounded to bf16), so that backward, which re-reads it, agrees
        float d[8];
        unpack<DT_BF16>(ld16(delta + row * D + v * 8), d);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[j][k] += d[k];
        const Vec16 r = pack<DT_BF16>(f[j]);
        st16(sum_out + row * D + v * 8, r);
        unpack<DT_BF16>(r, f[j]);
      }
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
                                                     const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dres,
                                                     __nv_bfloat16* __restrict__ dx, float* __restrict__ part_g,
                                                     float* __restrict__ part_b, float* __restrict__ part_c, long long rows, int D) {
  __shared__ float scratch[16];
  const int nvec = D >> 3;
  float g[MAXV][8], ag[MAXV][8], ab[MAXV][8], ac[MAXV][8];
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int v = threadIdx.x + j * 256;
#pragma unroll
    for (int k = 0; k < 8; ++k) { ag[j][k] = 0.f; ab[j][k] = 0.f; ac[j][k] = 0.f; g[j][k] = 0.f; }
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
        if (dres) {
          float r[8];
          unpack<DT_BF16>(ld16(dres + row * D + v * 8), r);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += r[k];
        }
        if (part_c) {
#pragma unroll
          for (int k = 0; k < 8; ++k) ac[j][k] += o[k];
        }
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
      if (part_c) {
        float* pc = part_c + static_cast<long long>(blockIdx.x) * D + v * 8;
        st16(pc, pack<DT_F32>(ac[j])); st16(pc + 4, pack<DT_F32>(ac[j] + 4));
      }
    }
  }
}

// Backward for D = NV * 256 <= 2048 with one WARP per row: a lane keeps NV 16-byte vectors of x, dy (and dres) of its
// row in flight at once (up to 12 KiB per warp), the row statistics need only warp shuffles (no CTA barrier per row),
// and the column sums (dgamma, dbeta, bias gradient) are accumulated in shared memory that is private to the warp:
// 8 warps x 3 arrays x D floats, laid out as two planes of 4-float halves so that consecutive lanes touch consecutive
// 16-byte words (no bank conflicts).  At the end the CTA adds its 8 private copies and writes one partial row per
// array; with one CTA per SM that leaves at most 148 partial rows for the reduce kernel.
template <int NV>
__global__ void __launch_bounds__(256, 1) ln_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                             const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean,
                                                             const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dres,
                                                             __nv_bfloat16* __restrict__ dx, float* __restrict__ part_g,
                                                             float* __restrict__ part_b, float* __restrict__ part_c, long long rows) {
  constexpr int D = NV * 256;
  constexpr int HALF = D / 8;                 // float4 slots per plane
  extern __shared__ __align__(16) float ln_acc[];          // [8 warps][3 arrays][2 planes][D / 8][4], then gamma (bf16 [D])
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 8 * 3 * D / 4; i += 256) reinterpret_cast<float4*>(ln_acc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  Vec16* gq = reinterpret_cast<Vec16*>(ln_acc + 8 * 3 * D);      // read per use: keeps 4 * NV registers free
  for (int i = threadIdx.x; i < D / 8; i += 256) gq[i] = ld16(gamma + i * 8);
  __syncthreads();
  float4* acc_g = reinterpret_cast<float4*>(ln_acc + (warp * 3 + 0) * D);
  float4* acc_b = reinterpret_cast<float4*>(ln_acc + (warp * 3 + 1) * D);
  float4* acc_c = reinterpret_cast<float4*>(ln_acc + (warp * 3 + 2) * D);
  const float inv_d = 1.0f / D;
  for (long long row = static_cast<long long>(blockIdx.x) * 8 + warp; row < rows; row += static_cast<long long>(gridDim.x) * 8) {
    const long long base = row * D + lane * 8;
    Vec16 vx[NV], vd[NV], vr[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      vx[j] = ld16(x + base + j * 256);
      vd[j] = ld16(dy + base + j * 256);
      if (dres) vr[j] = ld16(dres + base + j * 256);
    }
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float xf[8], df[8], gf[8];
      unpack<DT_BF16>(vx[j], xf);
      unpack<DT_BF16>(vd[j], df);
      unpack<DT_BF16>(gq[j * 32 + lane], gf);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float dg = df[k] * gf[k];
        s1 += dg;
        s2 += dg * ((xf[k] - mu) * rs);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    const float m1 = s1 * inv_d, m2 = s2 * inv_d;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float xf[8], df[8], gf[8], of[8];
      unpack<DT_BF16>(vx[j], xf);
      unpack<DT_BF16>(vd[j], df);
      unpack<DT_BF16>(gq[j * 32 + lane], gf);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        xf[k] = (xf[k] - mu) * rs;
        of[k] = rs * (df[k] * gf[k] - m1 - xf[k] * m2);
      }
      if (dres) {
        float rf[8];
        unpack<DT_BF16>(vr[j], rf);
#pragma unroll
        for (int k = 0; k < 8; ++k) of[k] += rf[k];
      }
      st16(dx + base + j * 256, pack<DT_BF16>(of));
      const int vec = j * 32 + lane;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float4 a = acc_g[h * HALF + vec], b = acc_b[h * HALF + vec];
        a.x += df[4 * h] * xf[4 * h]; a.y += df[4 * h + 1] * xf[4 * h + 1]; a.z += df[4 * h + 2] * xf[4 * h + 2]; a.w += df[4 * h + 3] * xf[4 * h + 3];
        b.x += df[4 * h]; b.y += df[4 * h + 1]; b.z += df[4 * h + 2]; b.w += df[4 * h + 3];
        acc_g[h * HALF + vec] = a;
        acc_b[h * HALF + vec] = b;
        if (part_c) {
          float4 c = acc_c[h * HALF + vec];
          c.x += of[4 * h]; c.y += of[4 * h + 1]; c.z += of[4 * h + 2]; c.w += of[4 * h + 3];
          acc_c[h * HALF + vec] = c;
        }
      }
    }
  }
  __syncthreads();
  const int narr = part_c ? 3 : 2;
  for (int i = threadIdx.x; i < narr * (D / 4); i += 256) {
    const int arr = i / (D / 4), idx = i % (D / 4);
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float4 v = reinterpret_cast<const float4*>(ln_acc + (w * 3 + arr) * D)[idx];
      t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
    }
    const int h = idx / HALF, vec = idx % HALF;
    float* dst = (arr == 0 ? part_g : (arr == 1 ? part_b : part_c)) + static_cast<long long>(blockIdx.x) * D + vec * 8 + h * 4;
    *reinterpret_cast<float4*>(dst) = t;
  }
}

// Adds the partial rows of up to three arrays [nparts, D] column by column into bf16 vectors of length D.  A CTA owns
// 32 columns; its 32 warps each walk every 32nd partial row, so the rows are read 32 at a time with full coalescing.
struct ReduceJob {
  const float* part[3];
  __nv_bfloat16* out[3];
  int n;
};

__global__ void __launch_bounds__(1024) partial_rows_reduce_kernel(ReduceJob job, int nparts, int D) {
  __shared__ float sm[3][32][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  float acc[3] = {0.f, 0.f, 0.f};
  if (col < D) {
    for (int p = warp; p < nparts; p += 32) {
#pragma unroll
      for (int a = 0; a < 3; ++a)
        if (a < job.n) acc[a] += job.part[a][static_cast<long long>(p) * D + col];
    }
  }
#pragma unroll
  for (int a = 0; a < 3; ++a) sm[a][warp][lane] = acc[a];
  __syncthreads();
  if (warp < job.n && col < D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += sm[warp][k][lane];
    job.out[warp][col] = __float2bfloat16_rn(t);
  }
}

// Column sums of a bf16 matrix [rows, N] (row stride ld): the bias gradient of a linear layer whose output gradient
// comes from elsewhere.  A CTA owns 256 columns (one 16-byte vector per lane, 8 warps = 8 rows at a time) and a block
// of rows; it writes one partial row, which partial_rows_reduce_kernel adds up.
__global__ void __launch_bounds__(256) colsum_partial_kernel(const __nv_bfloat16* __restrict__ x, long long ld, long long rows, int N,
                                                             int rows_per_part, float* __restrict__ part) {
  __shared__ float sm[8][256 + 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_part;
  const long long r1 = r0 + rows_per_part < rows ? r0 + rows_per_part : rows;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < N) {
    long long r = r0 + warp;
    for (; r + 24 < r1; r += 32) {         // four independent loads in flight
      float a[8], b[8], c[8], d[8];
      const Vec16 va = ld16(x + r * ld + col), vb = ld16(x + (r + 8) * ld + col);
      const Vec16 vc = ld16(x + (r + 16) * ld + col), vd = ld16(x + (r + 24) * ld + col);
      unpack<DT_BF16>(va, a);
      unpack<DT_BF16>(vb, b);
      unpack<DT_BF16>(vc, c);
      unpack<DT_BF16>(vd, d);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += (a[k] + b[k]) + (c[k] + d[k]);
    }
    for (; r < r1; r += 8) {
      float a[8];
      unpack<DT_BF16>(ld16(x + r * ld + col), a);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += a[k];
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) sm[warp][lane * 8 + k] = acc[k];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < N) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sm[w][threadIdx.x];
    part[static_cast<long long>(blockIdx.y) * N + c] = t;
  }
}

}  // namespace

int launchLayerNormFwd(const void* x, const void* delta, void* sum_out, const void* gamma, const void* beta, void* y, float* mean,
                       float* rstd, long long rows, int D, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 8 || D > 8192 || (delta && !sum_out)) return static_cast<int>(cudaErrorInvalidValue);
  auto X = static_cast<const __nv_bfloat16*>(x); auto G = static_cast<const __nv_bfloat16*>(gamma);
  auto B = static_cast<const __nv_bfloat16*>(beta); auto Y = static_cast<__nv_bfloat16*>(y);
  auto DL = static_cast<const __nv_bfloat16*>(delta); auto S = static_cast<__nv_bfloat16*>(sum_out);
  const unsigned grid = static_cast<unsigned>(rows);
  if (D <= 2048) ln_fwd_kernel<1><<<grid, 256, 0, stream>>>(X, DL, S, G, B, Y, mean, rstd, D, eps);
  else if (D <= 4096) ln_fwd_kernel<2><<<grid, 256, 0, stream>>>(X, DL, S, G, B, Y, mean, rstd, D, eps);
  else ln_fwd_kernel<4><<<grid, 256, 0, stream>>>(X, DL, S, G, B, Y, mean, rstd, D, eps);
  return static_cast<int>(cudaGetLastError());
}

int layerNormBwdParts(long long rows) { return static_cast<int>(rows < 148 * 8 ? rows : 148 * 8); }

int launchLayerNormBwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dres, void* dx,
                       void* dgamma, void* dbeta, void* dcolsum, float* partials, long long rows, int D, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 8 || D > 8192) return static_cast<int>(cudaErrorInvalidValue);
  const int parts = layerNormBwdParts(rows);
  float* pg = partials;
  float* pb = partials + static_cast<long long>(parts) * D;
  float* pc = dcolsum ? partials + 2ll * parts * D : nullptr;
  auto DY = static_cast<const __nv_bfloat16*>(dy); auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const __nv_bfloat16*>(gamma); auto DX = static_cast<__nv_bfloat16*>(dx);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  int nparts = parts;
  const int nv = D / 256;
  if (D % 256 == 0 && (nv == 1 || nv == 2 || nv == 4 || nv == 8)) {
    // one warp per row, one CTA per SM
    const int grid = static_cast<int>(rows < 148 * 8 ? (rows + 7) / 8 : 148);
    const size_t smem = 8ull * 3 * D * sizeof(float) + static_cast<size_t>(D) * 2;
    cudaError_t e = cudaSuccess;
    auto go = [&](auto kern) {
      if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e == cudaSuccess) kern<<<grid, 256, smem, stream>>>(DY, X, G, mean, rstd, DR, DX, pg, pb, pc, rows);
    };
    if (nv == 1) go(ln_bwd_warp_kernel<1>);
    else if (nv == 2) go(ln_bwd_warp_kernel<2>);
    else if (nv == 4) go(ln_bwd_warp_kernel<4>);
    else go(ln_bwd_warp_kernel<8>);
    if (e != cudaSuccess) return static_cast<int>(e);
    nparts = grid;
  } else if (D <= 2048) ln_bwd_kernel<1><<<parts, 256, 0, stream>>>(DY, X, G, mean, rstd, DR, DX, pg, pb, pc, rows, D);
  else if (D <= 4096) ln_bwd_kernel<2><<<parts, 256, 0, stream>>>(DY, X, G, mean, rstd, DR, DX, pg, pb, pc, rows, D);
  else ln_bwd_kernel<4><<<parts, 256, 0, stream>>>(DY, X, G, mean, rstd, DR, DX, pg, pb, pc, rows, D);
  ReduceJob job{{pg, pb, pc}, {static_cast<__nv_bfloat16*>(dgamma), static_cast<__nv_bfloat16*>(dbeta), static_cast<__nv_bfloat16*>(dcolsum)},
                dcolsum ? 3 : 2};
  partial_rows_reduce_kernel<<<(D + 31) / 32, 1024, 0, stream>>>(job, nparts, D);
  return static_cast<int>(cudaGetLastError());
}

int colSumParts(long long rows) { return static_cast<int>((rows + 255) / 256 < 64 ? (rows + 255) / 256 : 64); }

int launchColSum(const void* x, long long ld, long long rows, int N, void* out_bf16, float* partials, cudaStream_t stream) {
  if (rows <= 0 || N <= 0) return 0;
  if (N % 8 || ld % 8 || reinterpret_cast<uintptr_t>(x) % 16) return static_cast<int>(cudaErrorInvalidValue);
  const int parts = colSumParts(rows);
  const int rows_per_part = static_cast<int>((rows + parts - 1) / parts);
  dim3 grid((N + 255) / 256, parts);
  colsum_partial_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ld, rows, N, rows_per_part, partials);
  ReduceJob job{{partials, nullptr, nullptr}, {static_cast<__nv_bfloat16*>(out_bf16), nullptr, nullptr}, 1};
  partial_rows_reduce_kernel<<<(N + 31) / 32, 1024, 0, stream>>>(job, parts, N);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace pccl
