// Element-wise / row-wise kernels of the training path (AdamW, cross-entropy, LayerNorm).  No counterpart in the reference.
// Host entry points of the memory-bound training kernels (elementwise.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace pccl {

// AdamW step `step` (1-based) on n elements: p/m/v fp32 are updated in place from g * grad_scale,
// and the new parameters are also written as bf16 to p_bf16.
int launchAdamW(float* p, float* m, float* v, const float* g, void* p_bf16, long long n, float lr, float b1, float b2,
                float eps, float wd, int step, float grad_scale, cudaStream_t stream);

// Softmax cross-entropy over bf16 logits [rows, vocab] with row stride ld (multiple of 8):
// loss[row] = logsumexp - logit[target]; the logits are overwritten by
// (softmax - onehot) * grad_scale (rows whose target equals ignore_index get zeros).  Targets must lie in [0, vocab);
// any other value is treated like ignore_index (loss 0, zero gradient, no access outside the row) and, when `status`
// (4 x u32, device, may be null) is given and still clear, recorded there as {ST_BOUNDS, row, target, 0xCE}.
int launchCrossEntropy(void* logits, const long long* targets, float* loss, long long rows, int vocab, long long ld,
                       float grad_scale, long long ignore_index, uint32_t* status, cudaStream_t stream);

// LayerNorm over the last dimension D (multiple of 8, <= 8192) of bf16 [rows, D]; mean / rstd are fp32 [rows].
// With `delta` (bf16 [rows, D], may be null) the norm is taken of s = x + delta and s is stored to `sum_out`:
// the residual connection of a pre-norm block and the norm in one pass.
int launchLayerNormFwd(const void* x, const void* delta, void* sum_out, const void* gamma, const void* beta, void* y, float* mean,
                       float* rstd, long long rows, int D, float eps, cudaStream_t stream);
// Backward: dx bf16 [rows, D] = d(norm input) + dres (bf16 [rows, D], may be null: the gradient on the residual stream);
// dgamma / dbeta bf16 [D]; dcolsum (bf16 [D], may be null) receives the column sums of dx, which is the bias gradient of
// the linear layer that fed the residual sum.  `x` is the norm's input (the stored sum when forward had a delta).
// `partials` is fp32 scratch of 3 * layerNormBwdParts(rows) * D elements.
int layerNormBwdParts(long long rows);
int launchLayerNormBwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dres, void* dx,
                       void* dgamma, void* dbeta, void* dcolsum, float* partials, long long rows, int D, cudaStream_t stream);

// out[n] = sum over rows of x[row, n] for bf16 x [rows, N] with row stride ld (elements, multiple of 8); N a multiple of 8.
// `partials`: fp32 scratch of colSumParts(rows) * N elements.
int colSumParts(long long rows);
int launchColSum(const void* x, long long ld, long long rows, int N, void* out_bf16, float* partials, cudaStream_t stream);

}  // namespace pccl
