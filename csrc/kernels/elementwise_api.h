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
// (softmax - onehot) * grad_scale (rows whose target equals ignore_index get zeros).
int launchCrossEntropy(void* logits, const long long* targets, float* loss, long long rows, int vocab, long long ld,
                       float grad_scale, long long ignore_index, cudaStream_t stream);

// LayerNorm over the last dimension D (multiple of 8, <= 8192) of bf16 [rows, D]; mean / rstd are fp32 [rows].
int launchLayerNormFwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, long long rows, int D,
                       float eps, cudaStream_t stream);
// Backward: dx bf16 [rows, D], dgamma / dbeta bf16 [D]; `partials` is fp32 scratch of 2 * layerNormBwdParts(rows) * D elements.
int layerNormBwdParts(long long rows);
int launchLayerNormBwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx, void* dgamma,
                       void* dbeta, float* partials, long long rows, int D, cudaStream_t stream);

}  // namespace pccl
