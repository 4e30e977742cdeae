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

}  // namespace pccl
