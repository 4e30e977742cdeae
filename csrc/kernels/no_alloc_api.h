// Allocation-free entry point (this has no counterpart in the reference, which has no kernels).
//
// Who needs it: callers that must not, or cannot, allocate device memory at the moment they need a
// loss value -- a serving or training runtime that handed all of the GPU's memory to its own arena
// at start-up (so cudaMalloc would fail), code that runs where allocation is forbidden by its
// host framework's rules, or a plugin that may only touch the buffers it is given.  The regular
// path (launchCrossEntropy + a sum in PyTorch) allocates a per-row loss buffer on every call.
//
// pccl_cross_entropy_mean_noalloc computes the mean softmax cross-entropy of bf16 logits and, like
// the regular kernel, overwrites the logits with their gradient (softmax - onehot) / rows.  Its only
// scratch, one fp32 loss per row, lives in a static device array inside the library:
//   * capacity PCCL_NOALLOC_MAX_ROWS rows (256 KiB per GPU that loads the library, held until the
//     process exits); more rows are rejected with PCCL_NOALLOC_TOO_LARGE and nothing is launched;
//   * the first call on each device resolves the array's device address (cudaGetSymbolAddress, with
//     that device current) -- make that first call outside any stream capture;
//   * it calls no cudaMalloc / cudaFree and no allocating library routine;
//   * all calls on a device share the array: two calls that overlap on the GPU (different streams)
//     race on it.  Nothing in it needs to start at zero: every launch rewrites the rows it then sums;
//   * targets must lie in [0, vocab).  There is no ignore value to pass: a target outside that range (the
//     customary -100 included) makes an ignored row -- its loss is 0, its gradient is all zeros, nothing outside the
//     row is read -- and the mean is still taken over all `rows`;
//   * the per-device set-up state is written without a lock: two host threads that make the first call on one
//     device at the same moment both store the same values, which is harmless.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PCCL_NOALLOC_MAX_ROWS 65536

enum {
  PCCL_NOALLOC_OK = 0,
  PCCL_NOALLOC_TOO_LARGE = -1,      // rows > PCCL_NOALLOC_MAX_ROWS
  PCCL_NOALLOC_BAD_ARGUMENT = -2,   // null pointer, vocab too large for one CTA's shared memory, misaligned logits
  PCCL_NOALLOC_CUDA_ERROR = -3      // a CUDA call failed; see pccl_noalloc_last_cuda_error()
};

// logits: device, bf16 [rows, vocab] with row stride `ld` elements (multiple of 8, base 16-byte aligned)
// targets: device, int64 [rows], each in [0, vocab) (anything else: ignored row, see above); mean_loss: device, one float (output)
// Asynchronous on `stream`.  Returns one of the codes above.
__attribute__((visibility("default")))
int pccl_cross_entropy_mean_noalloc(void* logits, const long long* targets, float* mean_loss, long long rows, int vocab,
                                    long long ld, cudaStream_t stream);

__attribute__((visibility("default")))
int pccl_noalloc_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
