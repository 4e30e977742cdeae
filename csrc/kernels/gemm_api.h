// Host entry points of the tcgen05 GEMM family (defined in gemm_*.cu).  Raw pointers, no torch.
// (The reference has no GEMM: cutlass and composable_kernel are empty submodules, .gitmodules:4-9.)
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "api.h"

namespace pccl {

enum GemmFlags : uint32_t {
  GEMM_A_MN = 1u << 0,        // A is the transposed view of a row-major [K, M] tensor
  GEMM_B_MN = 1u << 1,        // B is the transposed view of a row-major [K, N] tensor
  GEMM_OUT_F32 = 1u << 2,     // D is fp32 (default bf16)
  GEMM_ACCUMULATE = 1u << 3,  // D += A*B^T (D is read)
  GEMM_GELU = 1u << 4,        // D2 = gelu_tanh(D) written next to D (D keeps the pre-activation)
  GEMM_BIAS = 1u << 5,        // D = A*B^T + bias[n] (bf16 bias)
  GEMM_GELU_INPLACE = 1u << 6,  // D = gelu_tanh(A*B^T (+bias)); no separate pre-activation
  GEMM_PAIR = 1u << 7,        // CTA pairs (cta_group::2, 256 x 256 tiles) instead of single CTAs (128 x 256)
  GEMM_ADD_D2 = 1u << 8,      // D = A*B^T (+bias) + D2 (bf16, D's layout, read only): a residual connection; not with GEMM_GELU
  GEMM_ROW_STORES = 1u << 9,  // epilogue stores straight from the accumulator layout (a row per lane) instead of through the
                              // coalescing patch: for comparison runs
};

// D[M,N] (ldd) = A * B^T.  K-major operands: A is [M,K] with row stride lda, B is [N,K] with row
// stride ldb.  MN-major operands: A is stored [K,M] (row stride lda), B is stored [K,N] (ldb).
// All strides in elements and multiples of 8; pointers 16-byte aligned.  Asynchronous on `stream`.
// `sms` limits the CTAs (0 = one per SM).  `status` (device, 4 x u32, may be null... must not be
// null) receives ST_TIMEOUT if a pipeline wait runs out.
int gemmBf16(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K,
             uint32_t flags, const void* bias, void* D2, int sms, uint32_t* status, cudaStream_t stream);

// D[M,N] = (A * B^T) .* gelu_tanh'(pre[M,N]) in bf16, and colsum[n] += sum_m D[m,n] (fp32, may be null): the
// backward of "linear -> GELU -> linear" between the second layer's input gradient and the first layer's output
// gradient, with the first layer's bias gradient as a by-product.  `pre` has D's row stride.  CTA pairs; M a multiple
// of 256 and N a multiple of 256; flags: GEMM_A_MN / GEMM_B_MN only.
int gemmBf16Dgelu(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, const void* pre, float* colsum,
                  int M, int N, int K, uint32_t flags, int sms, uint32_t* status, cudaStream_t stream);

// Two GEMMs of the same K and operand forms as ONE launch: their tiles form one list for the persistent CTA pairs, so the
// partly filled last wave is paid once instead of twice (the two weight-gradient GEMMs of an MLP: 256 + 256 tiles on 74
// CTA pairs take 7 rounds instead of 4 + 4).  bf16 or fp32 output; `accumulate` per problem.
struct GemmProblem {
  const void* A; int64_t lda;
  const void* B; int64_t ldb;
  void* D; int64_t ldd;
  int M, N;
  bool accumulate;
};
int gemmBf16Dual(const GemmProblem& p0, const GemmProblem& p1, int K, uint32_t flags, int sms, uint32_t* status, cudaStream_t stream);

// Grouped GEMM for expert layers: group g multiplies rows [row_off[g], row_off[g+1]) of A [*, K] with
// the g-th [N, K] block of B (stacked [groups*N, K]) into the same rows of D [*, N].  `row_off`
// (groups+1 int32) lives on the device, so no host synchronisation is needed to know the sizes.
// flags: GEMM_GELU_INPLACE.
int gemmGroupedBf16(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, const int* row_off,
                    int groups, int max_rows, int N, int K, uint32_t flags, int sms, uint32_t* status, cudaStream_t stream);

// Block-scaled fp8: A is e4m3 [M, K] (row stride lda bytes = elements) with fp32 scales sa [M, ld_sa], one per row and
// 128 values of K; B is e4m3 [N, K] with fp32 scales sb [ceil(N/128), ld_sb], one per 128 x 128 block.
//   D[m, n] = sum_kb sa[m, kb] * sb[n/128, kb] * dot(A[m, kb*128 .. +128], B[n, kb*128 .. +128])
// K a multiple of 128; flags: GEMM_OUT_F32, GEMM_ACCUMULATE, GEMM_GELU, GEMM_BIAS, GEMM_GELU_INPLACE.
int gemmFp8(const void* A, int64_t lda, const float* sa, int ld_sa, const void* B, int64_t ldb, const float* sb, int ld_sb,
            void* D, int64_t ldd, int M, int N, int K, uint32_t flags, const void* bias, void* D2, int sms, uint32_t* status,
            cudaStream_t stream);
const char* gemmFp8LastError();

// fp8 with HARDWARE block scaling (tcgen05 kind::mxf8f6f4.block_scale): like gemmFp8, but the scales are UE8M0 bytes
// (value 2^(byte - 127)): sa [M, ld_sa], sb [ceil(N/128), ld_sb], one byte per 128 values of K.
int gemmMx8(const void* A, int64_t lda, const uint8_t* sa, int ld_sa, const void* B, int64_t ldb, const uint8_t* sb, int ld_sb,
            void* D, int64_t ldd, int M, int N, int K, uint32_t flags, const void* bias, void* D2, int sms, uint32_t* status,
            cudaStream_t stream);
// bf16 -> e4m3 with power-of-two scales: rows [rows, k] -> q + bytes [rows, k/128]; weights [rows, cols] -> q + bytes [rows/128, cols/128]
int launchQuantMx8Rows(const void* x, void* q, uint8_t* scales, long long rows, int k, cudaStream_t stream);
int launchQuantMx8Blocks(const void* w, void* q, uint8_t* scales, int rows, int cols, cudaStream_t stream);
const char* gemmMx8LastError();

const char* gemmLastError();
// Tile scheduling of the CTA-pair kernels: 1 = tiles are handed out at run time (an atomic counter per stream), 0 = fixed
// round-robin lists, -1 = what the environment says (PCCL_GEMM_DYNAMIC, default 1).
void gemmSetDynamic(int mode);
// Zeroes this device's tile counters (after a device synchronisation).  A launch leaves its counter at zero by itself; one
// that gave up on a bounded wait does not, and every later launch on that stream would skip tiles.  The Python status check
// calls this whenever it finds a failure recorded.
int gemmResetTileCounters();

}  // namespace pccl
