// Bindings of the tcgen05 GEMM family (pointers in, nothing allocated here).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>

#include "kernels/elementwise_api.h"
#include "kernels/gemm_api.h"

namespace py = pybind11;
using namespace pccl;

void bindGemm(py::module_& m) {
  m.def("gemm_bf16",
        [](uint64_t a, int64_t lda, uint64_t b, int64_t ldb, uint64_t d, int64_t ldd, int M, int N, int K, uint32_t flags,
           uint64_t bias, uint64_t d2, int sms, uint64_t status, uint64_t stream) {
          int err = gemmBf16(reinterpret_cast<const void*>(a), lda, reinterpret_cast<const void*>(b), ldb,
                             reinterpret_cast<void*>(d), ldd, M, N, K, flags, reinterpret_cast<const void*>(bias),
                             reinterpret_cast<void*>(d2), sms, reinterpret_cast<uint32_t*>(status),
                             reinterpret_cast<cudaStream_t>(stream));
          if (err != 0) throw std::runtime_error(std::string("gemm_bf16: ") + cudaErrorName(err) + " " + gemmLastError());
        },
        py::arg("a"), py::arg("lda"), py::arg("b"), py::arg("ldb"), py::arg("d"), py::arg("ldd"), py::arg("M"),
        py::arg("N"), py::arg("K"), py::arg("flags"), py::arg("bias") = 0, py::arg("d2") = 0, py::arg("sms") = 0,
        py::arg("status") = 0, py::arg("stream") = 0);
  m.def("gemm_bf16_dgelu",
        [](uint64_t a, int64_t lda, uint64_t b, int64_t ldb, uint64_t d, int64_t ldd, uint64_t pre, uint64_t colsum, int M, int N, int K,
           uint32_t flags, int sms, uint64_t status, uint64_t stream) {
          int err = gemmBf16Dgelu(reinterpret_cast<const void*>(a), lda, reinterpret_cast<const void*>(b), ldb, reinterpret_cast<void*>(d),
                                  ldd, reinterpret_cast<const void*>(pre), reinterpret_cast<float*>(colsum), M, N, K, flags, sms,
                                  reinterpret_cast<uint32_t*>(status), reinterpret_cast<cudaStream_t>(stream));
          if (err != 0) throw std::runtime_error(std::string("gemm_bf16_dgelu: ") + cudaErrorName(err) + " " + gemmLastError());
        });
  m.def("gemm_set_dynamic", &gemmSetDynamic);
  m.def("gemm_reset_tile_counters", &gemmResetTileCounters);
  m.def("gemm_bf16_dual",
        [](uint64_t a0, int64_t lda0, uint64_t b0, int64_t ldb0, uint64_t d0, int64_t ldd0, int M0, int N0, bool acc0, uint64_t a1, int64_t lda1,
           uint64_t b1, int64_t ldb1, uint64_t d1, int64_t ldd1, int M1, int N1, bool acc1, int K, uint32_t flags, int sms, uint64_t status,
           uint64_t stream) {
          GemmProblem p0{reinterpret_cast<const void*>(a0), lda0, reinterpret_cast<const void*>(b0), ldb0, reinterpret_cast<void*>(d0), ldd0, M0, N0, acc0};
          GemmProblem p1{reinterpret_cast<const void*>(a1), lda1, reinterpret_cast<const void*>(b1), ldb1, reinterpret_cast<void*>(d1), ldd1, M1, N1, acc1};
          int err = gemmBf16Dual(p0, p1, K, flags, sms, reinterpret_cast<uint32_t*>(status), reinterpret_cast<cudaStream_t>(stream));
          if (err != 0) throw std::runtime_error(std::string("gemm_bf16_dual: ") + cudaErrorName(err) + " " + gemmLastError());
        });
  m.def("gemm_fp8",
        [](uint64_t a, int64_t lda, uint64_t sa, int ld_sa, uint64_t b, int64_t ldb, uint64_t sb, int ld_sb, uint64_t d, int64_t ldd,
           int M, int N, int K, uint32_t flags, uint64_t bias, uint64_t d2, int sms, uint64_t status, uint64_t stream) {
          int err = gemmFp8(reinterpret_cast<const void*>(a), lda, reinterpret_cast<const float*>(sa), ld_sa,
                            reinterpret_cast<const void*>(b), ldb, reinterpret_cast<const float*>(sb), ld_sb,
                            reinterpret_cast<void*>(d), ldd, M, N, K, flags, reinterpret_cast<const void*>(bias),
                            reinterpret_cast<void*>(d2), sms, reinterpret_cast<uint32_t*>(status),
                            reinterpret_cast<cudaStream_t>(stream));
          if (err != 0) throw std::runtime_error(std::string("gemm_fp8: ") + cudaErrorName(err) + " " + gemmFp8LastError());
        },
        py::arg("a"), py::arg("lda"), py::arg("sa"), py::arg("ld_sa"), py::arg("b"), py::arg("ldb"), py::arg("sb"), py::arg("ld_sb"),
        py::arg("d"), py::arg("ldd"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("flags"), py::arg("bias") = 0,
        py::arg("d2") = 0, py::arg("sms") = 0, py::arg("status") = 0, py::arg("stream") = 0);
  m.def("gemm_mx8",
        [](uint64_t a, int64_t lda, uint64_t sa, int ld_sa, uint64_t b, int64_t ldb, uint64_t sb, int ld_sb, uint64_t d, int64_t ldd,
           int M, int N, int K, uint32_t flags, uint64_t bias, uint64_t d2, int sms, uint64_t status, uint64_t stream) {
          int err = gemmMx8(reinterpret_cast<const void*>(a), lda, reinterpret_cast<const uint8_t*>(sa), ld_sa,
                            reinterpret_cast<const void*>(b), ldb, reinterpret_cast<const uint8_t*>(sb), ld_sb,
                            reinterpret_cast<void*>(d), ldd, M, N, K, flags, reinterpret_cast<const void*>(bias),
                            reinterpret_cast<void*>(d2), sms, reinterpret_cast<uint32_t*>(status),
                            reinterpret_cast<cudaStream_t>(stream));
          if (err != 0) throw std::runtime_error(std::string("gemm_mx8: ") + cudaErrorName(err) + " " + gemmMx8LastError());
        },
        py::arg("a"), py::arg("lda"), py::arg("sa"), py::arg("ld_sa"), py::arg("b"), py::arg("ldb"), py::arg("sb"), py::arg("ld_sb"),
        py::arg("d"), py::arg("ldd"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("flags"), py::arg("bias") = 0,
        py::arg("d2") = 0, py::arg("sms") = 0, py::arg("status") = 0, py::arg("stream") = 0);
  m.def("quant_mx8_rows", [](uint64_t x, uint64_t q, uint64_t s, long long rows, int k, uint64_t stream) {
    int err = launchQuantMx8Rows(reinterpret_cast<const void*>(x), reinterpret_cast<void*>(q), reinterpret_cast<uint8_t*>(s), rows, k,
                                 reinterpret_cast<cudaStream_t>(stream));
    if (err != 0) throw std::runtime_error(std::string("quant_mx8_rows: ") + cudaErrorName(err));
  });
  m.def("quant_mx8_blocks", [](uint64_t w, uint64_t q, uint64_t s, int rows, int cols, uint64_t stream) {
    int err = launchQuantMx8Blocks(reinterpret_cast<const void*>(w), reinterpret_cast<void*>(q), reinterpret_cast<uint8_t*>(s), rows, cols,
                                   reinterpret_cast<cudaStream_t>(stream));
    if (err != 0) throw std::runtime_error(std::string("quant_mx8_blocks: ") + cudaErrorName(err));
  });
  m.def("adamw", [](uint64_t p, uint64_t mm, uint64_t v, uint64_t g, uint64_t pb, long long n, float lr, float b1, float b2,
                    float eps, float wd, int step, float grad_scale, uint64_t stream) {
    int err = launchAdamW(reinterpret_cast<float*>(p), reinterpret_cast<float*>(mm), reinterpret_cast<float*>(v),
                          reinterpret_cast<const float*>(g), reinterpret_cast<void*>(pb), n, lr, b1, b2, eps, wd, step,
                          grad_scale, reinterpret_cast<cudaStream_t>(stream));
    if (err != 0) throw std::runtime_error(std::string("adamw: ") + cudaErrorName(err));
  });
  m.def("cross_entropy", [](uint64_t logits, uint64_t targets, uint64_t loss, long long rows, int vocab, long long ld,
                            float grad_scale, long long ignore_index, uint64_t status, uint64_t stream) {
    int err = launchCrossEntropy(reinterpret_cast<void*>(logits), reinterpret_cast<const long long*>(targets),
                                 reinterpret_cast<float*>(loss), rows, vocab, ld, grad_scale, ignore_index,
                                 reinterpret_cast<uint32_t*>(status), reinterpret_cast<cudaStream_t>(stream));
    if (err != 0) throw std::runtime_error(std::string("cross_entropy: ") + cudaErrorName(err));
  });
  m.def("layernorm_fwd", [](uint64_t x, uint64_t delta, uint64_t sum_out, uint64_t g, uint64_t b, uint64_t y, uint64_t mean, uint64_t rstd,
                            long long rows, int D, float eps, uint64_t stream) {
    int err = launchLayerNormFwd(reinterpret_cast<const void*>(x), reinterpret_cast<const void*>(delta), reinterpret_cast<void*>(sum_out),
                                 reinterpret_cast<const void*>(g), reinterpret_cast<const void*>(b), reinterpret_cast<void*>(y),
                                 reinterpret_cast<float*>(mean), reinterpret_cast<float*>(rstd), rows, D, eps,
                                 reinterpret_cast<cudaStream_t>(stream));
    if (err != 0) throw std::runtime_error(std::string("layernorm_fwd: ") + cudaErrorName(err));
  });
  m.def("layernorm_bwd_parts", &layerNormBwdParts);
  m.def("layernorm_bwd", [](uint64_t dy, uint64_t x, uint64_t g, uint64_t mean, uint64_t rstd, uint64_t dres, uint64_t dx, uint64_t dg,
                            uint64_t db, uint64_t dcolsum, uint64_t partials, long long rows, int D, uint64_t stream) {
    int err = launchLayerNormBwd(reinterpret_cast<const void*>(dy), reinterpret_cast<const void*>(x), reinterpret_cast<const void*>(g),
                                 reinterpret_cast<const float*>(mean), reinterpret_cast<const float*>(rstd),
                                 reinterpret_cast<const void*>(dres), reinterpret_cast<void*>(dx), reinterpret_cast<void*>(dg),
                                 reinterpret_cast<void*>(db), reinterpret_cast<void*>(dcolsum), reinterpret_cast<float*>(partials), rows, D,
                                 reinterpret_cast<cudaStream_t>(stream));
    if (err != 0) throw std::runtime_error(std::string("layernorm_bwd: ") + cudaErrorName(err));
  });
  m.def("colsum_parts", &colSumParts);
  m.def("colsum", [](uint64_t x, long long ld, long long rows, int N, uint64_t out, uint64_t partials, uint64_t stream) {
    int err = launchColSum(reinterpret_cast<const void*>(x), ld, rows, N, reinterpret_cast<void*>(out), reinterpret_cast<float*>(partials),
                           reinterpret_cast<cudaStream_t>(stream));
    if (err != 0) throw std::runtime_error(std::string("colsum: ") + cudaErrorName(err));
  });
  m.attr("GEMM_A_MN") = static_cast<uint32_t>(GEMM_A_MN);
  m.attr("GEMM_B_MN") = static_cast<uint32_t>(GEMM_B_MN);
  m.attr("GEMM_OUT_F32") = static_cast<uint32_t>(GEMM_OUT_F32);
  m.attr("GEMM_ACCUMULATE") = static_cast<uint32_t>(GEMM_ACCUMULATE);
  m.attr("GEMM_GELU") = static_cast<uint32_t>(GEMM_GELU);
  m.attr("GEMM_BIAS") = static_cast<uint32_t>(GEMM_BIAS);
  m.attr("GEMM_PAIR") = static_cast<uint32_t>(GEMM_PAIR);
  m.attr("GEMM_ADD_D2") = static_cast<uint32_t>(GEMM_ADD_D2);
  m.attr("GEMM_ROW_STORES") = static_cast<uint32_t>(GEMM_ROW_STORES);
}
