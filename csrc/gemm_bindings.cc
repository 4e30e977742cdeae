// Bindings of the tcgen05 GEMM family (pointers in, nothing allocated here).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>

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
  m.attr("GEMM_A_MN") = static_cast<uint32_t>(GEMM_A_MN);
  m.attr("GEMM_B_MN") = static_cast<uint32_t>(GEMM_B_MN);
  m.attr("GEMM_OUT_F32") = static_cast<uint32_t>(GEMM_OUT_F32);
  m.attr("GEMM_ACCUMULATE") = static_cast<uint32_t>(GEMM_ACCUMULATE);
  m.attr("GEMM_GELU") = static_cast<uint32_t>(GEMM_GELU);
  m.attr("GEMM_BIAS") = static_cast<uint32_t>(GEMM_BIAS);
}
