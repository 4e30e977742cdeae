// Bindings of the fused collective+GEMM kernels.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "engine.h"
#include "kernels/fused_api.h"
#include "kernels/gemm_api.h"

namespace py = pybind11;
using namespace pccl;

namespace {

World emuWorld2(const std::vector<uint64_t>& heaps, uint64_t flag_off) {
  World w{};
  w.world = static_cast<int>(heaps.size());
  for (size_t r = 0; r < heaps.size(); ++r) w.heap[r] = reinterpret_cast<char*>(heaps[r]);
  w.flag_off = flag_off;
  return w;
}

void check(int err, const char* what) {
  if (err != 0) throw std::runtime_error(std::string(what) + ": " + cudaErrorName(err) + " " + fusedLastError());
}

}  // namespace

void bindFused(py::module_& m) {
  // ---- production: this process is one rank -------------------------------------------------------
  m.def("ag_gemm", [](Engine& e, uint64_t x_off, int M, int N, int K, uint64_t w, int64_t ldw, uint64_t d, int64_t ldd,
                      uint64_t bias, uint64_t ready, uint64_t epoch, int n_copy, int ctas, int flag_lane, uint64_t status,
                      uint64_t stream) {
    AgGemmArgs A{};
    A.w = e.worldTable();
    A.nvirt = 1;
    A.M = M; A.N = N; A.K = K; A.M_local = M / e.world();
    A.x_off = x_off; A.epoch = epoch; A.n_copy = n_copy; A.flag_lane = flag_lane; A.spin_ns = kDefaultSpinLimit;
    A.flags = bias ? GEMM_BIAS : 0;
    A.r[0].D = reinterpret_cast<void*>(d); A.r[0].ldd = ldd; A.r[0].bias = reinterpret_cast<const void*>(bias);
    A.r[0].ready = reinterpret_cast<uint32_t*>(ready); A.r[0].status = reinterpret_cast<uint32_t*>(status);
    A.r[0].rank = e.rank();
    AgGemmHost h{reinterpret_cast<const void*>(w), ldw};
    check(launchAgGemm(A, &h, ctas, reinterpret_cast<cudaStream_t>(stream)), "ag_gemm");
  });
  m.def("gemm_rs", [](Engine& e, uint64_t y, int64_t ldy, uint64_t w, int64_t ldw, uint64_t out, int64_t ldo, int M, int N, int K,
                      uint64_t stage_off, uint64_t flag_off2, uint64_t epoch, int ctas, uint64_t status, uint64_t stream) {
    GemmRsArgs A{};
    A.w = e.worldTable();
    A.nvirt = 1;
    A.M = M; A.N = N; A.K = K; A.M_local = M / e.world();
    A.stage_off = stage_off; A.flag_off2 = flag_off2; A.epoch = epoch; A.spin_ns = kDefaultSpinLimit;
    A.r[0].out = reinterpret_cast<void*>(out); A.r[0].ldo = ldo; A.r[0].status = reinterpret_cast<uint32_t*>(status);
    A.r[0].rank = e.rank();
    GemmRsHost h{reinterpret_cast<const void*>(y), ldy, reinterpret_cast<const void*>(w), ldw};
    check(launchGemmRs(A, &h, ctas, reinterpret_cast<cudaStream_t>(stream)), "gemm_rs");
  });
  // ---- single-GPU emulation of all ranks in one cooperative launch (tests) ------------------------
  m.def("emu_ag_gemm", [](const std::vector<uint64_t>& heaps, uint64_t flag_off, uint64_t x_off, int M, int N, int K,
                          const std::vector<uint64_t>& w, int64_t ldw, const std::vector<uint64_t>& d, int64_t ldd,
                          const std::vector<uint64_t>& ready, uint64_t epoch, int n_copy, int ctas,
                          const std::vector<uint64_t>& status, uint64_t spin_ns, uint64_t stream) {
    AgGemmArgs A{};
    A.w = emuWorld2(heaps, flag_off);
    int n = A.w.world;
    A.nvirt = n;
    A.M = M; A.N = N; A.K = K; A.M_local = M / n;
    A.x_off = x_off; A.epoch = epoch; A.n_copy = n_copy; A.flag_lane = 0; A.spin_ns = spin_ns ? spin_ns : kDefaultSpinLimit;
    std::vector<AgGemmHost> h(n);
    for (int r = 0; r < n; ++r) {
      A.r[r].D = reinterpret_cast<void*>(d.at(r)); A.r[r].ldd = ldd;
      A.r[r].ready = reinterpret_cast<uint32_t*>(ready.at(r)); A.r[r].status = reinterpret_cast<uint32_t*>(status.at(r));
      A.r[r].rank = r;
      h[r] = AgGemmHost{reinterpret_cast<const void*>(w.at(r)), ldw};
    }
    check(launchAgGemm(A, h.data(), ctas, reinterpret_cast<cudaStream_t>(stream)), "emu_ag_gemm");
  });
  m.def("emu_gemm_rs", [](const std::vector<uint64_t>& heaps, const std::vector<uint64_t>& y, int64_t ldy,
                          const std::vector<uint64_t>& w, int64_t ldw, const std::vector<uint64_t>& out, int64_t ldo, int M,
                          int N, int K, uint64_t stage_off, uint64_t flag_off2, uint64_t epoch, int ctas,
                          const std::vector<uint64_t>& status, uint64_t spin_ns, uint64_t stream) {
    GemmRsArgs A{};
    A.w = emuWorld2(heaps, 0);
    int n = A.w.world;
    A.nvirt = n;
    A.M = M; A.N = N; A.K = K; A.M_local = M / n;
    A.stage_off = stage_off; A.flag_off2 = flag_off2; A.epoch = epoch; A.spin_ns = spin_ns ? spin_ns : kDefaultSpinLimit;
    std::vector<GemmRsHost> h(n);
    for (int r = 0; r < n; ++r) {
      A.r[r].out = reinterpret_cast<void*>(out.at(r)); A.r[r].ldo = ldo;
      A.r[r].status = reinterpret_cast<uint32_t*>(status.at(r)); A.r[r].rank = r;
      h[r] = GemmRsHost{reinterpret_cast<const void*>(y.at(r)), ldy, reinterpret_cast<const void*>(w.at(r)), ldw};
    }
    check(launchGemmRs(A, h.data(), ctas, reinterpret_cast<cudaStream_t>(stream)), "emu_gemm_rs");
  });
}
