// Bindings of the fused collective+GEMM kernels.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "engine.h"
#include "common/env.h"
#include "kernels/fused_api.h"
#include "kernels/gemm_api.h"
#include "kernels/moe_api.h"

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

namespace {
MoeArgs moeArgs(const World& w, int nvirt, int rank, int tokens, int hidden, int topk, int epr, uint64_t recv_q_off,
                uint64_t recv_s_off, uint64_t y_off, uint64_t epoch, int flag_lane, uint64_t spin_ns) {
  MoeArgs a{};
  a.w = w; a.nvirt = nvirt; a.rank = rank; a.tokens = tokens; a.hidden = hidden; a.topk = topk; a.experts_per_rank = epr;
  a.recv_q_off = recv_q_off; a.recv_s_off = recv_s_off; a.y_off = y_off; a.epoch = epoch; a.flag_lane = flag_lane;
  a.spin_ns = spin_ns ? spin_ns : kDefaultSpinLimit;
  return a;
}
}  // namespace

void bindFused(py::module_& m) {
  // ---- MoE ---------------------------------------------------------------------------------------
  // kind: "dispatch" | "combine".  Lists carry one entry per (virtual) rank: 1 in production.
  m.def("moe_exchange", [](const std::string& kind, Engine* e, const std::vector<uint64_t>& heaps, uint64_t flag_off, int tokens,
                           int hidden, int topk, int epr, uint64_t recv_q_off, uint64_t recv_s_off, uint64_t y_off, uint64_t epoch,
                           int flag_lane, const std::vector<uint64_t>& x, const std::vector<uint64_t>& ids,
                           const std::vector<uint64_t>& rows, const std::vector<uint64_t>& probs, const std::vector<uint64_t>& out,
                           const std::vector<uint64_t>& status, int blocks, uint64_t spin_ns, uint64_t stream, uint64_t alias_off,
                           uint64_t group_off, uint64_t z_off, const std::vector<uint64_t>& gate, bool dedupe) {
    MoeArgs a;
    if (e) {
      // barrier values come from the engine's per-lane counter, shared with every other user of the lane
      a = moeArgs(e->worldTable(), 1, e->rank(), tokens, hidden, topk, epr, recv_q_off, recv_s_off, y_off, e->nextEpoch(flag_lane),
                  flag_lane, spin_ns);
    } else {
      a = moeArgs(emuWorld2(heaps, flag_off), static_cast<int>(heaps.size()), 0, tokens, hidden, topk, epr, recv_q_off, recv_s_off,
                  y_off, epoch, flag_lane, spin_ns);
    }
    a.dedupe = dedupe && alias_off != 0 ? 1 : 0;
    a.alias_off = alias_off;
    a.group_off = group_off;
    a.z_off = z_off;
    size_t n = e ? 1 : heaps.size();
    for (size_t r = 0; r < n; ++r) {
      a.gate[r] = gate.empty() ? nullptr : reinterpret_cast<const float*>(gate.at(r));
      a.x[r] = x.empty() ? nullptr : reinterpret_cast<const void*>(x.at(r));
      a.expert_ids[r] = reinterpret_cast<const int*>(ids.at(r));
      a.dst_rows[r] = reinterpret_cast<const int*>(rows.at(r));
      a.probs[r] = probs.empty() ? nullptr : reinterpret_cast<const float*>(probs.at(r));
      a.out[r] = out.empty() ? nullptr : reinterpret_cast<void*>(out.at(r));
      a.status[r] = reinterpret_cast<uint32_t*>(status.at(r));
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int err = kind == "dispatch" ? launchMoeDispatch(a, blocks, st)
              : kind == "combine_dot" ? launchMoeCombineDot(a, blocks, st) : launchMoeCombine(a, blocks, st);
    check(err, kind.c_str());
  }, py::arg("kind"), py::arg("engine").none(true), py::arg("heaps"), py::arg("flag_off"), py::arg("tokens"), py::arg("hidden"),
     py::arg("topk"), py::arg("experts_per_rank"), py::arg("recv_q_off"), py::arg("recv_s_off"), py::arg("y_off"), py::arg("epoch"),
     py::arg("flag_lane"), py::arg("x"), py::arg("ids"), py::arg("rows"), py::arg("probs"), py::arg("out"), py::arg("status"),
     py::arg("blocks"), py::arg("spin_ns"), py::arg("stream"), py::arg("alias_off") = 0, py::arg("group_off") = 0, py::arg("z_off") = 0,
     py::arg("gate") = std::vector<uint64_t>{}, py::arg("dedupe") = false);
  m.def("moe_route", [](uint64_t logits, uint64_t ids, uint64_t probs, uint64_t pos, uint64_t counts, int tokens, int experts, int topk,
                        uint64_t stream) {
    check(launchMoeRoute(reinterpret_cast<const float*>(logits), reinterpret_cast<int*>(ids), reinterpret_cast<float*>(probs),
                         reinterpret_cast<int*>(pos), reinterpret_cast<int*>(counts), tokens, experts, topk,
                         reinterpret_cast<cudaStream_t>(stream)), "moe_route");
  });
  m.def("moe_plan", [](uint64_t counts_all, uint64_t ids, uint64_t pos, uint64_t rows, uint64_t row_off, int world, int rank, int experts,
                       int tokens, int topk, int cap, uint64_t stream) {
    check(launchMoePlan(reinterpret_cast<const int*>(counts_all), reinterpret_cast<const int*>(ids), reinterpret_cast<const int*>(pos),
                        reinterpret_cast<int*>(rows), reinterpret_cast<int*>(row_off), world, rank, experts, tokens, topk, cap,
                        reinterpret_cast<cudaStream_t>(stream)), "moe_plan");
  });
  m.def("moe_dequant", [](uint64_t q, uint64_t s, uint64_t out, uint64_t n_rows, int max_rows, int hidden, uint64_t stream, uint64_t alias) {
    check(launchMoeDequant(reinterpret_cast<const void*>(q), reinterpret_cast<const float*>(s), reinterpret_cast<void*>(out),
                           reinterpret_cast<const int*>(n_rows), max_rows, hidden, reinterpret_cast<const int*>(alias),
                           reinterpret_cast<cudaStream_t>(stream)), "moe_dequant");
  }, py::arg("q"), py::arg("scales"), py::arg("out"), py::arg("n_rows"), py::arg("max_rows"), py::arg("hidden"), py::arg("stream"),
     py::arg("alias") = 0);
  m.def("moe_reduce_groups", [](uint64_t y, uint64_t z, uint64_t alias, uint64_t groups, uint64_t n_rows, int max_rows, int hidden,
                                uint64_t stream) {
    check(launchMoeReduceGroups(reinterpret_cast<const void*>(y), reinterpret_cast<void*>(z), reinterpret_cast<const int*>(alias),
                                reinterpret_cast<const void*>(groups), reinterpret_cast<const int*>(n_rows), max_rows, hidden,
                                reinterpret_cast<cudaStream_t>(stream)), "moe_reduce_groups");
  });
  m.def("quant_fp8_rows", [](uint64_t x, uint64_t q, uint64_t s, long long rows, int hidden, uint64_t stream) {
    check(launchQuantFp8Rows(reinterpret_cast<const void*>(x), reinterpret_cast<void*>(q), reinterpret_cast<float*>(s), rows, hidden,
                             reinterpret_cast<cudaStream_t>(stream)), "quant_fp8_rows");
  });
  m.def("quant_fp8_blocks", [](uint64_t w, uint64_t q, uint64_t s, int rows, int cols, uint64_t stream) {
    check(launchQuantFp8Blocks(reinterpret_cast<const void*>(w), reinterpret_cast<void*>(q), reinterpret_cast<float*>(s), rows, cols,
                               reinterpret_cast<cudaStream_t>(stream)), "quant_fp8_blocks");
  });
  m.def("gemm_grouped", [](uint64_t a, int64_t lda, uint64_t b, int64_t ldb, uint64_t d, int64_t ldd, uint64_t row_off, int groups,
                           int max_rows, int N, int K, uint32_t flags, int sms, uint64_t status, uint64_t stream) {
    check(gemmGroupedBf16(reinterpret_cast<const void*>(a), lda, reinterpret_cast<const void*>(b), ldb, reinterpret_cast<void*>(d), ldd,
                          reinterpret_cast<const int*>(row_off), groups, max_rows, N, K, flags, sms,
                          reinterpret_cast<uint32_t*>(status), reinterpret_cast<cudaStream_t>(stream)), "gemm_grouped");
  });
  m.attr("GEMM_GELU_INPLACE") = static_cast<uint32_t>(GEMM_GELU_INPLACE);

  // ---- production: this process is one rank -------------------------------------------------------
  m.def("ag_gemm", [](Engine& e, uint64_t x_off, int M, int N, int K, uint64_t w, int64_t ldw, uint64_t d, int64_t ldd,
                      uint64_t bias, uint64_t ready, uint64_t epoch, int n_copy, int ctas, int flag_lane, uint64_t status,
                      uint64_t stream, bool b_mn) {
    AgGemmArgs A{};
    A.w = e.worldTable();
    A.nvirt = 1;
    A.M = M; A.N = N; A.K = K; A.M_local = M / e.world();
    A.x_off = x_off; A.epoch = epoch; A.bar_epoch = e.nextEpoch(flag_lane); A.n_copy = n_copy; A.flag_lane = flag_lane;
    A.spin_ns = kDefaultSpinLimit;
    A.tail_tiles = static_cast<int>(LaunchEnvironments::getInt("PCCL_AG_TAIL", -1));     // -1: from the cost model
    A.flags = bias ? GEMM_BIAS : 0;
    A.r[0].D = reinterpret_cast<void*>(d); A.r[0].ldd = ldd; A.r[0].bias = reinterpret_cast<const void*>(bias);
    A.ready_off = ready; A.r[0].status = reinterpret_cast<uint32_t*>(status);
    A.r[0].rank = e.rank();
    AgGemmHost h{reinterpret_cast<const void*>(w), ldw, b_mn};
    check(launchAgGemm(A, &h, ctas, reinterpret_cast<cudaStream_t>(stream)), "ag_gemm");
  }, py::arg("engine"), py::arg("x_off"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("w"), py::arg("ldw"), py::arg("d"), py::arg("ldd"),
     py::arg("bias"), py::arg("ready"), py::arg("epoch"), py::arg("n_copy"), py::arg("ctas"), py::arg("flag_lane"), py::arg("status"),
     py::arg("stream"), py::arg("b_mn") = false);
  m.def("gemm_rs", [](Engine& e, uint64_t y, int64_t ldy, uint64_t w, int64_t ldw, uint64_t out, int64_t ldo, int M, int N, int K,
                      uint64_t stage_off, uint64_t flag_off2, uint64_t epoch, int ctas, uint64_t status, uint64_t stream, bool b_mn) {
    GemmRsArgs A{};
    A.w = e.worldTable();
    A.nvirt = 1;
    A.M = M; A.N = N; A.K = K; A.M_local = M / e.world();
    A.stage_off = stage_off; A.flag_off2 = flag_off2; A.epoch = epoch; A.spin_ns = kDefaultSpinLimit;
    A.r[0].out = reinterpret_cast<void*>(out); A.r[0].ldo = ldo; A.r[0].status = reinterpret_cast<uint32_t*>(status);
    A.r[0].rank = e.rank();
    GemmRsHost h{reinterpret_cast<const void*>(y), ldy, reinterpret_cast<const void*>(w), ldw, b_mn};
    check(launchGemmRs(A, &h, ctas, reinterpret_cast<cudaStream_t>(stream)), "gemm_rs");
  }, py::arg("engine"), py::arg("y"), py::arg("ldy"), py::arg("w"), py::arg("ldw"), py::arg("out"), py::arg("ldo"), py::arg("M"), py::arg("N"),
     py::arg("K"), py::arg("stage_off"), py::arg("flag_off2"), py::arg("epoch"), py::arg("ctas"), py::arg("status"), py::arg("stream"),
     py::arg("b_mn") = false);
  // ---- block-scaled fp8 forms ------------------------------------------------------------------------
  // One entry per (virtual) rank in the lists; with an engine the lists have one entry and the world is the engine's.
  m.def("ag_gemm_fp8", [](Engine* e, const std::vector<uint64_t>& heaps, uint64_t flag_off, uint64_t x_off, uint64_t xs_off, int M, int N,
                          int K, const std::vector<uint64_t>& w, int64_t ldw, const std::vector<uint64_t>& w_scale, int ld_ws,
                          const std::vector<uint64_t>& d, int64_t ldd, const std::vector<uint64_t>& dq, const std::vector<uint64_t>& ds,
                          int64_t ldq, uint64_t bias, uint32_t flags, uint64_t ready_off, uint64_t epoch, int n_copy, int ctas,
                          int flag_lane, const std::vector<uint64_t>& status, uint64_t spin_ns, uint64_t stream, bool mx) {
    AgGemmArgs A{};
    const int n = e ? 1 : static_cast<int>(heaps.size());
    A.w = e ? e->worldTable() : emuWorld2(heaps, flag_off);
    A.nvirt = e ? 1 : n;
    A.M = M; A.N = N; A.K = K; A.M_local = M / A.w.world;
    A.x_off = x_off; A.xs_off = xs_off; A.elem_bytes = 1; A.ready_off = ready_off; A.epoch = epoch;
    A.bar_epoch = e ? e->nextEpoch(flag_lane) : epoch;
    A.n_copy = n_copy; A.flag_lane = flag_lane; A.spin_ns = spin_ns ? spin_ns : kDefaultSpinLimit;
    A.flags = flags | (bias ? GEMM_BIAS : 0);
    std::vector<AgGemmHost> h(n);
    for (int r = 0; r < n; ++r) {
      A.r[r].D = d.empty() ? nullptr : reinterpret_cast<void*>(d.at(r)); A.r[r].ldd = ldd;
      A.r[r].Dq = dq.empty() ? nullptr : reinterpret_cast<void*>(dq.at(r));
      A.r[r].Ds = ds.empty() ? nullptr : reinterpret_cast<float*>(ds.at(r));
      A.r[r].ldq = ldq;
      A.r[r].bias = reinterpret_cast<const void*>(bias);
      A.r[r].w_scale = reinterpret_cast<const float*>(w_scale.at(r)); A.r[r].ld_ws = ld_ws;
      A.r[r].status = reinterpret_cast<uint32_t*>(status.at(r));
      A.r[r].rank = e ? e->rank() : r;
      h[r] = AgGemmHost{reinterpret_cast<const void*>(w.at(r)), ldw, false};
    }
    check(mx ? launchAgGemmMx8(A, h.data(), ctas, reinterpret_cast<cudaStream_t>(stream))
             : launchAgGemmFp8(A, h.data(), ctas, reinterpret_cast<cudaStream_t>(stream)), "ag_gemm_fp8");
  }, py::arg("engine").none(true), py::arg("heaps"), py::arg("flag_off"), py::arg("x_off"), py::arg("xs_off"), py::arg("M"), py::arg("N"),
     py::arg("K"), py::arg("w"), py::arg("ldw"), py::arg("w_scale"), py::arg("ld_ws"), py::arg("d"), py::arg("ldd"), py::arg("dq"),
     py::arg("ds"), py::arg("ldq"), py::arg("bias"), py::arg("flags"), py::arg("ready_off"), py::arg("epoch"), py::arg("n_copy"),
     py::arg("ctas"), py::arg("flag_lane"), py::arg("status"), py::arg("spin_ns"), py::arg("stream"), py::arg("mx") = false);
  m.def("gemm_rs_fp8", [](Engine* e, const std::vector<uint64_t>& heaps, const std::vector<uint64_t>& y, int64_t ldy,
                          const std::vector<uint64_t>& y_scale, int ld_ys, const std::vector<uint64_t>& w, int64_t ldw,
                          const std::vector<uint64_t>& w_scale, int ld_ws, const std::vector<uint64_t>& out, int64_t ldo, int M, int N,
                          int K, uint64_t stage_off, uint64_t flag_off2, uint64_t epoch, int ctas,
                          const std::vector<uint64_t>& status, uint64_t spin_ns, uint64_t stream) {
    GemmRsArgs A{};
    const int n = e ? 1 : static_cast<int>(heaps.size());
    A.w = e ? e->worldTable() : emuWorld2(heaps, 0);
    A.nvirt = e ? 1 : n;
    A.M = M; A.N = N; A.K = K; A.M_local = M / A.w.world;
    A.stage_off = stage_off; A.flag_off2 = flag_off2; A.epoch = epoch; A.spin_ns = spin_ns ? spin_ns : kDefaultSpinLimit;
    std::vector<GemmRsHost> h(n);
    for (int r = 0; r < n; ++r) {
      A.r[r].out = reinterpret_cast<void*>(out.at(r)); A.r[r].ldo = ldo;
      A.r[r].status = reinterpret_cast<uint32_t*>(status.at(r));
      A.r[r].rank = e ? e->rank() : r;
      A.r[r].y_scale = reinterpret_cast<const float*>(y_scale.at(r)); A.r[r].ld_ys = ld_ys;
      A.r[r].w_scale = reinterpret_cast<const float*>(w_scale.at(r)); A.r[r].ld_ws = ld_ws;
      h[r] = GemmRsHost{reinterpret_cast<const void*>(y.at(r)), ldy, reinterpret_cast<const void*>(w.at(r)), ldw, false};
    }
    check(launchGemmRsFp8(A, h.data(), ctas, reinterpret_cast<cudaStream_t>(stream)), "gemm_rs_fp8");
  }, py::arg("engine").none(true), py::arg("heaps"), py::arg("y"), py::arg("ldy"), py::arg("y_scale"), py::arg("ld_ys"), py::arg("w"),
     py::arg("ldw"), py::arg("w_scale"), py::arg("ld_ws"), py::arg("out"), py::arg("ldo"), py::arg("M"), py::arg("N"), py::arg("K"),
     py::arg("stage_off"), py::arg("flag_off2"), py::arg("epoch"), py::arg("ctas"), py::arg("status"), py::arg("spin_ns"),
     py::arg("stream"));
  // ---- single-GPU emulation of all ranks in one cooperative launch (tests) ------------------------
  m.def("emu_ag_gemm", [](const std::vector<uint64_t>& heaps, uint64_t flag_off, uint64_t x_off, int M, int N, int K,
                          const std::vector<uint64_t>& w, int64_t ldw, const std::vector<uint64_t>& d, int64_t ldd,
                          uint64_t ready_off, uint64_t epoch, int n_copy, int ctas,
                          const std::vector<uint64_t>& status, uint64_t spin_ns, uint64_t stream, int tail_tiles) {
    AgGemmArgs A{};
    A.ready_off = ready_off;
    A.w = emuWorld2(heaps, flag_off);
    int n = A.w.world;
    A.nvirt = n;
    A.M = M; A.N = N; A.K = K; A.M_local = M / n;
    A.x_off = x_off; A.epoch = epoch; A.bar_epoch = epoch; A.n_copy = n_copy; A.flag_lane = 0; A.spin_ns = spin_ns ? spin_ns : kDefaultSpinLimit;
    A.tail_tiles = tail_tiles;
    std::vector<AgGemmHost> h(n);
    for (int r = 0; r < n; ++r) {
      A.r[r].D = reinterpret_cast<void*>(d.at(r)); A.r[r].ldd = ldd;
      A.r[r].status = reinterpret_cast<uint32_t*>(status.at(r));
      A.r[r].rank = r;
      h[r] = AgGemmHost{reinterpret_cast<const void*>(w.at(r)), ldw, false};
    }
    check(launchAgGemm(A, h.data(), ctas, reinterpret_cast<cudaStream_t>(stream)), "emu_ag_gemm");
  }, py::arg("heaps"), py::arg("flag_off"), py::arg("x_off"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("w"), py::arg("ldw"),
     py::arg("d"), py::arg("ldd"), py::arg("ready_off"), py::arg("epoch"), py::arg("n_copy"), py::arg("ctas"), py::arg("status"),
     py::arg("spin_ns"), py::arg("stream"), py::arg("tail_tiles") = -1);
  // time attribution of the fused kernels: a zeroed device buffer of PROBE_WORDS u64 per CTA, or 0 to switch it off
  m.def("fused_set_probe", [](uint64_t ptr) { setFusedProbe(reinterpret_cast<unsigned long long*>(ptr)); });
  m.attr("PROBE_WORDS") = kProbeWords;
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
      h[r] = GemmRsHost{reinterpret_cast<const void*>(y.at(r)), ldy, reinterpret_cast<const void*>(w.at(r)), ldw, false};
    }
    check(launchGemmRs(A, h.data(), ctas, reinterpret_cast<cudaStream_t>(stream)), "emu_gemm_rs");
  });
}
