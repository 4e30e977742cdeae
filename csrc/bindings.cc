// Python bindings (pybind11, no torch headers: tensors cross the boundary as data_ptr() integers
// and the CUDA stream as its handle).  Module layout follows the reference's
// (csrc/python_api.cc:10-28): class Engine with initEngine / regOp / exeOp / exportEndpoint /
// joinCluster / exitCluster, and a `utils` submodule with LaunchEnvironments.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cuda_runtime.h>

#include <cmath>
#include <map>

#include "base/registry.h"
#include "common/clock.h"
#include "common/env.h"
#include "common/hash.h"
#include "common/hex.h"
#include "common/json.h"
#include "common/log.h"
#include "engine.h"
#include "exec/reduce_cpu.h"
#include "kernels/api.h"
#include "kernels/gemm_api.h"

namespace py = pybind11;
using namespace pccl;

namespace {

void throwIfCuda(int err, const char* what) {
  if (err != 0) throw std::runtime_error(std::string(what) + ": " + cudaErrorName(err));
}

CollArgs makeCollArgs(const World& w, int nvirt, int rank, const std::string& algo, const std::string& dtype,
                      const std::string& redop, uint64_t in_off, uint64_t out_off, uint64_t count, uint64_t epoch,
                      int flag_lane, float scale, const std::string& out_dtype, uint64_t spin_limit) {
  CollArgs a{};
  a.w = w;
  a.nvirt = nvirt;
  a.rank = rank;
  a.algo = algo == "nvls" ? ALGO_NVLS : ALGO_P2P;
  a.dtype = parseDType(dtype);
  a.redop = parseRedOp(redop);
  a.in_off = in_off;
  a.out_off = out_off;
  a.count = count;
  a.epoch = epoch;
  a.flag_lane = flag_lane;
  a.scale = scale;
  a.out_dtype = out_dtype.empty() ? a.dtype : parseDType(out_dtype);
  a.spin_limit = spin_limit ? spin_limit : kDefaultSpinLimit;
  return a;
}

int launchKind(const std::string& kind, const CollArgs& a, int blocks, int threads, cudaStream_t s) {
  if (kind == "allreduce") return launchAllReduce(a, blocks, threads, s);
  if (kind == "reduce_scatter") return launchReduceScatter(a, blocks, threads, s);
  if (kind == "allgather") return launchAllGather(a, blocks, threads, s);
  if (kind == "alltoall") return launchAllToAll(a, blocks, threads, s);
  if (kind == "allreduce_fp8") return launchAllReduceFp8(a, blocks, threads, s);
  if (kind == "reduce_scatter_fp8") return launchReduceScatterFp8(a, blocks, threads, s);
  throw std::runtime_error("unknown collective '" + kind + "'");
}

// Production path: this process is rank engine.rank() of engine.world().
void collective(Engine& e, const std::string& kind, const std::string& algo, const std::string& dtype,
                const std::string& redop, uint64_t in_off, uint64_t out_off, uint64_t count, int flag_lane,
                float scale, const std::string& out_dtype, int blocks, int threads, uint64_t stream,
                uint64_t local_in, uint64_t local_out, uint64_t spin_limit, uint64_t s_in_off, uint64_t s_out_off) {
  CollArgs a = makeCollArgs(e.worldTable(), 1, e.rank(), algo, dtype, redop, in_off, out_off, count,
                            e.nextEpoch(flag_lane), flag_lane, scale, out_dtype, spin_limit);
  a.s_in_off = s_in_off;
  a.s_out_off = s_out_off;
  a.status[0] = reinterpret_cast<uint32_t*>(e.statusPtr(8 + flag_lane));
  a.local_in[0] = reinterpret_cast<const void*>(local_in);
  a.local_out[0] = reinterpret_cast<void*>(local_out);
  if (flag_lane >= 0 && flag_lane < kLlLanes && e.layout().ll_off && LaunchEnvironments::getBool("PCCL_LL", true))
    a.ll_off = e.layout().ll_off + static_cast<uint64_t>(flag_lane) * kLlLaneBytes;
  throwIfCuda(launchKind(kind, a, blocks, threads, reinterpret_cast<cudaStream_t>(stream)), kind.c_str());
}

World emuWorld(const std::vector<uint64_t>& heaps, uint64_t signal_off, uint64_t flag_off) {
  if (heaps.empty() || heaps.size() > kMaxRanks) throw std::runtime_error("emulated world: 1..16 heaps");
  World w{};
  w.world = static_cast<int>(heaps.size());
  for (size_t r = 0; r < heaps.size(); ++r) w.heap[r] = reinterpret_cast<char*>(heaps[r]);
  w.signal_off = signal_off;
  w.flag_off = flag_off;
  return w;
}

// Single-GPU emulation: all ranks' heaps are buffers of one GPU, one cooperative launch plays every rank.
void emuCollective(const std::string& kind, const std::vector<uint64_t>& heaps, uint64_t signal_off, uint64_t flag_off,
                   const std::string& dtype, const std::string& redop, uint64_t in_off, uint64_t out_off, uint64_t count,
                   uint64_t epoch, int flag_lane, float scale, const std::string& out_dtype, int blocks, int threads,
                   uint64_t stream, const std::vector<uint64_t>& status, const std::vector<uint64_t>& local_in,
                   const std::vector<uint64_t>& local_out, uint64_t spin_limit, uint64_t s_in_off, uint64_t s_out_off, uint64_t ll_off) {
  World w = emuWorld(heaps, signal_off, flag_off);
  CollArgs a = makeCollArgs(w, w.world, 0, "p2p", dtype, redop, in_off, out_off, count, epoch, flag_lane, scale, out_dtype, spin_limit);
  a.s_in_off = s_in_off;
  a.s_out_off = s_out_off;
  a.ll_off = ll_off;
  for (int r = 0; r < w.world; ++r) {
    a.status[r] = reinterpret_cast<uint32_t*>(status.at(r));
    a.local_in[r] = local_in.empty() ? nullptr : reinterpret_cast<const void*>(local_in.at(r));
    a.local_out[r] = local_out.empty() ? nullptr : reinterpret_cast<void*>(local_out.at(r));
  }
  throwIfCuda(launchKind(kind, a, blocks, threads, reinterpret_cast<cudaStream_t>(stream)), kind.c_str());
}

// Runs a schedule document for every rank of an emulated world on one GPU.  `skip_ranks` lists
// ranks whose streams are left out, which makes their peers' waits run out: the bounded-wait test.
void emuProgram(const std::string& schedule_json, const std::vector<uint64_t>& heaps, uint64_t signal_off,
                const std::vector<uint64_t>& inputs, const std::vector<uint64_t>& outputs, uint64_t in_bytes,
                const std::string& dtype, int width, uint64_t scratch_off, uint32_t slot_base, uint64_t epoch,
                uint64_t spin_limit, const std::vector<uint64_t>& status, const std::vector<int>& skip_ranks,
                uint64_t stream) {
  Program p = Program::fromJson(Json::parse(schedule_json));
  World w = emuWorld(heaps, signal_off, 0);
  if (p.world != w.world) throw std::runtime_error("emulated program: world size mismatch");
  InterpLaunch L{};
  L.w = w;
  L.nvirt = w.world;
  L.slot_base = slot_base;
  L.epoch = epoch;
  L.dtype = parseDType(dtype);
  L.redop = parseRedOp(p.redop);
  L.spin_limit = spin_limit ? spin_limit : kDefaultSpinLimit;
  L.bounds_check = 1;
  uint64_t bb = p.blockBytesForInput(in_bytes);
  std::vector<void*> to_free;
  auto cleanup = [&] { for (void* q : to_free) cudaFree(q); };
  try {
    for (int r = 0; r < w.world; ++r) {
      Materialized m = p.materialize(r, bb, width);
      bool skip = false;
      for (int s : skip_ranks) skip = skip || s == r;
      std::vector<Instr> flat;
      std::vector<uint32_t> starts;
      if (!skip)
        for (auto& s : m.streams) {
          starts.push_back(static_cast<uint32_t>(flat.size()));
          flat.insert(flat.end(), s.begin(), s.end());
        }
      InterpRank& R = L.r[r];
      R.rank = r;
      R.n_streams = static_cast<int>(starts.size());
      if (!flat.empty()) {
        flat.resize(flat.size() + kInstrPad, Instr{});      // the kernel reads whole chunks: no-ops behind the last stream
        Instr* di = nullptr;
        uint32_t* ds = nullptr;
        throwIfCuda(cudaMalloc(&di, flat.size() * sizeof(Instr)), "cudaMalloc");
        to_free.push_back(di);
        throwIfCuda(cudaMalloc(&ds, starts.size() * sizeof(uint32_t)), "cudaMalloc");
        to_free.push_back(ds);
        throwIfCuda(cudaMemcpy(di, flat.data(), flat.size() * sizeof(Instr), cudaMemcpyHostToDevice), "cudaMemcpy");
        throwIfCuda(cudaMemcpy(ds, starts.data(), starts.size() * sizeof(uint32_t), cudaMemcpyHostToDevice), "cudaMemcpy");
        R.instrs = di;
        R.stream_start = ds;
      }
      R.input = reinterpret_cast<char*>(inputs.at(r));
      R.output = reinterpret_cast<char*>(p.in_place ? inputs.at(r) : outputs.at(r));
      auto heapOff = [&](uint64_t ptr) -> long long {
        return (ptr >= heaps[r] && ptr - heaps[r] < (1ull << 40)) ? static_cast<long long>(ptr - heaps[r]) : -1;
      };
      R.input_heap_off = p.remote_io ? heapOff(inputs.at(r)) : -1;
      R.output_heap_off = p.remote_io ? heapOff(p.in_place ? inputs.at(r) : outputs.at(r)) : -1;
      R.scratch_off = scratch_off;
      for (int b = 0; b < static_cast<int>(BUF_COUNT); ++b) R.buf_bytes[b] = m.buf_bytes[b];
      R.status = reinterpret_cast<uint32_t*>(status.at(r));
    }
    throwIfCuda(launchInterpreter(L, 256, reinterpret_cast<cudaStream_t>(stream)), "interpreter launch");
    throwIfCuda(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)), "interpreter run");
  } catch (...) {
    cleanup();
    throw;
  }
  cleanup();
}

py::dict layoutDict(const Engine& e) {
  const HeapLayout& L = e.layout();
  py::dict d;
  d["workspace_bytes"] = L.workspace_bytes;
  d["signal_off"] = L.signal_off;
  d["num_signals"] = L.num_signals;
  d["flag_off"] = L.flag_off;
  d["status_off"] = L.status_off;
  d["user_off"] = L.user_off;
  d["total"] = L.total;
  d["lanes"] = L.lanes;
  return d;
}

}  // namespace

void bindGemm(py::module_& m);    // gemm_bindings.cc
void bindFused(py::module_& m);   // fused_bindings.cc

PYBIND11_MODULE(_C, m) {
  m.doc() = "pccl_b200 native runtime";
  registerBuiltinOptions();

  py::class_<Engine>(m, "Engine")
      .def(py::init<int, int>(), py::arg("rank"), py::arg("world"))
      .def("initEngine", &Engine::initEngine, py::arg("device") = "auto", py::arg("heap_bytes") = 0)
      .def("regOp", &Engine::regOp, py::arg("name"), py::arg("path_or_json"))
      .def("exeOp", &Engine::exeOp, py::arg("name"), py::arg("in_ptr"), py::arg("out_ptr"), py::arg("in_bytes"),
           py::arg("dtype"), py::arg("width") = 1, py::arg("lane") = 0, py::arg("stream") = 0,
           py::call_guard<py::gil_scoped_release>())
      .def("prepareOp", &Engine::prepareOp, py::arg("name"), py::arg("width") = 1)
      .def("exportEndpoint", &Engine::exportEndpoint)
      .def("importEndpoints", &Engine::importEndpoints, py::call_guard<py::gil_scoped_release>())
      .def("joinCluster", &Engine::joinCluster, py::arg("master_endpoint"), py::arg("timeout_ms") = 60000,
           py::call_guard<py::gil_scoped_release>())
      .def("exitCluster", &Engine::exitCluster, py::call_guard<py::gil_scoped_release>())
      .def("stats", &Engine::stats)
      .def("trace", &Engine::trace)
      .def("ingestDeviceTrace", &Engine::ingestDeviceTrace, py::arg("name"), py::arg("in_bytes"), py::arg("width"), py::arg("stamps"))
      .def("deviceKind", &Engine::deviceKind)
      .def("heapBase", &Engine::heapBase)
      .def("heapBytes", &Engine::heapBytes)
      .def("allocSymmetric", &Engine::allocSymmetric, py::arg("bytes"), py::arg("align") = 256)
      .def("resetSymmetric", &Engine::resetSymmetric)
      .def("symmetricMark", &Engine::symmetricMark)
      .def("layout", &layoutDict)
      .def("multicastSupported", &Engine::multicastSupported)
      .def("mcCreate", &Engine::mcCreate)
      .def("mcJoin", &Engine::mcJoin)
      .def("mcBind", &Engine::mcBind)
      .def("mcBase", &Engine::mcBase)
      .def("checkStatus", &Engine::checkStatus, py::arg("lane") = 0)
      .def("statusPtr", &Engine::statusPtr)
      .def("aliveRanks", &Engine::aliveRanks)
      .def("resizeWorld", &Engine::resizeWorld)
      .def("lastResize", &Engine::lastResize)
      .def("waitForDeparture", &Engine::waitForDeparture, py::call_guard<py::gil_scoped_release>())
      .def("rebind", &Engine::rebind)
      .def("injectFault", &Engine::injectFault)
      .def("nextEpoch", &Engine::nextEpoch)
      .def("mixedHosts", &Engine::mixedHosts)
      .def("materializedStreams", [](Engine& e, const std::string& name, uint64_t in_bytes, int width) {
        uint64_t bb[BUF_COUNT] = {0, 0, 0};
        auto streams = e.materializedStreams(name, in_bytes, width, bb);
        py::list out;
        for (auto& s : streams) {
          py::list one;
          for (auto& in : s)
            one.append(py::make_tuple(in.op, in.src_rank, in.dst_rank, in.src_buf, in.dst_buf, in.slot, in.value, in.count, in.src_off,
                                      in.dst_off, in.bytes));
          out.append(one);
        }
        return py::make_tuple(out, py::make_tuple(bb[0], bb[1], bb[2]));
      }, py::arg("name"), py::arg("in_bytes"), py::arg("width") = 1)
      .def("opInfo", &Engine::opInfo)
      .def("planLaunch", [](Engine& e, const std::string& name, uint64_t in_bytes, int width, int lane) {
        Engine::LaunchPlan L = e.planLaunch(name, in_bytes, width, lane);
        py::dict d;
        d["slot_base"] = L.slot_base; d["turn_slot"] = L.turn_slot; d["finish_slot"] = L.finish_slot; d["epoch"] = L.epoch;
        d["launch_no"] = L.launch_no; d["scratch_off"] = L.scratch_off; d["spin_limit"] = L.spin_limit; d["status_ptr"] = L.status_ptr;
        d["signal_off"] = L.signal_off; d["mc_base"] = L.mc_base;
        return d;
      }, py::arg("name"), py::arg("in_bytes"), py::arg("width") = 1, py::arg("lane") = 0)
      .def("startResident", &Engine::startResident, py::arg("width") = 4)
      .def("enqueueOp", &Engine::enqueueOp, py::arg("name"), py::arg("in_ptr"), py::arg("out_ptr"), py::arg("in_bytes"), py::arg("dtype"),
           py::arg("lane") = 0, py::arg("stream") = 0, py::call_guard<py::gil_scoped_release>())
      .def("waitOp", &Engine::waitOp, py::arg("ticket"), py::arg("timeout_ms") = 0, py::call_guard<py::gil_scoped_release>())
      .def("stopResident", &Engine::stopResident, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("rank", &Engine::rank)
      .def_property_readonly("world", &Engine::world);

  m.def("collective", &collective, py::arg("engine"), py::arg("kind"), py::arg("algo"), py::arg("dtype"),
        py::arg("redop"), py::arg("in_off"), py::arg("out_off"), py::arg("count"), py::arg("flag_lane") = 0,
        py::arg("scale") = 1.0f, py::arg("out_dtype") = "", py::arg("blocks") = 32, py::arg("threads") = 512,
        py::arg("stream") = 0, py::arg("local_in") = 0, py::arg("local_out") = 0, py::arg("spin_limit") = 0,
        py::arg("s_in_off") = 0, py::arg("s_out_off") = 0);
  m.def("reduce_scatter_adamw", [](Engine& e, const std::string& algo, uint64_t in_off, uint64_t count, int flag_lane, float scale,
                                   uint64_t p, uint64_t mm, uint64_t v, uint64_t p_bf16, float lr, float b1, float b2, float eps,
                                   float wd, int step, int blocks, int threads, uint64_t stream) {
    CollArgs a = makeCollArgs(e.worldTable(), 1, e.rank(), algo, "bf16", "sum", in_off, 0, count, e.nextEpoch(flag_lane), flag_lane,
                              scale, "", 0);
    a.status[0] = reinterpret_cast<uint32_t*>(e.statusPtr(8 + flag_lane));
    AdamArgs o{};
    o.p = reinterpret_cast<float*>(p); o.m = reinterpret_cast<float*>(mm); o.v = reinterpret_cast<float*>(v);
    o.p_bf16 = reinterpret_cast<void*>(p_bf16);
    o.lr = lr; o.b1 = b1; o.b2 = b2; o.eps = eps; o.wd = wd;
    o.inv_bc1 = 1.0f / (1.0f - std::pow(b1, static_cast<float>(step)));
    o.inv_sqrt_bc2 = 1.0f / std::sqrt(1.0f - std::pow(b2, static_cast<float>(step)));
    throwIfCuda(launchReduceScatterAdamW(a, o, blocks, threads, reinterpret_cast<cudaStream_t>(stream)), "reduce_scatter_adamw");
  });
  m.def("emu_collective", &emuCollective, py::arg("kind"), py::arg("heaps"), py::arg("signal_off"), py::arg("flag_off"), py::arg("dtype"),
        py::arg("redop"), py::arg("in_off"), py::arg("out_off"), py::arg("count"), py::arg("epoch"), py::arg("flag_lane"), py::arg("scale"),
        py::arg("out_dtype"), py::arg("blocks"), py::arg("threads"), py::arg("stream"), py::arg("status"), py::arg("local_in"),
        py::arg("local_out"), py::arg("spin_limit"), py::arg("s_in_off") = 0, py::arg("s_out_off") = 0, py::arg("ll_off") = 0);
  m.attr("LL_LANE_BYTES") = kLlLaneBytes;
  m.attr("LL_MAX_BYTES") = kLlMaxBytes;
  m.def("emu_program", &emuProgram);
  m.def("interp_set_fusion", [](int mask) { throwIfCuda(setInterpreterFusion(mask), "interp_set_fusion"); });
  m.def("wait_timeout_probe", [](uint64_t flag, uint64_t spin_limit, uint64_t status, uint64_t stream) {
    throwIfCuda(launchWaitTimeoutProbe(reinterpret_cast<uint64_t*>(flag), spin_limit, reinterpret_cast<uint32_t*>(status),
                                       reinterpret_cast<cudaStream_t>(stream)), "wait_timeout_probe");
  });
  m.def("memcpy_d2d", [](uint64_t dst, uint64_t src, uint64_t nbytes, uint64_t stream) {
    throwIfCuda(static_cast<int>(cudaMemcpyAsync(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), nbytes,
                                                 cudaMemcpyDeviceToDevice, reinterpret_cast<cudaStream_t>(stream))), "memcpy_d2d");
  });
  m.def("sm_count", &deviceSmCount);
  m.attr("MAX_RANKS") = kMaxRanks;
  m.attr("NO_TURN_SLOT") = kNoTurnSlot;
  m.attr("MAX_BLOCKS_PER_COLL") = kMaxBlocksPerColl;

  bindGemm(m);
  bindFused(m);

  auto utils = m.def_submodule("utils");
  py::class_<LaunchEnvironments, std::unique_ptr<LaunchEnvironments, py::nodelete>>(utils, "LaunchEnvironments")
      .def_static("listOpt", &LaunchEnvironments::listOpt)
      .def_static("getEnv", &LaunchEnvironments::getEnv)
      .def_static("registerOpt", &LaunchEnvironments::registerOpt, py::arg("name"), py::arg("help") = "")
      .def_static("helpOf", &LaunchEnvironments::helpOf)
      .def_static("setOverride", &LaunchEnvironments::setOverride);
  utils.def("encode_hex", [](py::bytes b) { std::string s = b; return encodeHex(s.data(), s.size()); });
  utils.def("decode_hex", [](const std::string& t) {
    bool ok = false;
    std::string s = decodeHexToString(t, &ok);
    if (!ok) throw std::runtime_error("decode_hex: malformed input");
    return py::bytes(s);
  });
  utils.def("fnv1a", [](const std::string& s) { return fnv1a(s); });
  // The CUDA device plugin by itself (no engine, no CUDA runtime call): what the CPU tests drive against a stand-in
  // driver library (PCCL_CUDA_DRIVER_LIB).  Multicast objects are kept here under small integer ids.
  auto cudaDev = [] {
    registerCudaDevice();
    return static_cast<CudaDevice*>(getDev("cuda").get());
  };
  static std::map<int, CudaDevice::McObject> mc_objects;
  static int mc_next = 1;
  utils.def("cuda_device_available", [cudaDev] { return cudaDev()->allocatorAvailable(); });
  utils.def("cuda_device_alloc", [cudaDev](uint64_t bytes) {
    std::string handle;
    void* p = cudaDev()->allocateIpcBuffer(bytes, &handle);
    return py::make_tuple(reinterpret_cast<uint64_t>(p), handle);
  });
  utils.def("cuda_device_map", [cudaDev](const std::string& handle) { return reinterpret_cast<uint64_t>(cudaDev()->mapBuffer(handle)); },
            py::call_guard<py::gil_scoped_release>());
  utils.def("cuda_device_free", [cudaDev](uint64_t ptr) { cudaDev()->deallocate(reinterpret_cast<void*>(ptr)); });
  utils.def("cuda_fd_probe", &CudaDevice::probeFdServer, py::call_guard<py::gil_scoped_release>());
  utils.def("cuda_fd_refused", [cudaDev] { return cudaDev()->refusedRequests(); });
  utils.def("cuda_mc_new", [] { mc_objects[mc_next] = CudaDevice::McObject{}; return mc_next++; });
  utils.def("cuda_mc_create", [cudaDev](int id, uint64_t bytes, int n) { return cudaDev()->multicastCreate(bytes, n, &mc_objects.at(id)); });
  utils.def("cuda_mc_join", [cudaDev](int id, const std::string& h) { cudaDev()->multicastJoin(h, &mc_objects.at(id)); });
  utils.def("cuda_mc_bind", [cudaDev](int id, uint64_t ptr) {
    return reinterpret_cast<uint64_t>(cudaDev()->multicastBind(reinterpret_cast<void*>(ptr), &mc_objects.at(id)));
  });
  utils.def("cuda_mc_release", [cudaDev](int id) { cudaDev()->multicastRelease(&mc_objects.at(id)); });
  utils.def("cuda_mc_state", [](int id) {
    const auto& m = mc_objects.at(id);
    return py::make_tuple(static_cast<uint64_t>(m.handle), reinterpret_cast<uint64_t>(m.va), m.bound);
  });
  utils.def("now_nanos", &nowNanos);
  utils.def("launch_timestamp", &launchTimestamp);
  utils.def("log", [](const std::string& level, const std::string& msg) {
    LogLevel l = Logger::parseLevel(level, LogLevel::Info);
    if (Logger::get().enabled(l)) Logger::get().log(l, "python", 0, "%s", msg.c_str());
  });
  utils.def("log_path", [] { return Logger::get().path(); });
  utils.def("log_count", [](const std::string& level) { return Logger::get().count(Logger::parseLevel(level, LogLevel::Info)); });
  utils.def("set_log_level", [](const std::string& level) { Logger::get().setLevel(Logger::parseLevel(level, LogLevel::Warn)); });
  utils.def("json_roundtrip", [](const std::string& s) { return Json::parse(s).dump(); });
  utils.def("register_type", [](int ns, const std::string& name) { return static_cast<int>(TypeRegistry::registerType(static_cast<TypeRegistry::Namespace>(ns), name)); });
  utils.def("type_names", [](int ns) { return TypeRegistry::names(static_cast<TypeRegistry::Namespace>(ns)); });
  utils.def("set_compatible", [](const std::string& ex, int ns, const std::string& t) { TypeRegistry::setCompatible(ex, static_cast<TypeRegistry::Namespace>(ns), t); });
  utils.def("executors_for", [](int ns, const std::string& t) { return TypeRegistry::executorsFor(static_cast<TypeRegistry::Namespace>(ns), t); });
  utils.def("bf16_roundtrip", [](float f) { return bf16ToFloat(floatToBf16(f)); });
  utils.def("f16_roundtrip", [](float f) { return f16ToFloat(floatToF16(f)); });
  utils.def("e4m3_roundtrip", [](float f) { return e4m3ToFloat(floatToE4m3(f)); });
  utils.def("cpu_reduce", [](uint64_t dst, uint64_t src, uint64_t bytes, const std::string& dtype, const std::string& op) {
    return reduceInto(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), bytes, parseDType(dtype), parseRedOp(op));
  });
}
