// Engine: the runtime object behind `pccl.engine`.
//
// Same public surface as the reference engine (include/engine.h:13-33, csrc/python_api.cc:13-20):
// Engine(rank, world) with initEngine, regOp, exeOp, exportEndpoint, joinCluster, exitCluster.
// In the reference initEngine allocates a 256 MiB workspace plus 256 int signals per device and
// fills a flat endpoint map (csrc/engine.cc:42-100); regOp is empty and the other four methods have
// no definition.  Here:
//   * one symmetric heap per rank = [scratch workspace | uint64 signal words | barrier flags |
//     status | user region]; the heap is POSIX shm for CPU ranks and a VMM allocation (peer-mapped
//     over NVLink, optionally bound to an NVLS multicast object) for CUDA ranks;
//   * regOp parses a schedule document and reserves a private range of signal words for it;
//   * exeOp binds the schedule to the tensors, a worker budget (`width` -> CTAs or threads: the
//     reference's "runtime resource control") and a workspace lane (ops on different lanes may run
//     concurrently on different streams: "comm-comm overlap"), then runs it on the CPU executor or
//     launches the persistent interpreter kernel;
//   * joinCluster/exitCluster drive the control-plane daemon; importEndpoints is the same peer
//     set-up for launchers that already have a rendezvous (torchrun).
#pragma once
#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "cluster/manager.h"
#include "exec/cpu_executor.h"
#include "exec/program.h"
#include "kernels/api.h"
#include "mem/cuda_device.h"
#include "transport/tcp_transport.h"
#include "transport/verbs_transport.h"

namespace pccl {

struct HeapLayout {
  uint64_t workspace_bytes = 0;
  uint64_t signal_off = 0, num_signals = 0;
  uint64_t flag_off = 0, flag_bytes = 0;
  uint64_t status_off = 0, status_bytes = 0;
  uint64_t ll_off = 0;                       // low-latency all-reduce receive areas, kLlLanes x kLlLaneBytes
  uint64_t user_off = 0;
  uint64_t total = 0;
  int lanes = 2;
  // The last signal words are not handed to programs: kMaxLanes x kMaxRanks "launches finished" counters and
  // kMaxLanes "streams ended" counters of the workspace turn-taking (kernels/api.h, InterpLaunch).
  uint32_t turn_base = 0, finish_base = 0;
};
constexpr int kMaxLanes = 8;

class Engine {
 public:
  Engine(int rank, int world);
  ~Engine();

  void initEngine(const std::string& device = "auto", uint64_t heap_bytes = 0);
  void regOp(const std::string& name, const std::string& path_or_json);
  // Returns an ExecStatus for CPU ranks (synchronous); 0 for CUDA ranks (asynchronous on `stream`;
  // call checkStatus() to synchronise and read the device status words).
  // Hands the signal words of (op, width) out now.  exeOp does it at the first launch by itself; threads that launch
  // DIFFERENT ops concurrently call this first, in one order on every rank, so that all ranks number the words alike.
  void prepareOp(const std::string& name, int width);
  int exeOp(const std::string& name, uint64_t in_ptr, uint64_t out_ptr, uint64_t in_bytes,
            const std::string& dtype, int width, int lane, uint64_t stream);
  // ---- resident executor (CUDA engines): a kernel that stays on the GPU and takes launches from a host-filled queue ----
  // Counterpart of the reference's ring buffer between executor kinds and of its completed / total operator counters
  // (include/base/operator.h:7-17, 31-38).  startResident launches the kernel with `width` CTAs (cooperatively: it is
  // refused when they cannot all be resident); enqueueOp writes one descriptor -- no kernel launch -- and returns a
  // ticket; waitOp blocks until the kernel has finished that ticket.  The program runs at the resident width.  The
  // tensors must be complete when enqueueOp is called (it synchronises `stream` first when one is given) and must stay
  // alive until the ticket is done.  The kernel leaves by itself after PCCL_RESIDENT_IDLE_MS without work (default 20)
  // and is started again by the next enqueueOp, so device-wide synchronisation never waits longer than that.
  // ---- hooks for kernels compiled at run time for one program (pccl_b200/jit.py) ----------------------------------------
  // The instruction streams of this rank for (program, message size, width), as the executors would run them.
  std::vector<std::vector<Instr>> materializedStreams(const std::string& name, uint64_t in_bytes, int width, uint64_t* buf_bytes);
  // Everything a launch of (program, width) on `lane` needs besides the tensors, with the same book-keeping as exeOp:
  // the variant's signal range and launch number, the lane's scratch half and turn-taking words.
  struct LaunchPlan {
    uint32_t slot_base, turn_slot, finish_slot;
    uint64_t epoch, launch_no, scratch_off, spin_limit, status_ptr, signal_off, mc_base;
  };
  LaunchPlan planLaunch(const std::string& name, uint64_t in_bytes, int width, int lane);
  std::map<std::string, std::string> opInfo(const std::string& name);     // collective, redop, world, channels, in_place, ...
  void startResident(int width);
  uint64_t enqueueOp(const std::string& name, uint64_t in_ptr, uint64_t out_ptr, uint64_t in_bytes, const std::string& dtype, int lane,
                     uint64_t stream);
  bool waitOp(uint64_t ticket, int timeout_ms);
  void stopResident();
  std::string exportEndpoint();
  void importEndpoints(const std::vector<std::string>& docs);
  void joinCluster(const std::string& master_endpoint, int timeout_ms = 60000);
  void exitCluster();
  std::string stats();
  // Chrome-trace ("traceEvents") JSON of the instructions recorded while PCCL_TRACE=1: the CPU executor's
  // with host timestamps, the interpreter kernel's with the device's %globaltimer (a traced GPU launch is
  // followed by a synchronize of its stream, so tracing is for inspection, not for timed runs or graph capture);
  // clears the record.
  std::string trace();
  // Adds the spans of one interpreter launch from its raw stamp buffer (two %globaltimer words per instruction
  // of this rank's streams at `width`, streams back to back): for buffers captured outside exeOp.
  void ingestDeviceTrace(const std::string& name, uint64_t in_bytes, int width, const std::vector<uint64_t>& stamps);

  // symmetric heap
  const std::string& deviceKind() const { return device_; }
  uint64_t heapBase(int rank) const;
  uint64_t heapBytes() const { return layout_.total; }
  uint64_t allocSymmetric(uint64_t bytes, uint64_t align);   // returns heap offset (same on all ranks
                                                             // when called in the same order)
  void resetSymmetric(uint64_t mark);
  uint64_t symmetricMark() const { return user_top_; }
  const HeapLayout& layout() const { return layout_; }
  World worldTable() const;

  // NVLS multicast bring-up (three steps with a barrier of the caller's choice between them)
  bool multicastSupported();
  std::string mcCreate();
  void mcJoin(const std::string& handle);
  void mcBind();
  uint64_t mcBase() const { return reinterpret_cast<uint64_t>(mc_base_); }

  // status / elastic
  std::vector<uint32_t> checkStatus(int lane);
  uint64_t statusPtr(int lane) const;
  std::vector<int> aliveRanks();
  std::map<int, int> resizeWorld();      // master: renumber the survivors and announce it
  std::map<int, int> lastResize();
  bool waitForDeparture(int rank, int timeout_ms);
  void rebind(int new_rank, int new_world);   // adopt a ResizeWorld result (drops peer mappings)
  void injectFault(const std::string& kind);  // host-side fault injection for tests
  bool mixedHosts() const { return mixed_hosts_; }   // CUDA ranks on more than one host: programs only, host-driven
  int rank() const { return rank_; }
  int world() const { return world_; }
  uint64_t nextEpoch(int flag_lane);          // per-lane launch counter for hand-written collectives

 private:
  struct Op {
    Program program;
    // A program is materialised per width (replicas of every channel); each width has its own signal words and
    // its own launch count, because signals only ever count up: "launch e expects e * count + k" holds only
    // among launches that use the same words the same way.
    struct Variant { uint32_t slot_base = 0; uint64_t epoch = 0; };
    std::map<int, Variant> variants;
    uint64_t launches = 0, bytes = 0, nanos = 0, timeouts = 0;
    struct DeviceCopy { Instr* instrs = nullptr; uint32_t* starts = nullptr; int n_streams = 0; Materialized m; };
    std::map<std::pair<uint64_t, int>, DeviceCopy> device_cache;
    std::map<std::pair<uint64_t, int>, Materialized> host_cache;
  };
  void buildLayout(uint64_t heap_bytes);
  void setupPeers(const std::map<int, NodeMeta>& nodes);
  void dropPeers();
  Op::Variant& variantFor(Op& op, int width);     // caller holds mu_
  int exeOnCpu(Op& op, uint64_t in_ptr, uint64_t out_ptr, uint64_t in_bytes, uint32_t dtype, int width, int lane);
  int exeOnCuda(Op& op, uint64_t in_ptr, uint64_t out_ptr, uint64_t in_bytes, uint32_t dtype, int width, int lane, uint64_t stream);
  // Turns the interpreter kernel's stamps (two words per instruction, streams back to back) into spans; caller holds mu_.
  void addDeviceSpans(const std::string& name, const Materialized& m, const std::vector<uint64_t>& stamps);

  int rank_, world_;
  bool initialized_ = false;
  std::string device_;
  std::string host_id_;
  HeapLayout layout_;
  char* heap_ = nullptr;
  std::string heap_handle_;
  std::vector<char*> peer_heaps_;
  void* mc_base_ = nullptr;
  CudaDevice::McObject mc_;                 // this engine's NVLS multicast object (none until mcCreate / mcJoin)
  uint64_t user_top_ = 0;
  std::map<std::string, std::string> configs_;
  std::unique_ptr<ClusterManager> cluster_;
  std::unique_ptr<TcpTransport> tcp_;
  uint32_t tcp_key_ = 0;
  // InfiniBand / RoCE data plane (PCCL_TRANSPORT=verbs on CPU ranks): used instead of tcp_ for peers that are reached
  // over the network; remote_ points at whichever of the two carries remote PUT / SIGNAL traffic.
  std::unique_ptr<VerbsTransport> verbs_;
  uint32_t verbs_key_ = 0;
  RemoteCommunicatorBase* remote_ = nullptr;
  uint32_t remote_key_ = 0;
  // CUDA ranks that do not all share one host (the reference pairs every communicator device with every memory device,
  // csrc/engine.cc:52-95): peers on this host keep their NVLink mapping for data, peers elsewhere are reached over the
  // host/TCP transport through a pinned host shadow of the workspace, and every signal travels over TCP into host
  // signal words.  Programs then run on the host-driven executor (instruction streams on host threads, bytes on the GPU).
  // resident executor state
  ResidentQueue* rq_host_ = nullptr;      // pinned host memory
  ResidentQueue* rq_dev_ = nullptr;       // the same memory as the device sees it
  ResidentCtl* rctl_ = nullptr;
  void* resident_stream_ = nullptr;
  int resident_width_ = 0;
  uint64_t resident_launches_ = 0, resident_ops_ = 0;
  void launchResidentKernel();            // caller holds mu_
  bool mixed_hosts_ = false;
  int cuda_ordinal_ = 0;
  char* shadow_ = nullptr;
  std::atomic<uint64_t>* host_signals_ = nullptr;
  void* shadow_stream_ = nullptr;
  std::unique_ptr<MemOps> device_mem_ops_;
  void ensureMixedHostResources();
  int exeOnCudaHost(Op& op, uint64_t in_ptr, uint64_t out_ptr, uint64_t in_bytes, uint32_t dtype, int width, int lane, uint64_t stream);
  std::map<std::string, Op> ops_;
  uint32_t next_slot_ = 0;
  std::mutex mu_;
  std::vector<uint64_t> lane_epochs_;
  std::vector<uint64_t> lane_launches_;     // programs launched per workspace lane: picks the scratch half
  int timeout_ms_ = 30000;
  uint64_t spin_limit_ = kDefaultSpinLimit;
  bool bounds_check_ = true;
  bool trace_ = false;
  struct Span { std::string op; uint32_t stream, pc, opcode; uint64_t t0, t1, bytes; };
  std::vector<Span> spans_;
  // Device trace buffers, one per workspace lane (two %globaltimer words per instruction), grown on demand.
  struct DeviceTrace { uint64_t* words = nullptr; size_t cap = 0; };
  std::vector<DeviceTrace> dtrace_;
  int max_width_ = 32;
  int exec_delay_us_ = 0, exec_delay_rank_ = -1;   // testing aid: PCCL_EXEC_DELAY_US on rank PCCL_EXEC_DELAY_RANK
};

}  // namespace pccl
