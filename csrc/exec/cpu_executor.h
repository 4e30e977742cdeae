// CPU executor: runs a rank's instruction streams on host threads.
//
// The reference's cpu executor header is empty (include/plugins/cpu_executor/executor.h); its
// intended loop is "pop an op, run the primitive, release dependants" over the layouts of
// include/base/operator.h:7-38.  Here each stream (channel x width replica) gets one thread that
// walks its instructions in order; COPY / REDUCE touch local memory, a same-host peer's mapped
// workspace, or go through the TCP transport; NOTIFY / WAIT / BARRIER use counting signal words.
// Every wait is bounded: on time-out the worker records ST_TIMEOUT, raises the abort flag so its
// sibling workers stop too, and the call returns the status to the caller.
#pragma once
#include <atomic>
#include <cstdint>
#include <vector>

#include "../transport/tcp_transport.h"
#include "program.h"

namespace pccl {

// How the executor touches the buffers of a launch.  Null means plain host memory (memmove, host reduce).  A CUDA
// engine whose peers are partly on other hosts runs its programs with this executor too -- the instruction streams
// walk on host threads, the bytes stay on the device -- and supplies copies and reductions that act on device memory.
struct MemOps {
  virtual ~MemOps() = default;
  virtual bool copy(void* dst, const void* src, uint64_t bytes) = 0;
  virtual bool reduce(void* dst, const void* src, uint64_t bytes, uint32_t dtype, uint32_t redop) = 0;
  // host-readable copy of `bytes` at `src`, valid until the calling thread's next call
  virtual const void* toHost(const void* src, uint64_t bytes) = 0;
};

struct CpuExecContext {
  int rank = 0, world = 1;
  char* local[BUF_COUNT] = {nullptr, nullptr, nullptr};   // input, output, scratch (this launch's lane)
  uint64_t local_bytes[BUF_COUNT] = {0, 0, 0};
  std::vector<char*> peer_scratch;                         // per rank; nullptr = reach it over TCP
  std::vector<std::atomic<uint64_t>*> peer_signals;        // per rank; nullptr = over TCP
  RemoteCommunicatorBase* tcp = nullptr;              // the data plane for peers that cannot be mapped (TCP or verbs)
  uint32_t tcp_scratch_key = 0;
  uint64_t tcp_scratch_off = 0;      // lane offset inside the peer's registered workspace
  uint32_t slot_base = 0;            // first signal slot of this op
  uint64_t epoch = 0;                // launches of this op so far
  uint32_t dtype = DT_F32, redop = RED_SUM;
  int timeout_ms = 30000;
  bool bounds_check = true;
  bool trace = false;                // record one TraceEvent per executed instruction
  // Workspace turn-taking (see InterpLaunch in kernels/api.h): before the launch every peer must have finished
  // launch_no - 2 on this lane; after it this rank adds one to its word on every peer.  turn_slot < 0: off.
  int64_t turn_slot = -1;
  uint64_t launch_no = 0;
  // Testing aid (PCCL_EXEC_DELAY_US with PCCL_EXEC_DELAY_RANK): sleep this long before every instruction, which
  // makes one rank lag behind the others deterministically.
  int delay_us = 0;
  MemOps* mem = nullptr;
};

struct TraceEvent {
  uint32_t stream, pc, op;
  uint64_t t0_ns, t1_ns, bytes;      // monotonic clock
};

struct CpuExecResult {
  uint32_t status = ST_OK;
  int failed_stream = -1;
  int failed_pc = -1;
  uint64_t nanos = 0;
  std::vector<TraceEvent> trace;
};

CpuExecResult runOnCpu(const Materialized& m, const CpuExecContext& ctx);

}  // namespace pccl
