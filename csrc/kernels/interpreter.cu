// Persistent interpreter of lowered collective programs (one CTA = one instruction stream).
//
// This is the CUDA executor the reference never wrote (include/plugins/cuda_executor/executor.h is
// empty) for the operator graph it sketched (include/base/operator.h:19-38).  A CTA fetches its
// 64-byte instructions in order and runs them with all of its threads:
//   COPY / REDUCE        16-byte vector loops over local memory or a peer's mapped heap (NVLink)
//   NOTIFY / WAIT        counting signal words: red.release.sys on the consumer's heap, bounded
//                        ld.acquire.sys polling on our own
//   BARRIER              every rank increments one word on every rank
//   MM_LD_REDUCE / MM_ST in-switch reduction / multicast store through the NVLS mapping
// A wait that runs out of polls writes ST_TIMEOUT with the stream and pc into the status words and
// the CTA leaves; sibling CTAs notice the status word and leave too.  Nothing traps or spins forever.
// With a trace buffer attached, thread 0 stamps %globaltimer around every instruction (the end stamp
// after a CTA barrier, so it covers the slowest thread); the host turns the stamps into trace events.
#include <cooperative_groups.h>

#include "api.h"
#include "interp_ops.cuh"
#include "prims.cuh"

namespace pccl {

using namespace dev;
using namespace iops;

namespace {

// Which of the COPY foldings are on: bit 0 "copy + reduces as one pass", bit 1 "one source to several destinations"
// (setInterpreterFusion; the tests switch them off to compare).
__device__ int g_copy_fusion = 3;

// One CTA runs stream `stream` of rank R.  LaunchT is InterpLaunch (a kernel argument) or ResidentDesc (a queued launch
// read from memory): both carry the world table and the per-launch scalars under the same names.
template <class LaunchT>
__device__ __forceinline__ void interp_body(const LaunchT& L, const InterpRank& R, const int stream) {
  const bool turns = L.turn_slot != kNoTurnSlot;
  // a rank without instructions still takes its turn on the lane (one CTA that only runs the hand-shake)
  const int n_workers = turns && R.n_streams == 0 ? 1 : R.n_streams;
  if (stream >= n_workers) return;
  __shared__ uint32_t s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();

  const World& W = L.w;
  const int me = R.rank;
  uint64_t* const sig0 = reinterpret_cast<uint64_t*>(W.heap[me] + W.signal_off);
  uint64_t* my_sig = sig0 + L.slot_base;
  if (turns && L.launch_no >= 2 && R.buf_bytes[BUF_SCRATCH] != 0) {
    // nobody may still be using the scratch half of launch_no - 2 when this launch starts to write it (a launch that
    // moves nothing through scratch has nothing to wait for); one thread per peer, so the checks overlap
    if (threadIdx.x < static_cast<uint32_t>(W.world) && static_cast<int>(threadIdx.x) != me &&
        !wait_ge(sig0 + L.turn_slot + threadIdx.x, L.launch_no - 1, L.spin_limit, R.status))
      s_fail = ST_TIMEOUT;
    __syncthreads();
    if (s_fail) {
      if (threadIdx.x == 0) report(R.status, ST_TIMEOUT, static_cast<uint32_t>(stream), 0xffffu, OP_WAIT);
      return;
    }
  }
  if (R.n_streams == 0) {
    if (threadIdx.x == 0)
      for (int q = 0; q < W.world; ++q)
        if (q != me) red_add_release_sys(reinterpret_cast<uint64_t*>(W.heap[q] + W.signal_off) + L.turn_slot + me, 1);
    return;
  }
  const Instr* prog = R.instrs + R.stream_start[stream];
  uint64_t* const trace = R.trace ? R.trace + 2ull * R.stream_start[stream] : nullptr;

  // Address of (rank q, buffer b, offset) or nullptr when q's buffer b is not reachable.
  auto resolve = [&](int q, uint32_t b, uint64_t off) -> char* {
    if (b == BUF_SCRATCH) return W.heap[q] + R.scratch_off + off;
    if (q == me) return (b == BUF_INPUT ? R.input : R.output) + off;
    long long ho = b == BUF_INPUT ? R.input_heap_off : R.output_heap_off;
    return ho < 0 ? nullptr : W.heap[q] + ho + off;
  };
  auto resolve_mc = [&](uint32_t b, uint64_t off) -> char* {
    if (!W.mc_heap) return nullptr;
    if (b == BUF_SCRATCH) return W.mc_heap + R.scratch_off + off;
    long long ho = b == BUF_INPUT ? R.input_heap_off : R.output_heap_off;
    return ho < 0 ? nullptr : W.mc_heap + ho + off;
  };

  // The stream is read through shared memory, kChunk instructions at a time (the CTA loads a chunk with 16-byte
  // vectors; a thread then reads its instruction from shared memory instead of 64 bytes of global memory each).
  constexpr uint32_t kChunk = kInstrPad;
  __shared__ __align__(16) Instr s_prog[kChunk];
  uint32_t chunk_base = 0x80000000u;                   // "no chunk loaded": pc - chunk_base is then far above kChunk
  auto fetch = [&](uint32_t pc) -> const Instr& {       // uniform over the CTA
    if (pc - chunk_base >= kChunk) {
      __syncthreads();                                   // everybody is done with the previous chunk
      chunk_base = pc;
      // the host pads the instruction array with kInstrPad no-ops, so a whole chunk can always be read
      const Vec16* g = reinterpret_cast<const Vec16*>(prog + pc);
      Vec16* sm = reinterpret_cast<Vec16*>(s_prog);
      for (uint32_t i = threadIdx.x; i < kChunk * 4; i += blockDim.x) sm[i] = g[i];
      __syncthreads();
    }
    return s_prog[pc - chunk_base];
  };

  for (uint32_t pc = 0;; ++pc) {
    const Instr in = fetch(pc);
    if (in.op == OP_END) break;
    uint32_t fail = 0;
    if (trace && threadIdx.x == 0) trace[2ull * pc] = global_timer_ns();
    switch (in.op) {
      case OP_NOP: break;
      case OP_COPY:
      case OP_REDUCE:
      case OP_MM_LD_REDUCE:
      case OP_MM_ST: {
        if (in.bytes == 0) break;
        if (L.bounds_check && (in.src_off + in.bytes > R.buf_bytes[in.src_buf] || in.dst_off + in.bytes > R.buf_bytes[in.dst_buf])) {
          fail = ST_BOUNDS;
          break;
        }
        if (in.op == OP_COPY || in.op == OP_REDUCE) {
          char* s = resolve(in.src_rank, in.src_buf, in.src_off);
          char* d = resolve(in.dst_rank, in.dst_buf, in.dst_off);
          if (!s || !d) { fail = ST_UNSUPPORTED; break; }
          // Folding of what follows into this instruction (all inside the chunk that is in shared memory; "WAIT; REDUCE"
          // pairs count, their waits are taken first, which only delays this stream):
          //   REDUCE ... -> d, REDUCE ... -> d            one pass over d instead of one per source
          //   COPY a -> d, REDUCE ... -> d, ...           the same without reading d at all (the pull forms)
          //   COPY a -> d0, COPY a -> d1, ...             a is read once (a rank's slice going out to every peer)
          const bool fusable = !trace && (L.dtype == DT_F32 || L.dtype == DT_BF16 || L.dtype == DT_F16) &&
                               ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d) | in.bytes) & 15) == 0;
          char* srcs[kMaxFused];
          srcs[0] = s;
          int k = 1;
          uint32_t j = pc + 1;
          while (fusable && k < kMaxFused && !fail && (in.op == OP_REDUCE || (s != d && (g_copy_fusion & 1)))) {
            const uint32_t idx = j - chunk_base;
            if (idx + 1 >= kChunk) break;
            const Instr& a = s_prog[idx];
            const bool waits = a.op == OP_WAIT && s_prog[idx + 1].op == OP_REDUCE;
            if (!waits && a.op != OP_REDUCE) break;
            const Instr& r = waits ? s_prog[idx + 1] : a;
            if (r.dst_rank != in.dst_rank || r.dst_buf != in.dst_buf || r.dst_off != in.dst_off || r.bytes != in.bytes) break;
            if (L.bounds_check && r.src_off + r.bytes > R.buf_bytes[r.src_buf]) break;      // left to the plain path, which reports it
            char* sp = resolve(r.src_rank, r.src_buf, r.src_off);
            if (!sp || (reinterpret_cast<uintptr_t>(sp) & 15)) break;
            if (waits) {
              if (threadIdx.x == 0 && !wait_ge(my_sig + a.slot, L.epoch * a.count + a.value, L.spin_limit, R.status)) s_fail = ST_TIMEOUT;
              __syncthreads();
              if (s_fail) { fail = s_fail; pc = j; break; }
            }
            srcs[k++] = sp;
            j += waits ? 2 : 1;
          }
          if (fail) break;
          if (in.op == OP_COPY) {
            if (k > 1) {                                          // copy + reduces: d = srcs[0] (op) srcs[1] ...
              bool ok = false;
              switch (L.redop) {
                case RED_SUM: ok = reduce_n_from_dispatch<RED_SUM>(L.dtype, d, srcs, k, in.bytes); break;
                case RED_MAX: ok = reduce_n_from_dispatch<RED_MAX>(L.dtype, d, srcs, k, in.bytes); break;
                case RED_MIN: ok = reduce_n_from_dispatch<RED_MIN>(L.dtype, d, srcs, k, in.bytes); break;
                case RED_PROD: ok = reduce_n_from_dispatch<RED_PROD>(L.dtype, d, srcs, k, in.bytes); break;
              }
              if (!ok) fail = ST_UNSUPPORTED;
              // The destination was written without having been read first, and the next instruction usually reads it (the
              // reduced slice going out to the peers).  Measured on B200: without a fence between the two, that read now and
              // then returned what the destination held BEFORE the stores, 64 bytes at a time, on the first launch of a
              // process (found by the emulated-rank test of the staged all-reduce; a __threadfence() alone, or a
              // __syncthreads() alone, removed it in every run).  The n-ary REDUCE and the plain REDUCE load the destination
              // before they store to it and have never shown this.  One fence and one barrier per folded instruction.
              __threadfence();
              __syncthreads();
              pc = j - 1;
              break;
            }
            // the same source to several destinations
            char* dsts[kMaxFused];
            dsts[0] = d;
            int n = 1;
            while (fusable && s != d && n < kMaxFused && (g_copy_fusion & 2)) {
              const uint32_t idx = j - chunk_base;
              if (idx >= kChunk) break;
              const Instr& c = s_prog[idx];
              if (c.op != OP_COPY || c.src_rank != in.src_rank || c.src_buf != in.src_buf || c.src_off != in.src_off || c.bytes != in.bytes) break;
              if (L.bounds_check && c.dst_off + c.bytes > R.buf_bytes[c.dst_buf]) break;
              char* dp = resolve(c.dst_rank, c.dst_buf, c.dst_off);
              if (!dp || dp == s || (reinterpret_cast<uintptr_t>(dp) & 15)) break;
              dsts[n++] = dp;
              ++j;
            }
            if (n > 1) {
              copy_fan_range(dsts, n, s, in.bytes);
              __threadfence();                                    // see the note at the copy + reduce folding above
              __syncthreads();
              pc = j - 1;
            } else if (s != d) {
              copy_range(d, s, in.bytes);
              __threadfence_block();                              // a later instruction of this stream may read d (same note)
            }
          } else {
            if (fail) break;
            bool ok = false;
            if (k > 1) {
              switch (L.redop) {
                case RED_SUM: ok = reduce_n_dispatch<RED_SUM>(L.dtype, d, srcs, k, in.bytes); break;
                case RED_MAX: ok = reduce_n_dispatch<RED_MAX>(L.dtype, d, srcs, k, in.bytes); break;
                case RED_MIN: ok = reduce_n_dispatch<RED_MIN>(L.dtype, d, srcs, k, in.bytes); break;
                case RED_PROD: ok = reduce_n_dispatch<RED_PROD>(L.dtype, d, srcs, k, in.bytes); break;
              }
              pc = j - 1;                                        // the folded instructions are done
            } else {
              switch (L.redop) {
                case RED_SUM: ok = reduce_dispatch<RED_SUM>(L.dtype, d, s, in.bytes); break;
                case RED_MAX: ok = reduce_dispatch<RED_MAX>(L.dtype, d, s, in.bytes); break;
                case RED_MIN: ok = reduce_dispatch<RED_MIN>(L.dtype, d, s, in.bytes); break;
                case RED_PROD: ok = reduce_dispatch<RED_PROD>(L.dtype, d, s, in.bytes); break;
              }
            }
            if (!ok) fail = ST_UNSUPPORTED;
          }
        } else if (in.op == OP_MM_LD_REDUCE) {
          char* mc = resolve_mc(in.src_buf, in.src_off);
          char* d = resolve(me, in.dst_buf, in.dst_off);
          // "reduce my slice in the switch, then multicast it from where it landed": when the next instruction stores
          // exactly this result to the same place on every rank, the two become one loop (the multicast store also
          // writes this rank's own copy)
          const uint32_t nidx = pc + 1 - chunk_base;
          if (!trace && mc && d && nidx < kChunk && s_prog[nidx].op == OP_MM_ST && s_prog[nidx].src_buf == in.dst_buf &&
              s_prog[nidx].src_off == in.dst_off && s_prog[nidx].dst_buf == in.dst_buf && s_prog[nidx].dst_off == in.dst_off &&
              s_prog[nidx].bytes == in.bytes) {
            char* mcd = resolve_mc(in.dst_buf, in.dst_off);
            if (mcd && !((reinterpret_cast<uintptr_t>(mc) | reinterpret_cast<uintptr_t>(mcd) | in.bytes) & 15) &&
                mm_reduce_bcast_dispatch(L.dtype, L.redop, mcd, mc, in.bytes)) {
              ++pc;
              break;
            }
          }
          if (!mc || !d || ((reinterpret_cast<uintptr_t>(mc) | reinterpret_cast<uintptr_t>(d) | in.bytes) & 15) ||
              !mm_ld_reduce_dispatch(L.dtype, L.redop, d, mc, in.bytes))
            fail = ST_UNSUPPORTED;
        } else {
          char* mc = resolve_mc(in.dst_buf, in.dst_off);
          char* s = resolve(me, in.src_buf, in.src_off);
          if (!mc || !s || ((reinterpret_cast<uintptr_t>(mc) | reinterpret_cast<uintptr_t>(s) | in.bytes) & 15)) fail = ST_UNSUPPORTED;
          else mm_st_range(mc, s, in.bytes);
        }
        break;
      }
      case OP_NOTIFY: {
        __syncthreads();   // every thread's stores of the preceding instruction are issued
        if (threadIdx.x == 0) {
          __threadfence_system();
          uint64_t* sig = reinterpret_cast<uint64_t*>(W.heap[in.dst_rank] + W.signal_off) + L.slot_base + in.slot;
          red_add_release_sys(sig, 1);
        }
        break;
      }
      case OP_WAIT: {
        if (threadIdx.x == 0) {
          uint64_t target = L.epoch * in.count + in.value;
          if (!wait_ge(my_sig + in.slot, target, L.spin_limit, R.status)) s_fail = ST_TIMEOUT;
        }
        __syncthreads();
        fail = s_fail;
        break;
      }
      case OP_BARRIER: {
        __syncthreads();
        if (threadIdx.x < static_cast<uint32_t>(W.world)) {
          __threadfence_system();
          uint64_t* sig = reinterpret_cast<uint64_t*>(W.heap[threadIdx.x] + W.signal_off) + L.slot_base + in.slot;
          red_add_release_sys(sig, 1);
        }
        if (threadIdx.x == 0) {
          uint64_t target = static_cast<uint64_t>(W.world) * (L.epoch * in.count + in.value);
          if (!wait_ge(my_sig + in.slot, target, L.spin_limit, R.status)) s_fail = ST_TIMEOUT;
        }
        __syncthreads();
        fail = s_fail;
        break;
      }
      default: fail = ST_BAD_OP;
    }
    if (trace) {                // uniform over the CTA: the pointer is a launch argument
      __syncthreads();
      if (threadIdx.x == 0) trace[2ull * pc + 1] = global_timer_ns();
    }
    if (fail) {
      if (threadIdx.x == 0) report(R.status, fail, static_cast<uint32_t>(stream), pc, in.op);
      return;
    }
  }
  if (turns) {
    // the last stream of this rank to end tells every peer that the rank has left this launch's scratch half
    // (one thread per peer: the releases go out together instead of one behind the other)
    __shared__ uint32_t s_last;
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      unsigned int* fin = reinterpret_cast<unsigned int*>(sig0 + L.finish_slot);
      s_last = atomicInc(fin, static_cast<unsigned int>(n_workers - 1)) == static_cast<unsigned int>(n_workers - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (s_last && threadIdx.x < static_cast<uint32_t>(W.world) && static_cast<int>(threadIdx.x) != me)
      red_add_release_sys(reinterpret_cast<uint64_t*>(W.heap[threadIdx.x] + W.signal_off) + L.turn_slot + me, 1);
  }
}

__global__ void __launch_bounds__(512) interp_kernel(const __grid_constant__ InterpLaunch L) {
  interp_body(L, L.r[blockIdx.y], static_cast<int>(blockIdx.x));
}

// ---------------------------------------------------------------------------------------------
// Resident form: the kernel stays on the GPU and takes launches from a queue that the host fills, so that a collective
// costs a 300-byte write to pinned memory instead of a kernel launch.  This is the device half of the reference's
// mirrored ring buffer between executors (include/base/operator.h:7-17: producer_buffer_, consumer_buffer_, head_,
// tail_) and of its completed_operator / total_operator counters (operator.h:31-38).  CTA 0 polls the queue's tail
// (host memory, read over PCIe), copies the next descriptor into device memory, the grid synchronises, every CTA runs
// its stream of the program, the grid synchronises again and CTA 0 publishes the completion count.  The kernel leaves by
// itself when the host says stop or when nothing has arrived for `idle_ns` (the host then launches it again on the next
// submission), so it can never spin without bound.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t ld_volatile_u64(const volatile uint64_t* p) {
  uint64_t v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(512) resident_kernel(ResidentQueue* q, ResidentCtl* ctl, uint64_t head) {
  cooperative_groups::grid_group grid = cooperative_groups::this_grid();
  for (;;) {
    if (blockIdx.x == 0 && threadIdx.x < 32) {
      uint32_t run = 1;
      if (threadIdx.x == 0) {
        const uint64_t t0 = global_timer_ns();
        while (ld_volatile_u64(&q->tail) <= head) {
          if (ld_volatile_u32(const_cast<const uint32_t*>(&q->stop)) != 0 || global_timer_ns() - t0 > q->idle_ns) { run = 0; break; }
          __nanosleep(100);
        }
      }
      run = __shfl_sync(0xffffffffu, run, 0);
      if (run) {
        // the descriptor crosses PCIe once, 16 bytes per lane, all loads in flight together
        const Vec16* src = reinterpret_cast<const Vec16*>(&q->slots[head % kResidentSlots]);
        Vec16* dst = reinterpret_cast<Vec16*>(&ctl->desc);
        for (uint32_t i = threadIdx.x; i < sizeof(ResidentDesc) / 16; i += 32) dst[i] = ld16(reinterpret_cast<const char*>(src + i));
      }
      __syncwarp();
      if (threadIdx.x == 0) {
        ctl->run = run;
        __threadfence();
      }
    }
    grid.sync();
    if (*const_cast<volatile uint32_t*>(&ctl->run) == 0) break;
    interp_body(ctl->desc, ctl->desc.r, static_cast<int>(blockIdx.x));
    grid.sync();
    ++head;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      __threadfence_system();
      asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(&q->completed), "l"(head) : "memory");
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(&q->running), "r"(0u) : "memory");
  }
}

__global__ void __launch_bounds__(512) device_reduce_kernel(char* dst, const char* src, uint64_t bytes, uint32_t dtype, uint32_t redop,
                                                            uint32_t* bad) {
  // each CTA takes a 16-byte aligned slice
  const uint64_t per = ((bytes + gridDim.x - 1) / gridDim.x + 15) & ~15ull;
  const uint64_t lo = per * blockIdx.x;
  if (lo >= bytes) return;
  const uint64_t n = bytes - lo < per ? bytes - lo : per;
  bool ok = false;
  switch (redop) {
    case RED_SUM: ok = reduce_dispatch<RED_SUM>(dtype, dst + lo, src + lo, n); break;
    case RED_MAX: ok = reduce_dispatch<RED_MAX>(dtype, dst + lo, src + lo, n); break;
    case RED_MIN: ok = reduce_dispatch<RED_MIN>(dtype, dst + lo, src + lo, n); break;
    case RED_PROD: ok = reduce_dispatch<RED_PROD>(dtype, dst + lo, src + lo, n); break;
  }
  if (!ok && threadIdx.x == 0) *bad = 1;
}

__global__ void wait_timeout_probe_kernel(uint64_t* flag, uint64_t spin_limit, uint32_t* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (!wait_ge(flag, 1, spin_limit, nullptr)) report(status, ST_TIMEOUT, 0, 0, OP_WAIT);
  }
}

}  // namespace

int setInterpreterFusion(int mask) {
  return static_cast<int>(cudaMemcpyToSymbol(g_copy_fusion, &mask, sizeof(int)));
}

int launchInterpreter(const InterpLaunch& L, int threads, cudaStream_t stream) {
  int max_streams = 0;
  for (int v = 0; v < L.nvirt; ++v) max_streams = L.r[v].n_streams > max_streams ? L.r[v].n_streams : max_streams;
  if (max_streams == 0 && L.turn_slot != kNoTurnSlot) max_streams = 1;      // the lane's hand-shake still runs
  if (max_streams == 0) return 0;
  dim3 grid(max_streams, L.nvirt), block(threads);
  void* args[] = {const_cast<InterpLaunch*>(&L)};
  // Streams wait on one another, so every CTA must be resident: a cooperative launch refuses
  // (instead of hanging) when the grid does not fit.
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(interp_kernel), grid, block, args, 0, stream));
}

int launchResident(ResidentQueue* queue_device_view, ResidentCtl* ctl, uint64_t head, int ctas, int threads, cudaStream_t stream) {
  void* args[] = {&queue_device_view, &ctl, &head};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(resident_kernel), dim3(ctas), dim3(threads), args, 0, stream));
}

int launchDeviceReduce(void* dst, const void* src, uint64_t bytes, uint32_t dtype, uint32_t redop, cudaStream_t stream) {
  if (bytes == 0) return 0;
  static uint32_t* bad = nullptr;                   // sticky "unsupported dtype / op" word, checked by the caller's status read
  if (!bad) {
    cudaError_t e = cudaMalloc(&bad, sizeof(uint32_t));
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaMemset(bad, 0, sizeof(uint32_t));
  }
  const uint32_t es = dtypeSize(dtype);
  if (bytes % es) return static_cast<int>(cudaErrorInvalidValue);
  int blocks = static_cast<int>((bytes + (256u << 10) - 1) / (256u << 10));
  if (blocks > 64) blocks = 64;
  device_reduce_kernel<<<blocks, 512, 0, stream>>>(static_cast<char*>(dst), static_cast<const char*>(src), bytes, dtype, redop, bad);
  return static_cast<int>(cudaGetLastError());
}

int launchWaitTimeoutProbe(uint64_t* flag, uint64_t spin_limit, uint32_t* status, cudaStream_t stream) {
  wait_timeout_probe_kernel<<<1, 32, 0, stream>>>(flag, spin_limit, status);
  return static_cast<int>(cudaGetLastError());
}

int deviceSmCount() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

const char* cudaErrorName(int err) { return cudaGetErrorString(static_cast<cudaError_t>(err)); }

}  // namespace pccl
