#include "cpu_executor.h"

#include <chrono>
#include <cstring>
#include <thread>

#include "../common/clock.h"
#include "../common/log.h"
#include "reduce_cpu.h"

namespace pccl {

namespace {

struct Shared {
  std::atomic<uint32_t> status{ST_OK};
  std::atomic<int> failed_stream{-1};
  std::atomic<int> failed_pc{-1};
  void fail(uint32_t st, int stream, int pc) {
    uint32_t expect = ST_OK;
    if (status.compare_exchange_strong(expect, st)) {
      failed_stream.store(stream);
      failed_pc.store(pc);
    }
  }
};

bool waitFor(std::atomic<uint64_t>* word, uint64_t target, const CpuExecContext& ctx, Shared& sh) {
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(ctx.timeout_ms);
  int spins = 0;
  while (word->load(std::memory_order_acquire) < target) {
    if (sh.status.load(std::memory_order_relaxed) != ST_OK) return false;
    if (++spins < 64) continue;
    spins = 0;
    std::this_thread::yield();
    if (std::chrono::steady_clock::now() >= deadline) return false;
  }
  return true;
}

void runStream(const std::vector<Instr>& prog, int stream, const CpuExecContext& ctx, Shared& sh, std::vector<TraceEvent>* trace) {
  std::atomic<uint64_t>* my_signals = ctx.peer_signals[ctx.rank];
  auto resolve = [&](int rank, uint32_t buf, uint64_t off, uint64_t bytes, bool* remote_tcp) -> char* {
    *remote_tcp = false;
    if (rank == ctx.rank) {
      if (ctx.bounds_check && (off > ctx.local_bytes[buf] || bytes > ctx.local_bytes[buf] - off)) return nullptr;
      return ctx.local[buf] + off;
    }
    if (buf != BUF_SCRATCH) return nullptr;   // peers only see the symmetric workspace
    if (ctx.bounds_check && (off > ctx.local_bytes[BUF_SCRATCH] || bytes > ctx.local_bytes[BUF_SCRATCH] - off)) return nullptr;
    if (ctx.peer_scratch[rank]) return ctx.peer_scratch[rank] + off;
    *remote_tcp = true;
    return reinterpret_cast<char*>(1);   // non-null marker; the caller must use the transport
  };
  for (size_t pc = 0; pc < prog.size(); ++pc) {
    if (sh.status.load(std::memory_order_relaxed) != ST_OK) return;
    const Instr& in = prog[pc];
    if (ctx.delay_us > 0 && in.op != OP_END) std::this_thread::sleep_for(std::chrono::microseconds(ctx.delay_us));
    struct Stamp {
      std::vector<TraceEvent>* out; uint32_t stream, pc, op; uint64_t bytes, t0;
      ~Stamp() { if (out) out->push_back(TraceEvent{stream, pc, op, t0, monotonicNanos(), bytes}); }
    } stamp{trace, static_cast<uint32_t>(stream), static_cast<uint32_t>(pc), in.op, in.bytes, trace ? monotonicNanos() : 0};
    switch (in.op) {
      case OP_NOP: break;
      case OP_END: return;
      case OP_COPY:
      case OP_REDUCE: {
        if (in.bytes == 0) break;
        bool src_tcp, dst_tcp;
        char* s = resolve(in.src_rank, in.src_buf, in.src_off, in.bytes, &src_tcp);
        char* d = resolve(in.dst_rank, in.dst_buf, in.dst_off, in.bytes, &dst_tcp);
        if (!s || !d) { sh.fail(ST_BOUNDS, stream, static_cast<int>(pc)); return; }
        if (src_tcp || (dst_tcp && in.op == OP_REDUCE)) { sh.fail(ST_UNSUPPORTED, stream, static_cast<int>(pc)); return; }
        if (dst_tcp) {
          // the transport reads host memory: device bytes are staged in pieces
          bool ok = ctx.tcp != nullptr;
          const uint64_t piece = ctx.mem ? (4ull << 20) : in.bytes;
          for (uint64_t o = 0; ok && o < in.bytes; o += piece) {
            const uint64_t n = in.bytes - o < piece ? in.bytes - o : piece;
            const void* h = ctx.mem ? ctx.mem->toHost(s + o, n) : s + o;
            ok = h && ctx.tcp->put(in.dst_rank, ctx.tcp_scratch_key, ctx.tcp_scratch_off + in.dst_off + o, h, n);
          }
          if (!ok) {
            sh.fail(ST_PEER_GONE, stream, static_cast<int>(pc));
            return;
          }
        } else if (in.op == OP_COPY) {
          if (s != d) {
            if (ctx.mem) {
              if (!ctx.mem->copy(d, s, in.bytes)) { sh.fail(ST_UNSUPPORTED, stream, static_cast<int>(pc)); return; }
            } else {
              std::memmove(d, s, in.bytes);
            }
          }
        } else if (ctx.mem ? !ctx.mem->reduce(d, s, in.bytes, ctx.dtype, ctx.redop) : !reduceInto(d, s, in.bytes, ctx.dtype, ctx.redop)) {
          sh.fail(ST_UNSUPPORTED, stream, static_cast<int>(pc));
          return;
        }
        break;
      }
      case OP_NOTIFY: {
        uint32_t slot = ctx.slot_base + in.slot;
        if (ctx.peer_signals[in.dst_rank]) {
          ctx.peer_signals[in.dst_rank][slot].fetch_add(1, std::memory_order_release);
        } else if (!ctx.tcp || !ctx.tcp->signal(in.dst_rank, slot, 1)) {
          sh.fail(ST_PEER_GONE, stream, static_cast<int>(pc));
          return;
        }
        break;
      }
      case OP_WAIT: {
        uint64_t target = ctx.epoch * in.count + in.value;
        if (!waitFor(&my_signals[ctx.slot_base + in.slot], target, ctx, sh)) {
          sh.fail(ST_TIMEOUT, stream, static_cast<int>(pc));
          return;
        }
        break;
      }
      case OP_BARRIER: {
        uint32_t slot = ctx.slot_base + in.slot;
        for (int r = 0; r < ctx.world; ++r) {
          if (ctx.peer_signals[r]) ctx.peer_signals[r][slot].fetch_add(1, std::memory_order_acq_rel);
          else if (!ctx.tcp || !ctx.tcp->signal(r, slot, 1)) {
            sh.fail(ST_PEER_GONE, stream, static_cast<int>(pc));
            return;
          }
        }
        uint64_t target = static_cast<uint64_t>(ctx.world) * (ctx.epoch * in.count + in.value);
        if (!waitFor(&my_signals[slot], target, ctx, sh)) {
          sh.fail(ST_TIMEOUT, stream, static_cast<int>(pc));
          return;
        }
        break;
      }
      default:   // multimem ops need NVSwitch hardware
        sh.fail(ST_UNSUPPORTED, stream, static_cast<int>(pc));
        return;
    }
  }
}

}  // namespace

CpuExecResult runOnCpu(const Materialized& m, const CpuExecContext& ctx) {
  Shared sh;
  uint64_t t0 = monotonicNanos();
  if (ctx.turn_slot >= 0 && ctx.launch_no >= 2) {
    std::atomic<uint64_t>* mine = ctx.peer_signals[ctx.rank];
    for (int r = 0; r < ctx.world; ++r)
      if (r != ctx.rank && !waitFor(&mine[ctx.turn_slot + r], ctx.launch_no - 1, ctx, sh)) {
        CpuExecResult bad;
        bad.status = ST_TIMEOUT;
        bad.failed_stream = -1;
        bad.failed_pc = -1;
        bad.nanos = monotonicNanos() - t0;
        return bad;
      }
  }
  std::vector<std::thread> threads;
  std::vector<std::vector<TraceEvent>> traces(ctx.trace ? m.streams.size() : 0);
  auto tr = [&](size_t i) { return ctx.trace ? &traces[i] : nullptr; };
  for (size_t i = 1; i < m.streams.size(); ++i)
    threads.emplace_back([&, i] { runStream(m.streams[i], static_cast<int>(i), ctx, sh, tr(i)); });
  if (!m.streams.empty()) runStream(m.streams[0], 0, ctx, sh, tr(0));
  for (auto& t : threads) t.join();
  if (ctx.turn_slot >= 0 && sh.status.load() == ST_OK) {
    const uint32_t word = static_cast<uint32_t>(ctx.turn_slot + ctx.rank);
    for (int q = 0; q < ctx.world; ++q) {
      if (q == ctx.rank) continue;
      if (ctx.peer_signals[q]) ctx.peer_signals[q][word].fetch_add(1, std::memory_order_release);
      else if (!ctx.tcp || !ctx.tcp->signal(q, word, 1)) sh.fail(ST_PEER_GONE, -1, -1);
    }
  }
  CpuExecResult r;
  for (auto& v : traces) r.trace.insert(r.trace.end(), v.begin(), v.end());
  r.status = sh.status.load();
  r.failed_stream = sh.failed_stream.load();
  r.failed_pc = sh.failed_pc.load();
  r.nanos = monotonicNanos() - t0;
  return r;
}

}  // namespace pccl
