"""Kernels compiled at run time for ONE registered program, message size and width.

The reference links nvrtc (setup.py:60) for kernels generated from its operator graphs and has no generator.  Here the
generator takes the instruction streams that the engine materialises for this rank (the same ones the interpreter
kernel would fetch and decode) and writes them out as straight-line CUDA: one ``case`` per stream, every offset, byte
count, signal slot and peer rank a constant, the data type and reduction baked into the template arguments, chains of
"wait, reduce into the same destination" already folded into one n-ary pass and "in-switch reduce, multicast store of
the result" into one loop.  The loops themselves are the interpreter's (``csrc/kernels/interp_ops.cuh``), so a generated
kernel moves data exactly like the interpreted program; what disappears is the fetch / decode / dispatch per
instruction.  NVRTC compiles the source to an sm_100a cubin (no GPU is needed for that), the CUDA driver loads it, and
a launch goes through ``Engine.planLaunch`` for the same signal ranges, launch numbers, scratch halves and lane
turn-taking as ``exeOp`` -- the two may be mixed freely on one engine.

    op = JitOp(engine, "ar")          # a program registered with regOp
    op(x, y, width=4)                 # compiles on first use of (bytes, dtype, width), then launches

Every wait is bounded like in the interpreter; a wait that runs out writes the status words and the kernel returns.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
from typing import Dict, List, Optional, Tuple

import torch

from .engine import Engine, PcclError, dtype_name

_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
OP = {"NOP": 0, "COPY": 1, "REDUCE": 2, "NOTIFY": 3, "WAIT": 4, "MM_LD_REDUCE": 5, "MM_ST": 6, "BARRIER": 7, "END": 8}
BUF_INPUT, BUF_OUTPUT, BUF_SCRATCH = 0, 1, 2
_DT = {"f32": "DT_F32", "bf16": "DT_BF16", "f16": "DT_F16"}
_RED = {"sum": "RED_SUM", "max": "RED_MAX", "min": "RED_MIN", "prod": "RED_PROD"}
_MM_OK = {("f32", "sum"), ("bf16", "sum"), ("bf16", "max"), ("bf16", "min"), ("f16", "sum"), ("f16", "max"), ("f16", "min")}
MAX_FUSED = 8

_PROLOGUE = r"""
#include "interp_ops.cuh"
using namespace pccl;
using namespace pccl::dev;
using namespace pccl::iops;

struct JitArgs {
  char* const* heap;              // device array: every rank's heap as mapped here
  char* mc_heap;
  unsigned long long signal_off;
  char* input;
  char* output;
  long long in_off, out_off;      // heap offsets of the tensors, or -1
  unsigned long long scratch_off, epoch, spin_limit, launch_no;
  unsigned int* status;
  unsigned int slot_base, turn_slot, finish_slot, pad;
};

__device__ __forceinline__ char* io_ptr(const JitArgs& a, int q, int me, bool is_input, unsigned long long off) {
  if (q == me) return (is_input ? a.input : a.output) + off;
  const long long ho = is_input ? a.in_off : a.out_off;
  return ho < 0 ? nullptr : a.heap[q] + ho + off;
}
"""


def _addr(rank: int, me: int, buf: int, off: int) -> str:
    if buf == BUF_SCRATCH:
        return f"(a.heap[{rank}] + a.scratch_off + {off}ull)"
    return f"io_ptr(a, {rank}, {me}, {'true' if buf == BUF_INPUT else 'false'}, {off}ull)"


def _mc_addr(buf: int, off: int) -> str:
    if buf == BUF_SCRATCH:
        return f"(a.mc_heap + a.scratch_off + {off}ull)"
    return f"(a.mc_heap + {'a.in_off' if buf == BUF_INPUT else 'a.out_off'} + {off}ull)"


def _wait(slot: int, count: int, value: int, stream: int, pc: int) -> List[str]:
    return [f"if (threadIdx.x == 0 && !wait_ge(my_sig + {slot}, a.epoch * {count}ull + {value}ull, a.spin_limit, a.status)) s_fail = ST_TIMEOUT;",
            "__syncthreads();",
            f"if (s_fail) {{ if (threadIdx.x == 0) report(a.status, ST_TIMEOUT, {stream}u, {pc}u, OP_WAIT); return; }}"]


def generate(streams: List[List[Tuple]], rank: int, world: int, dtype: str, redop: str, name: str = "pccl_jit") -> str:
    """CUDA source of the kernel that runs ``streams`` (tuples ``(op, src_rank, dst_rank, src_buf, dst_buf, slot, value,
    count, src_off, dst_off, bytes)`` per stream, as ``Engine.materializedStreams`` returns them) for rank ``rank``."""
    if dtype not in _DT or redop not in _RED:
        raise PcclError(f"jit: no generated form for dtype {dtype!r} / reduction {redop!r} (use exeOp)")
    DT, RED = _DT[dtype], _RED[redop]
    n_workers = max(1, len(streams))
    uses_scratch = any(ins[0] != OP["END"] and BUF_SCRATCH in (ins[3], ins[4]) and ins[0] in (OP["COPY"], OP["REDUCE"], OP["MM_LD_REDUCE"], OP["MM_ST"])
                       for prog in streams for ins in prog)
    out = [_PROLOGUE, f'extern "C" __global__ void __launch_bounds__(512) {name}(const JitArgs a) {{',
           "  __shared__ unsigned int s_fail;",
           f"  const int me = {rank};",
           f"  if (blockIdx.x >= {n_workers}u) return;",
           "  if (threadIdx.x == 0) s_fail = 0;",
           "  __syncthreads();",
           "  unsigned long long* const sig0 = reinterpret_cast<unsigned long long*>(a.heap[me] + a.signal_off);",
           "  unsigned long long* const my_sig = sig0 + a.slot_base;",
           "  const bool turns = a.turn_slot != 0xffffffffu;",
           # a program that moves nothing through scratch has no scratch half to wait for; one thread per peer otherwise
           f"  if (turns && a.launch_no >= 2 && {'true' if uses_scratch else 'false'}) {{",
           f"    if (threadIdx.x < {world}u && threadIdx.x != {rank}u && !wait_ge(sig0 + a.turn_slot + threadIdx.x, a.launch_no - 1, a.spin_limit, a.status))",
           "      s_fail = ST_TIMEOUT;",
           "    __syncthreads();",
           "    if (s_fail) { if (threadIdx.x == 0) report(a.status, ST_TIMEOUT, blockIdx.x, 0xffffu, OP_WAIT); return; }",
           "  }",
           "  switch (blockIdx.x) {"]
    for s, prog in enumerate(streams):
        body: List[str] = []
        pc = 0
        n = len(prog)
        while pc < n:
            op, src_rank, dst_rank, src_buf, dst_buf, slot, value, count, src_off, dst_off, nbytes = prog[pc]
            if op == OP["END"]:
                break
            if op == OP["NOP"] or (op in (OP["COPY"], OP["REDUCE"], OP["MM_LD_REDUCE"], OP["MM_ST"]) and nbytes == 0):
                pc += 1
                continue
            if op == OP["COPY"]:
                body.append(f"{{ char* d = {_addr(dst_rank, rank, dst_buf, dst_off)}; const char* sp = {_addr(src_rank, rank, src_buf, src_off)};")
                body.append(f"  if (!d || !sp) {{ if (threadIdx.x == 0) report(a.status, ST_UNSUPPORTED, {s}u, {pc}u, OP_COPY); return; }}")
                # fence + barrier: a later instruction of this stream may read d, which was stored to without having been
                # loaded first (the interpreter kernel's note on folded copies says what was seen without them)
                body.append(f"  if (d != sp) {{ copy_range(d, sp, {nbytes}ull); __threadfence(); }} }}")
                body.append("__syncthreads();")
                pc += 1
            elif op == OP["REDUCE"]:
                # fold the "WAIT; REDUCE" pairs and plain REDUCEs that follow with the same destination
                srcs = [(src_rank, src_buf, src_off)]
                waits: List[Tuple[int, int, int, int]] = []
                j = pc + 1
                aligned = nbytes % 16 == 0 and dst_off % 16 == 0 and src_off % 16 == 0
                while aligned and len(srcs) < MAX_FUSED and j < n:
                    nxt = prog[j]
                    is_wait = nxt[0] == OP["WAIT"] and j + 1 < n and prog[j + 1][0] == OP["REDUCE"]
                    r = prog[j + 1] if is_wait else nxt
                    if not is_wait and nxt[0] != OP["REDUCE"]:
                        break
                    if (r[2], r[4], r[9], r[10]) != (dst_rank, dst_buf, dst_off, nbytes) or r[8] % 16:
                        break
                    if is_wait:
                        waits.append((nxt[5], nxt[7], nxt[6], j))
                    srcs.append((r[1], r[3], r[8]))
                    j += 2 if is_wait else 1
                for (w_slot, w_count, w_value, w_pc) in waits:
                    body += _wait(w_slot, w_count, w_value, s, w_pc)
                body.append(f"{{ char* d = {_addr(dst_rank, rank, dst_buf, dst_off)};")
                body.append(f"  char* srcs[{MAX_FUSED}] = {{{', '.join(_addr(q, rank, b, o) for (q, b, o) in srcs)}}};")
                body.append("  bool ok = d != nullptr;")
                body.append(f"  for (int i = 0; i < {len(srcs)}; ++i) ok = ok && srcs[i] != nullptr;")
                body.append(f"  if (!ok) {{ if (threadIdx.x == 0) report(a.status, ST_UNSUPPORTED, {s}u, {pc}u, OP_REDUCE); return; }}")
                if len(srcs) > 1:
                    body.append(f"  if (((reinterpret_cast<unsigned long long>(d) | reinterpret_cast<unsigned long long>(srcs[0])) & 15) == 0) "
                                f"reduce_n_range_f<{DT}, {RED}>(d, srcs, {len(srcs)}, {nbytes}ull);")
                    body.append(f"  else for (int i = 0; i < {len(srcs)}; ++i) {{ reduce_range_f<{DT}, {RED}>(d, srcs[i], {nbytes}ull); __syncthreads(); }} }}")
                else:
                    body.append(f"  reduce_range_f<{DT}, {RED}>(d, srcs[0], {nbytes}ull); }}")
                pc = j
            elif op == OP["NOTIFY"]:
                body.append("__syncthreads();")
                body.append(f"if (threadIdx.x == 0) {{ __threadfence_system(); red_add_release_sys(reinterpret_cast<uint64_t*>(a.heap[{dst_rank}] + "
                            f"a.signal_off) + a.slot_base + {slot}, 1); }}")
                pc += 1
            elif op == OP["WAIT"]:
                body += _wait(slot, count, value, s, pc)
                pc += 1
            elif op == OP["BARRIER"]:
                body.append("__syncthreads();")
                body.append(f"if (threadIdx.x < {world}u) {{ __threadfence_system(); red_add_release_sys(reinterpret_cast<uint64_t*>(a.heap[threadIdx.x] + "
                            f"a.signal_off) + a.slot_base + {slot}, 1); }}")
                body.append(f"if (threadIdx.x == 0 && !wait_ge(my_sig + {slot}, {world}ull * (a.epoch * {count}ull + {value}ull), a.spin_limit, a.status)) "
                            "s_fail = ST_TIMEOUT;")
                body.append("__syncthreads();")
                body.append(f"if (s_fail) {{ if (threadIdx.x == 0) report(a.status, ST_TIMEOUT, {s}u, {pc}u, OP_BARRIER); return; }}")
                pc += 1
            elif op in (OP["MM_LD_REDUCE"], OP["MM_ST"]):
                if (dtype, redop) not in _MM_OK and op == OP["MM_LD_REDUCE"]:
                    raise PcclError(f"jit: no in-switch reduction for {dtype} / {redop}")
                if nbytes % 16 or src_off % 16 or dst_off % 16:
                    raise PcclError("jit: multimem instructions need 16-byte aligned ranges")
                fused = (op == OP["MM_LD_REDUCE"] and pc + 1 < n and prog[pc + 1][0] == OP["MM_ST"] and
                         (prog[pc + 1][3], prog[pc + 1][8]) == (dst_buf, dst_off) and (prog[pc + 1][4], prog[pc + 1][9]) == (dst_buf, dst_off)
                         and prog[pc + 1][10] == nbytes)
                body.append(f"if (!a.mc_heap) {{ if (threadIdx.x == 0) report(a.status, ST_UNSUPPORTED, {s}u, {pc}u, {op}u); return; }}")
                if fused:
                    body.append(f"mm_reduce_bcast_range<{DT}, {RED}>({_mc_addr(dst_buf, dst_off)}, {_mc_addr(src_buf, src_off)}, {nbytes}ull);")
                    pc += 2
                elif op == OP["MM_LD_REDUCE"]:
                    body.append(f"mm_ld_reduce_range<{DT}, {RED}>({_addr(rank, rank, dst_buf, dst_off)}, {_mc_addr(src_buf, src_off)}, {nbytes}ull);")
                    pc += 1
                else:
                    body.append(f"mm_st_range({_mc_addr(dst_buf, dst_off)}, {_addr(rank, rank, src_buf, src_off)}, {nbytes}ull);")
                    pc += 1
            else:
                raise PcclError(f"jit: opcode {op} has no generated form")
        out.append(f"    case {s}: {{")
        out += ["      " + line for line in body]
        out.append("    } break;")
    out += ["    default: break;", "  }",
            "  if (turns) {",
            "    __shared__ unsigned int s_last;",
            "    __syncthreads();",
            "    if (threadIdx.x == 0) {",
            "      __threadfence_system();",
            "      unsigned int* fin = reinterpret_cast<unsigned int*>(sig0 + a.finish_slot);",
            f"      s_last = atomicInc(fin, {n_workers - 1}u) == {n_workers - 1}u ? 1u : 0u;",
            "    }",
            "    __syncthreads();",
            f"    if (s_last && threadIdx.x < {world}u && threadIdx.x != {rank}u)",
            "      red_add_release_sys(reinterpret_cast<uint64_t*>(a.heap[threadIdx.x] + a.signal_off) + a.turn_slot + me, 1);",
            "  }", "}"]
    return "\n".join(out)


def compile_cubin(source: str, cuda_include: Optional[str] = None) -> bytes:
    """NVRTC: CUDA source -> sm_100a cubin.  Works without a GPU."""
    from cuda.bindings import nvrtc
    inc = cuda_include or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    opts = [b"--gpu-architecture=sm_100a", b"-std=c++17", b"-default-device", b"--use_fast_math",
            f"-I{os.path.join(_CSRC, 'kernels', 'jit_shim')}".encode(), f"-I{inc}".encode(),
            f"-I{os.path.join(_CSRC, 'kernels')}".encode(), f"-I{_CSRC}".encode()]
    err, prog = nvrtc.nvrtcCreateProgram(source.encode(), b"pccl_jit.cu", 0, [], [])
    if int(err) != 0:
        raise PcclError(f"nvrtcCreateProgram: {err}")
    try:
        (err,) = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
        if int(err) != 0:
            _, n = nvrtc.nvrtcGetProgramLogSize(prog)
            log = b" " * n
            nvrtc.nvrtcGetProgramLog(prog, log)
            raise PcclError("jit: compilation failed\n" + log.decode(errors="replace")[-4000:])
        _, n = nvrtc.nvrtcGetCUBINSize(prog)
        cubin = b" " * n
        (err,) = nvrtc.nvrtcGetCUBIN(prog, cubin)
        if int(err) != 0:
            raise PcclError(f"nvrtcGetCUBIN: {err}")
        return cubin
    finally:
        nvrtc.nvrtcDestroyProgram(prog)


def source_for(engine: Engine, name: str, nbytes: int, dtype: str, width: int = 1) -> str:
    """Generated source of program ``name`` as registered with ``engine`` (any device kind: generating and compiling need
    no GPU) for this rank, message size, data type and width."""
    streams, _ = engine._e.materializedStreams(name, nbytes, width)
    info = engine._e.opInfo(name)
    kname = "pccl_jit_" + hashlib.sha1(f"{name}/{nbytes}/{dtype}/{width}".encode()).hexdigest()[:12]
    return generate([list(s) for s in streams], engine.rank, engine.world, dtype, info["redop"], kname)


class _JitArgs(ctypes.Structure):
    _fields_ = [("heap", ctypes.c_uint64), ("mc_heap", ctypes.c_uint64), ("signal_off", ctypes.c_uint64), ("input", ctypes.c_uint64),
                ("output", ctypes.c_uint64), ("in_off", ctypes.c_int64), ("out_off", ctypes.c_int64), ("scratch_off", ctypes.c_uint64),
                ("epoch", ctypes.c_uint64), ("spin_limit", ctypes.c_uint64), ("launch_no", ctypes.c_uint64), ("status", ctypes.c_uint64),
                ("slot_base", ctypes.c_uint32), ("turn_slot", ctypes.c_uint32), ("finish_slot", ctypes.c_uint32), ("pad", ctypes.c_uint32)]


class JitOp:
    """A registered program as run-time compiled kernels, one per (message bytes, dtype, width)."""

    def __init__(self, engine: Engine, name: str):
        if engine.device != "cuda":
            raise PcclError("JitOp needs a CUDA engine")
        self.eng, self.name = engine, name
        self._kernels: Dict[Tuple[int, str, int], Tuple[object, object, int]] = {}
        self._heaps = torch.tensor([engine._e.heapBase(r) for r in range(engine.world)] + [0] * (16 - engine.world), dtype=torch.int64,
                                   device="cuda")
        self.compiled = 0
        info = engine._e.opInfo(name)
        self.redop, self.in_place = info["redop"], info["in_place"] == "1"

    def source(self, nbytes: int, dtype: str, width: int = 1) -> str:
        """The generated CUDA source for one (message bytes, dtype, width): for reading, or for compiling elsewhere."""
        return source_for(self.eng, self.name, nbytes, dtype, width)

    def _kernel(self, nbytes: int, dtype: str, width: int):
        key = (nbytes, dtype, width)
        hit = self._kernels.get(key)
        if hit is not None:
            return hit
        from cuda.bindings import driver
        streams, _ = self.eng._e.materializedStreams(self.name, nbytes, width)
        kname = "pccl_jit_" + hashlib.sha1(f"{self.name}/{nbytes}/{dtype}/{width}".encode()).hexdigest()[:12]
        src = generate([list(s) for s in streams], self.eng.rank, self.eng.world, dtype, self.redop, kname)
        cubin = compile_cubin(src)
        torch.cuda.current_stream()                      # the primary context is current
        err, mod = driver.cuModuleLoadData(cubin)
        if int(err) != 0:
            raise PcclError(f"cuModuleLoadData: {err}")
        err, fn = driver.cuModuleGetFunction(mod, kname.encode())
        if int(err) != 0:
            raise PcclError(f"cuModuleGetFunction: {err}")
        self.compiled += 1
        self._kernels[key] = (mod, fn, max(1, len(streams)))
        return self._kernels[key]

    def __call__(self, input: torch.Tensor, output: Optional[torch.Tensor] = None, *, width: int = 1, lane: int = 0,
                 stream: Optional["torch.cuda.Stream"] = None, in_place: bool = False) -> None:
        from cuda.bindings import driver
        if not input.is_cuda or not input.is_contiguous() or (output is not None and not output.is_contiguous()):
            raise PcclError("JitOp needs contiguous CUDA tensors")
        out = input if (output is None or in_place or self.in_place) else output
        nbytes = input.numel() * input.element_size()
        dt = dtype_name(input.dtype)
        _, fn, grid = self._kernel(nbytes, dt, width)
        plan = self.eng._e.planLaunch(self.name, nbytes, width, lane)
        base, total = self.eng._e.heapBase(self.eng.rank), self.eng._e.heapBytes()
        off = lambda p: p - base if base <= p < base + total else -1  # noqa: E731
        args = _JitArgs(self._heaps.data_ptr(), plan["mc_base"], plan["signal_off"], input.data_ptr(), out.data_ptr(), off(input.data_ptr()),
                        off(out.data_ptr()), plan["scratch_off"], plan["epoch"], plan["spin_limit"], plan["launch_no"], plan["status_ptr"],
                        plan["slot_base"], plan["turn_slot"], plan["finish_slot"], 0)
        s = (stream or torch.cuda.current_stream()).cuda_stream
        # the streams of a program wait on one another: cooperative launch, refused rather than hung when they do not fit
        holder = (ctypes.c_void_p * 1)(ctypes.addressof(args))
        (err,) = driver.cuLaunchCooperativeKernel(fn, grid, 1, 1, 512, 1, 1, 0, s, ctypes.addressof(holder))
        if int(err) != 0:
            raise PcclError(f"jit launch of '{self.name}': {err}")
