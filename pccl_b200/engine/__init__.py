"""``pccl.engine``: Python face of the C++ engine.

The reference leaves this package empty (pccl/engine/__init__.py is 0 bytes) and binds the C++
class directly as ``pccl.engine_c.Engine`` with ``initEngine / regOp / exeOp / exportEndpoint /
joinCluster / exitCluster`` (csrc/python_api.cc:13-20).  ``Engine`` here keeps those six names and
adds the torch-facing conveniences: tensors instead of pointers, a rendezvous through
``torch.distributed`` when one exists, symmetric tensors, NVLS bring-up and status checks.
"""
from __future__ import annotations

import json
import os
import tempfile
from typing import Dict, List, Optional, Sequence, Union

import torch

from .._native import C
from ..lang import CollectiveIR, to_schedule, verify
from ..lang import algorithms as _alg

engine_c = C     # the reference's module name for the raw bindings

_DTYPE_NAMES = {
    torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16", torch.float64: "f64",
    torch.int32: "i32", torch.int64: "i64", torch.uint8: "u8", torch.int8: "u8",
}
if hasattr(torch, "float8_e4m3fn"):
    _DTYPE_NAMES[torch.float8_e4m3fn] = "fp8_e4m3"

STATUS_NAMES = {0: "ok", 1: "timeout", 2: "bounds", 3: "bad_op", 4: "unsupported", 5: "peer_gone"}


class PcclError(RuntimeError):
    pass


class PcclTimeout(PcclError):
    """A bounded wait ran out: some peer never signalled (it left, died, or never launched)."""


def dtype_name(dt: torch.dtype) -> str:
    try:
        return _DTYPE_NAMES[dt]
    except KeyError:
        raise PcclError(f"unsupported dtype {dt}") from None


class _CudaBlob:
    """Exposes a raw device range to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}
        self._owner = owner


class Engine:
    """One rank of a PCCL job.

    >>> eng = Engine(rank, world); eng.initEngine(); eng.joinCluster("127.0.0.1:29700")
    >>> eng.regOp("ar", ring_allreduce(world))         # a CollectiveIR, a JSON path or JSON text
    >>> eng.exeOp("ar", x, y)
    """

    def __init__(self, rank: int, world: int):
        self._e = C.Engine(rank, world)
        self.rank, self.world = rank, world
        self._tmpfiles: List[str] = []
        self._initialized = False

    # -- the six reference methods ---------------------------------------------------------------
    def initEngine(self, device: str = "auto", heap_bytes: int = 0) -> None:
        if device == "auto":
            device = "cuda" if torch.cuda.is_available() else "cpu"
        if device == "cuda":
            torch.cuda.current_device()           # make the primary context current on this thread
            torch.zeros(1, device="cuda")
        self._e.initEngine(device, int(heap_bytes))
        self.device = device
        self._initialized = True

    def regOp(self, name: str, program: Union[str, CollectiveIR, dict], check: bool = True) -> None:
        """Register a collective program under ``name``.  ``program`` is a ``CollectiveIR`` (verified
        and lowered here), a schedule dict, JSON text, or the path of a schedule file."""
        if isinstance(program, CollectiveIR):
            if check:
                verify(program).raise_if_failed()
            program = to_schedule(program)
        elif check:
            self._check_document(program)
        if isinstance(program, dict):
            program = json.dumps(program)
        self._e.regOp(name, program)

    @staticmethod
    def _check_document(program) -> None:
        """A schedule document carries the op DAG it was lowered from: a sender that nothing holds back (unsafe to launch
        repeatedly) is refused here too.  Anything that does not parse is left to the native loader's error message."""
        from ..lang import VerificationError, relaunch_hazards
        try:
            doc = program
            if isinstance(program, str):
                if program.lstrip().startswith("{"):
                    doc = json.loads(program)
                else:
                    with open(program) as f:
                        doc = json.load(f)
            if not isinstance(doc, dict) or not doc.get("ops"):
                return
            hazards = relaunch_hazards(CollectiveIR.from_dict(doc))
        except (OSError, ValueError, KeyError, TypeError, AttributeError):
            return
        if hazards:
            s_, r_ = hazards[0]
            raise VerificationError(f"relaunch: rank {s_} writes into rank {r_}'s workspace but waits for nothing from it "
                                    f"(pccl.lang.add_acknowledgements closes this; check=False registers the program as it is)")

    def prepareOp(self, name: str, width: int = 1) -> None:
        """Reserve the signal words of ``name`` at ``width`` now.  Only needed when several host threads launch
        different ops at the same time (communication-communication overlap on the host executor): every rank
        prepares them in the same order first, so that all ranks number the words alike."""
        self._e.prepareOp(name, int(width))

    def exeOp(self, name: str, input: torch.Tensor, output: Optional[torch.Tensor] = None, *,
              width: int = 1, lane: int = 0, stream: Optional["torch.cuda.Stream"] = None,
              check: Optional[bool] = None) -> int:
        """Run a registered program on ``input`` (-> ``output``).  ``width`` replicates every channel
        (more CTAs or threads: runtime resource control); ``lane`` picks the workspace lane so that
        ops on different lanes may overlap on different streams."""
        if not input.is_contiguous() or (output is not None and not output.is_contiguous()):
            raise PcclError("exeOp needs contiguous tensors")
        out = input if output is None else output
        sh = 0
        if input.is_cuda:
            sh = (stream or torch.cuda.current_stream()).cuda_stream
        st = self._e.exeOp(name, input.data_ptr(), out.data_ptr(), input.numel() * input.element_size(),
                           dtype_name(input.dtype), int(width), int(lane), int(sh))
        if check is None:
            check = not input.is_cuda
        if check:
            if input.is_cuda:
                st = self.check_status(lane)[0]
            if st != 0:
                exc = PcclTimeout if st == 1 else PcclError
                raise exc(f"exeOp('{name}') finished with status {STATUS_NAMES.get(st, st)}")
        return st

    # -- resident executor: one kernel that stays on the GPU and takes launches from a queue -----------------------
    def start_resident(self, width: int = 4) -> None:
        """Launch the resident interpreter kernel with ``width`` CTAs per channel.  From then on ``enqueue`` hands it a
        registered program without a kernel launch (a descriptor written to pinned memory); ``wait`` blocks until a
        ticket is done.  The kernel leaves by itself after ``PCCL_RESIDENT_IDLE_MS`` without work and comes back with
        the next ``enqueue``."""
        self._e.startResident(int(width))

    def enqueue(self, name: str, input: torch.Tensor, output: Optional[torch.Tensor] = None, *, lane: int = 0,
                stream: Optional["torch.cuda.Stream"] = None, sync_inputs: bool = True) -> int:
        """Queue one run of program ``name`` for the resident kernel; returns its ticket.  With ``sync_inputs`` the
        producing stream (default: the current one) is synchronised first, because the resident kernel is not ordered
        behind any stream.  Keep the tensors alive until ``wait(ticket)`` has returned."""
        if not input.is_cuda or not input.is_contiguous() or (output is not None and not output.is_contiguous()):
            raise PcclError("enqueue needs contiguous CUDA tensors")
        out = input if output is None else output
        sh = (stream or torch.cuda.current_stream()).cuda_stream if sync_inputs else 0
        if sync_inputs and sh == 0:
            torch.cuda.current_stream().synchronize()
        return self._e.enqueueOp(name, input.data_ptr(), out.data_ptr(), input.numel() * input.element_size(),
                                 dtype_name(input.dtype), int(lane), int(sh))

    def wait(self, ticket: int, timeout_ms: int = 0) -> None:
        if not self._e.waitOp(int(ticket), int(timeout_ms)):
            raise PcclTimeout(f"resident executor: ticket {ticket} did not finish in time")

    def stop_resident(self) -> None:
        self._e.stopResident()

    def exportEndpoint(self) -> str:
        return self._e.exportEndpoint()

    def joinCluster(self, master_endpoint: str, timeout_ms: int = 60000) -> None:
        self._e.joinCluster(master_endpoint, timeout_ms)

    def exitCluster(self) -> None:
        self._e.exitCluster()

    # -- rendezvous through torch.distributed ----------------------------------------------------
    def connect(self, group=None, nvls: Optional[bool] = None) -> None:
        """Exchange endpoint documents over an existing ``torch.distributed`` group, map every
        peer's heap and (on NVSwitch machines) bind the heap to an NVLS multicast object."""
        import torch.distributed as dist
        self._group, self._connected_dist = group, True
        docs: List[Optional[str]] = [None] * self.world
        dist.all_gather_object(docs, self.exportEndpoint(), group=group)
        self._e.importEndpoints([d for d in docs if d is not None])
        if nvls is None:
            # PCCL_NVLS=0 or PCCL_TRANSPORT=p2p keep the heap off the multicast object: every kernel then takes its
            # peer-to-peer form
            nvls = os.environ.get("PCCL_NVLS", "1") != "0" and os.environ.get("PCCL_TRANSPORT", "") != "p2p"
        if self.device == "cuda" and nvls and self.world > 1 and not self._e.mixedHosts():
            flags = [None] * self.world
            dist.all_gather_object(flags, bool(self._e.multicastSupported()), group=group)
            if all(flags):
                handle = [self._e.mcCreate() if self.rank == 0 else None]
                dist.broadcast_object_list(handle, src=0, group=group)
                self._e.mcJoin(handle[0])
                dist.barrier(group=group)
                self._e.mcBind()
                dist.barrier(group=group)
        dist.barrier(group=group)

    def barrier(self) -> None:
        """Host barrier over the ranks of this engine (device work of this rank is synchronised first).  Objects
        that zero symmetric flags when they are built call it, so that no peer's first kernel can write
        a flag that is cleared afterwards.  A no-op for a world of one or an engine not connected through
        ``torch.distributed``."""
        if self.world == 1 or not getattr(self, "_connected_dist", False):
            return
        import torch.distributed as dist
        if self.device == "cuda":
            torch.cuda.synchronize()
        dist.barrier(group=self._group)

    # -- symmetric memory ------------------------------------------------------------------------
    def symmetric_tensor(self, shape: Sequence[int], dtype: torch.dtype, align: int = 256) -> torch.Tensor:
        """A tensor inside the symmetric heap.  Every rank must allocate the same sequence of shapes,
        which gives the tensor the same heap offset everywhere (peers address it by offset)."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = self._e.allocSymmetric(max(nbytes, 16), align)
        return self.tensor_at(off, shape, dtype)

    def tensor_at(self, heap_off: int, shape: Sequence[int], dtype: torch.dtype, rank: Optional[int] = None) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if rank is not None and rank != self.rank and self.device == "cuda":
            raise PcclError("a peer's heap cannot be wrapped as a torch tensor; use read_peer / write_peer")
        base = self._e.heapBase(self.rank if rank is None else rank)
        if base == 0:
            raise PcclError("that rank's heap is not mapped")
        if self.device == "cuda":
            t = torch.as_tensor(_CudaBlob(base + heap_off, max(nbytes, 1), self), device="cuda")
        else:
            import ctypes
            buf = (ctypes.c_uint8 * max(nbytes, 1)).from_address(base + heap_off)
            t = torch.frombuffer(buf, dtype=torch.uint8)
        return t[:nbytes].view(dtype).view(*shape)

    def read_peer(self, rank: int, heap_off: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """Copy of `shape` elements at `heap_off` of rank `rank`'s heap (a device-to-device copy over
        NVLink for CUDA ranks, a shared-memory read for CPU ranks)."""
        if self.device != "cuda":
            return self.tensor_at(heap_off, shape, dtype, rank=rank).clone()
        out = torch.empty(tuple(shape), dtype=dtype, device="cuda")
        base = self._e.heapBase(rank)
        if base == 0:
            raise PcclError("that rank's heap is not mapped")
        C.memcpy_d2d(out.data_ptr(), base + heap_off, out.numel() * out.element_size(), torch.cuda.current_stream().cuda_stream)
        return out

    def write_peer(self, rank: int, heap_off: int, src: torch.Tensor) -> None:
        if self.device != "cuda":
            self.tensor_at(heap_off, src.shape, src.dtype, rank=rank).copy_(src)
            return
        src = src.contiguous()
        C.memcpy_d2d(self._e.heapBase(rank) + heap_off, src.data_ptr(), src.numel() * src.element_size(),
                     torch.cuda.current_stream().cuda_stream)

    def heap_offset(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self._e.heapBase(self.rank)
        if off < 0 or off >= self._e.heapBytes():
            raise PcclError("tensor is not inside the symmetric heap")
        return off

    def is_symmetric(self, t: torch.Tensor) -> bool:
        off = t.data_ptr() - self._e.heapBase(self.rank)
        return 0 <= off < self._e.heapBytes()

    def symmetric_mark(self) -> int:
        return self._e.symmetricMark()

    def symmetric_reset(self, mark: int) -> None:
        self._e.resetSymmetric(mark)

    @property
    def has_nvls(self) -> bool:
        return self._e.mcBase() != 0

    # -- status / introspection --------------------------------------------------------------------
    def check_status(self, lane: int = 0) -> List[int]:
        return list(self._e.checkStatus(lane))

    def raise_on_status(self, lane: int = 0, what: str = "collective") -> None:
        st = self.check_status(lane)
        if st[0] != 0:
            exc = PcclTimeout if st[0] == 1 else PcclError
            raise exc(f"{what}: status {STATUS_NAMES.get(st[0], st[0])} (detail {st[1:]})")

    def stats(self) -> Dict:
        return json.loads(self._e.stats())

    def trace(self, path: Optional[str] = None) -> Dict:
        """Instruction-level Chrome trace (recorded while ``PCCL_TRACE=1``); written to ``path`` when given
        (open it in chrome://tracing or Perfetto).  The CPU executor stamps host time; the interpreter
        kernel stamps ``%globaltimer`` around every instruction, and a traced GPU launch is followed by a
        synchronize of its stream, so trace to look at a schedule and time with ``timed_exeOp``."""
        doc = json.loads(self._e.trace())
        if path:
            with open(path, "w") as f:
                json.dump(doc, f)
        return doc

    def timed_exeOp(self, name: str, input: torch.Tensor, output: Optional[torch.Tensor] = None, **kw) -> float:
        """``exeOp`` bracketed by CUDA events on the launching stream; returns milliseconds on the device."""
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        self.exeOp(name, input, output, **kw)
        b.record()
        b.synchronize()
        return a.elapsed_time(b)

    def layout(self) -> Dict:
        return dict(self._e.layout())

    @property
    def raw(self):
        return self._e

    # elastic membership
    def alive_ranks(self) -> List[int]:
        return list(self._e.aliveRanks())

    def wait_for_departure(self, rank: int, timeout_ms: int = 10000) -> bool:
        return bool(self._e.waitForDeparture(rank, timeout_ms))

    def resize_world(self) -> Dict[int, int]:
        return dict(self._e.resizeWorld())

    def last_resize(self) -> Dict[int, int]:
        return dict(self._e.lastResize())

    def rebind(self, new_rank: int, new_world: int) -> None:
        self._e.rebind(new_rank, new_world)
        self.rank, self.world = new_rank, new_world

    def inject_fault(self, kind: str) -> None:
        self._e.injectFault(kind)


class LaunchEnvironments:
    """Option registry (reference: ``utils.LaunchEnvironments`` in csrc/python_api.cc:22-27)."""
    listOpt = staticmethod(C.utils.LaunchEnvironments.listOpt)
    getEnv = staticmethod(C.utils.LaunchEnvironments.getEnv)
    registerOpt = staticmethod(C.utils.LaunchEnvironments.registerOpt)
    helpOf = staticmethod(C.utils.LaunchEnvironments.helpOf)
    setOverride = staticmethod(C.utils.LaunchEnvironments.setOverride)


__all__ = ["Engine", "LaunchEnvironments", "PcclError", "PcclTimeout", "engine_c", "dtype_name", "STATUS_NAMES"]
