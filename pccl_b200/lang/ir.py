"""Collective-program IR: chunks, devices, links, primitive ops and ``CollectiveIR``.

API parity with the reference vocabulary (pccl/lang/chunk.py:6-135): the four primitive op kinds
``COPY / REDUCE / NOTIFY / GET_NOTIFIED``, ``Chunk`` with its symbolic ``reduced_ranks`` set,
``Device``, ``Link``, ``PrimitiveOp`` and ``CollectiveIR`` with ``add_device / add_link /
create_operation / set_precondition / set_postcondition / validate_topology / validate_dag /
get_device_bandwidth_matrix / get_operation_sequence``.

What this module adds (the reference stops at an in-memory object that nothing consumes):

* chunk coordinates are *units* of a named buffer (``input`` / ``output`` / ``scratch``), so one
  program serves every message size; the engine scales units to bytes when it loads the program;
* three switch/NVLS op kinds (``MM_LD_REDUCE``, ``MM_ST``, ``BARRIER``);
* each op names the rank that executes it, a channel and a step (filled by the algorithm
  generators or by the MILP synthesiser);
* ``to_json`` / ``from_json``: the on-disk format that ``Engine.regOp(name, path)`` reads
  (include/engine.h:18 takes a file path; the reference never defined the file).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, Iterable, List, Optional, Set, Tuple

from .dag import DirectedGraph

SCHEMA_VERSION = 1
BUFFER_KINDS = ("input", "output", "scratch")


class PrimitiveOpType(Enum):
    COPY = 1
    REDUCE = 2
    NOTIFY = 3
    GET_NOTIFIED = 4
    # Blackwell/NVSwitch extensions: in-switch reduce-load, multicast store, world barrier.
    MM_LD_REDUCE = 5
    MM_ST = 6
    BARRIER = 7


class DeviceType(Enum):
    CUDA = 1
    CPU = 2
    ROCM = 3  # kept for vocabulary parity (chunk.py:15); no executor exists for it here


@dataclass
class Chunk:
    """A run of ``data_size`` units at ``offset`` of ``buffer`` on device ``cur_device_id``.

    ``reduced_ranks`` is the symbolic content: the set of ranks whose contribution has been
    folded into these units.  ``origin`` says which logical units they hold (default: the same
    position, which is right for reductions; all-gather / all-to-all set it explicitly).
    """
    reduced_ranks: Set[int]
    cur_device_id: int
    data_size: int
    offset: int
    buffer: str = "input"
    origin: Optional[int] = None

    def copy(self) -> "Chunk":
        return Chunk(set(self.reduced_ranks), self.cur_device_id, self.data_size, self.offset,
                     self.buffer, self.origin)

    def on(self, device: int, buffer: Optional[str] = None, offset: Optional[int] = None) -> "Chunk":
        c = self.copy()
        c.cur_device_id = device
        if buffer is not None:
            c.buffer = buffer
        if offset is not None:
            c.offset = offset
        return c

    def to_dict(self) -> Dict[str, Any]:
        d = {"ranks": sorted(self.reduced_ranks), "device": self.cur_device_id,
             "size": self.data_size, "offset": self.offset, "buffer": self.buffer}
        if self.origin is not None:
            d["origin"] = self.origin
        return d

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "Chunk":
        return Chunk(set(d.get("ranks", ())), d["device"], d["size"], d["offset"],
                     d.get("buffer", "input"), d.get("origin"))


@dataclass
class Device:
    device_id: int
    device_type: DeviceType = DeviceType.CUDA
    memory_bandwidth: float = 6.4e12   # bytes/s; measured HBM3e copy rate of a B200 is ~6.45e12
    compute_capability: float = 10.0


@dataclass
class Link:
    src_device: int
    dst_device: int
    bandwidth: float = 770e9   # bytes/s per direction; measured NVLink 5 peer-copy rate
    latency: float = 2.0e-6    # seconds


@dataclass
class PrimitiveOp:
    op_type: PrimitiveOpType
    op_id: int
    src_chunk: Optional[Chunk]
    tgt_chunk: Optional[Chunk]
    src_device: Optional[int]
    tgt_device: Optional[int]
    dependencies: List[int] = field(default_factory=list)
    metadata: Dict[str, Any] = field(default_factory=dict)

    @property
    def executor(self) -> int:
        """Rank whose executor runs this op.

        Default: a COPY is a push (runs where the source lives), a REDUCE folds into local
        memory (runs where the target lives), NOTIFY runs on the notifier, GET_NOTIFIED on the
        waiter.  ``metadata['executor']`` overrides (e.g. a pull-style COPY).
        """
        if "executor" in self.metadata:
            return int(self.metadata["executor"])
        t = self.op_type
        if t in (PrimitiveOpType.COPY, PrimitiveOpType.NOTIFY, PrimitiveOpType.MM_ST):
            return int(self.src_device if self.src_device is not None else self.tgt_device)
        return int(self.tgt_device if self.tgt_device is not None else self.src_device)

    @property
    def channel(self) -> int:
        return int(self.metadata.get("channel", 0))

    @property
    def step(self) -> int:
        return int(self.metadata.get("step", 0))


class CollectiveIR:
    """A collective as a DAG of primitive ops over chunks, with pre- and post-conditions."""

    def __init__(self, name: str, collective: str = "custom", units: int = 1,
                 redop: str = "sum", buffers: Optional[Dict[str, int]] = None,
                 in_place: bool = False) -> None:
        self.name = name
        self.collective = collective
        self.units = int(units)            # units in the logical (per-rank input) buffer
        self.redop = redop
        self.in_place = in_place
        # buffer name -> size in units (per rank)
        self.buffers: Dict[str, int] = dict(buffers or {"input": units, "output": units, "scratch": 0})
        self.precondition: List[Chunk] = []
        self.postcondition: List[Chunk] = []
        self.devices: Dict[int, Device] = {}
        self.links: List[Link] = []
        self.ops: Dict[int, PrimitiveOp] = {}
        self.op_dag = DirectedGraph()
        self.device_topology = DirectedGraph()
        self.attrs: Dict[str, Any] = {}
        self._next_op_id = 0

    # -- topology -----------------------------------------------------------------------------
    def add_device(self, device: Device) -> None:
        self.devices[device.device_id] = device
        self.device_topology.add_node(device.device_id, device)

    def add_link(self, link: Link) -> None:
        for d in (link.src_device, link.dst_device):
            if d not in self.devices:
                raise ValueError(f"link names unknown device {d}")
        self.links.append(link)
        self.device_topology.add_edge(link.src_device, link.dst_device, link)

    @property
    def world_size(self) -> int:
        return len(self.devices)

    def fully_connect(self, bandwidth: float = 770e9, latency: float = 2.0e-6) -> None:
        """NVSwitch view: every ordered device pair gets a link."""
        ids = sorted(self.devices)
        for a in ids:
            for b in ids:
                if a != b:
                    self.add_link(Link(a, b, bandwidth, latency))

    # -- ops ----------------------------------------------------------------------------------
    def create_operation(self, op_type: PrimitiveOpType, src_chunk: Optional[Chunk] = None,
                         tgt_chunk: Optional[Chunk] = None, src_device: Optional[int] = None,
                         tgt_device: Optional[int] = None,
                         dependencies: Optional[Iterable[int]] = None,
                         metadata: Optional[Dict[str, Any]] = None) -> int:
        deps = sorted(set(dependencies or ()))
        for d in deps:
            if d not in self.ops:
                raise ValueError(f"dependency {d} is not an op of this program")
        if src_device is None and src_chunk is not None:
            src_device = src_chunk.cur_device_id
        if tgt_device is None and tgt_chunk is not None:
            tgt_device = tgt_chunk.cur_device_id
        op_id = self._next_op_id
        self._next_op_id += 1
        self.ops[op_id] = PrimitiveOp(op_type, op_id, src_chunk, tgt_chunk, src_device, tgt_device,
                                      deps, dict(metadata or {}))
        self.op_dag.add_node(op_id)
        for d in deps:
            self.op_dag.add_edge(d, op_id)
        return op_id

    # convenience wrappers used by the algorithm library
    def copy(self, src: Chunk, dst: Chunk, deps=None, **meta) -> int:
        return self.create_operation(PrimitiveOpType.COPY, src, dst, dependencies=deps, metadata=meta)

    def reduce(self, src: Chunk, dst: Chunk, deps=None, **meta) -> int:
        return self.create_operation(PrimitiveOpType.REDUCE, src, dst, dependencies=deps, metadata=meta)

    def notify(self, src_device: int, tgt_device: int, deps=None, **meta) -> int:
        return self.create_operation(PrimitiveOpType.NOTIFY, None, None, src_device, tgt_device, deps, meta)

    def get_notified(self, src_device: int, tgt_device: int, deps=None, **meta) -> int:
        return self.create_operation(PrimitiveOpType.GET_NOTIFIED, None, None, src_device, tgt_device, deps, meta)

    def set_precondition(self, chunks: List[Chunk]) -> None:
        self.precondition = list(chunks)

    def set_postcondition(self, chunks: List[Chunk]) -> None:
        self.postcondition = list(chunks)

    # -- validation / queries -----------------------------------------------------------------
    def validate_topology(self) -> bool:
        return len(self.devices) > 0 and len(self.device_topology.get_connected_components()) == 1

    def validate_dag(self) -> bool:
        return self.op_dag.is_acyclic()

    def get_device_bandwidth_matrix(self) -> Dict[Tuple[int, int], float]:
        """bytes/s for every ordered pair that has a link (a link serves both directions unless
        the reverse link was given its own figure)."""
        m: Dict[Tuple[int, int], float] = {}
        for l in self.links:
            m.setdefault((l.dst_device, l.src_device), l.bandwidth)
        for l in self.links:
            m[(l.src_device, l.dst_device)] = l.bandwidth
        return m

    def get_operation_sequence(self) -> List[PrimitiveOp]:
        try:
            return [self.ops[i] for i in self.op_dag.topological_sort()]
        except ValueError:
            return []

    def num_steps(self) -> int:
        return 1 + max((op.step for op in self.ops.values()), default=-1)

    def num_channels(self) -> int:
        return 1 + max((op.channel for op in self.ops.values()), default=0)

    # -- JSON ---------------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        def chunk(c: Optional[Chunk]):
            return None if c is None else c.to_dict()
        return {
            "name": self.name, "version": SCHEMA_VERSION, "collective": self.collective,
            "world_size": self.world_size, "units": self.units, "redop": self.redop,
            "in_place": self.in_place, "buffers": dict(self.buffers), "attrs": dict(self.attrs),
            "devices": [{"id": d.device_id, "type": d.device_type.name, "mem_bw": d.memory_bandwidth,
                         "cc": d.compute_capability} for d in self.devices.values()],
            "links": [{"src": l.src_device, "dst": l.dst_device, "bw": l.bandwidth, "lat": l.latency}
                      for l in self.links],
            "precondition": [c.to_dict() for c in self.precondition],
            "postcondition": [c.to_dict() for c in self.postcondition],
            "ops": [{"id": op.op_id, "type": op.op_type.name, "src": chunk(op.src_chunk),
                     "dst": chunk(op.tgt_chunk), "src_device": op.src_device,
                     "dst_device": op.tgt_device, "deps": list(op.dependencies),
                     "executor": op.executor, "channel": op.channel, "step": op.step,
                     "meta": {k: v for k, v in op.metadata.items()
                              if k not in ("executor", "channel", "step")}}
                    for op in self.ops.values()],
        }

    def to_json(self, path: Optional[str] = None, indent: Optional[int] = None) -> str:
        s = json.dumps(self.to_dict(), indent=indent, sort_keys=False)
        if path is not None:
            with open(path, "w") as f:
                f.write(s)
        return s

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "CollectiveIR":
        if d.get("version", SCHEMA_VERSION) != SCHEMA_VERSION:
            raise ValueError(f"unsupported schedule version {d.get('version')}")
        ir = CollectiveIR(d["name"], d.get("collective", "custom"), d.get("units", 1),
                          d.get("redop", "sum"), d.get("buffers"), d.get("in_place", False))
        ir.attrs = dict(d.get("attrs", {}))
        for dev in d.get("devices", []):
            ir.add_device(Device(dev["id"], DeviceType[dev.get("type", "CUDA")],
                                 dev.get("mem_bw", 0.0), dev.get("cc", 0.0)))
        for l in d.get("links", []):
            ir.add_link(Link(l["src"], l["dst"], l.get("bw", 0.0), l.get("lat", 0.0)))
        ir.precondition = [Chunk.from_dict(c) for c in d.get("precondition", [])]
        ir.postcondition = [Chunk.from_dict(c) for c in d.get("postcondition", [])]
        remap: Dict[int, int] = {}
        for o in d.get("ops", []):
            meta = dict(o.get("meta", {}))
            for k in ("executor", "channel", "step"):
                if k in o:
                    meta[k] = o[k]
            new_id = ir.create_operation(
                PrimitiveOpType[o["type"]],
                Chunk.from_dict(o["src"]) if o.get("src") else None,
                Chunk.from_dict(o["dst"]) if o.get("dst") else None,
                o.get("src_device"), o.get("dst_device"),
                [remap[x] for x in o.get("deps", [])], meta)
            remap[o["id"]] = new_id
        return ir

    @staticmethod
    def from_json(text_or_path: str) -> "CollectiveIR":
        s = text_or_path.lstrip()
        if not s.startswith("{"):
            with open(text_or_path) as f:
                s = f.read()
        return CollectiveIR.from_dict(json.loads(s))
