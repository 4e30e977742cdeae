"""Cost model of a collective program on a topology, and algorithm selection with it.

``estimate`` prices a ``CollectiveIR`` with the model the MILP synthesiser optimises: the ops of one step run side by
side; a step costs a launch/flag latency (when it moves data between devices) plus the time of its busiest resource
-- a device's egress or ingress port, a directed link, a shared capacity such as a host's network card, or a device's
own memory for local copies and reductions.  ``choose`` prices every library algorithm of a collective that fits the
world and the topology's links (optionally the MILP schedule too) and returns them best first.  The reference has no
cost model; its ``Link`` records carry ``bandwidth`` and ``latency`` (pccl/lang/chunk.py:39-44) for one.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

from ..lang import ALGORITHMS, CollectiveIR, PrimitiveOpType
from .topology import Topology


def bytes_per_unit(ir: CollectiveIR, nbytes: int) -> float:
    """``nbytes`` is what ``Engine.exeOp`` is given as input: the whole vector (all-reduce, reduce-scatter, all-to-all) or
    one rank's shard (all-gather).  A program measures its buffers in units; its input buffer holds ``nbytes``."""
    return nbytes / float(ir.buffers["input"])


@dataclass
class Estimate:
    seconds: float
    steps: int
    remote_bytes: float                 # bytes that cross between devices, summed over the world
    busiest: str                        # what bounds the longest step
    per_step: List[float]


def estimate(ir: CollectiveIR, topo: Topology, nbytes: int, memory_gbs: float = 3000.0) -> Optional[Estimate]:
    """Seconds for ``ir`` to move/reduce ``nbytes`` on ``topo``; None when the program uses a link the topology lacks."""
    bpu = bytes_per_unit(ir, nbytes)
    steps: Dict[int, List] = {}
    for op in ir.ops.values():
        steps.setdefault(op.step, []).append(op)
    total, per_step, remote_total = 0.0, [], 0.0
    worst, worst_time = "", -1.0
    mem = memory_gbs * 1e9
    for s in sorted(steps):
        egress: Dict[int, float] = {}
        ingress: Dict[int, float] = {}
        link: Dict[Tuple[int, int], float] = {}
        local: Dict[int, float] = {}
        multimem = False
        for op in steps[s]:
            if op.op_type in (PrimitiveOpType.NOTIFY, PrimitiveOpType.GET_NOTIFIED, PrimitiveOpType.BARRIER):
                continue
            if op.op_type in (PrimitiveOpType.MM_LD_REDUCE, PrimitiveOpType.MM_ST):
                # in-switch: the issuing device's port carries the vector once, whatever the number of replicas
                dev = (op.tgt_chunk if op.op_type == PrimitiveOpType.MM_LD_REDUCE else op.src_chunk).cur_device_id
                nb = (op.tgt_chunk or op.src_chunk).data_size * bpu
                side = ingress if op.op_type == PrimitiveOpType.MM_LD_REDUCE else egress
                side[dev] = side.get(dev, 0.0) + nb
                other = egress if op.op_type == PrimitiveOpType.MM_LD_REDUCE else ingress
                for d in ir.devices:                # every replica's port carries its copy
                    if d != dev:
                        other[d] = other.get(d, 0.0) + nb
                multimem = True
                continue
            a, b = op.src_chunk.cur_device_id, op.tgt_chunk.cur_device_id
            nb = op.src_chunk.data_size * bpu
            if a == b:
                local[a] = local.get(a, 0.0) + nb * (3 if op.op_type == PrimitiveOpType.REDUCE else 2)     # read(s) + write
                continue
            if (a, b) not in topo.link_bw:
                return None
            egress[a] = egress.get(a, 0.0) + nb
            ingress[b] = ingress.get(b, 0.0) + nb
            link[(a, b)] = link.get((a, b), 0.0) + nb
            remote_total += nb
        cands = [(v / topo.egress_bw[d], f"egress port of device {d}") for d, v in egress.items()]
        cands += [(v / topo.ingress_bw[d], f"ingress port of device {d}") for d, v in ingress.items()]
        cands += [(v / topo.link_bw[k], f"link {k[0]}->{k[1]}") for k, v in link.items()]
        for links, cap in topo.shared_caps:
            v = sum(link.get(k, 0.0) for k in links)
            if v:
                cands.append((v / cap, f"shared capacity of {len(links)} links"))
        cands += [(v / mem, f"memory of device {d}") for d, v in local.items()]
        t, what = max(cands, default=(0.0, "nothing"))
        t += topo.alpha if (link or multimem) else 0.0
        per_step.append(t)
        total += t
        if t > worst_time:
            worst_time, worst = t, f"step {s}: {what}"
    return Estimate(total, len(per_step), remote_total, worst, per_step)


# Forms of one library algorithm that are priced separately.
_VARIANTS = {"broadcast": ({"tree": False}, {"tree": True})}


def choose(collective: str, topo: Topology, nbytes: int, channels: int = 1, include_milp: bool = False,
           nvls: bool = False, **build_kw) -> List[Tuple[str, Estimate, CollectiveIR]]:
    """Library algorithms of ``collective`` that run on ``topo`` (and, with ``include_milp``, the synthesised schedule),
    cheapest first: ``[(name, estimate, ir), ...]``.  NVLS programs are priced only when ``nvls`` says the machine has
    a multicast-capable switch."""
    import inspect
    out = []
    for name, gen in sorted(ALGORITHMS.items()):
        if name.startswith("nvls_") and not nvls:
            continue
        accepted = inspect.signature(gen).parameters
        kw = {k: v for k, v in build_kw.items() if k in accepted}      # per_host, redop, device_type: only where they apply
        for variant in _VARIANTS.get(name, ({},)):
            if any(k in kw for k in variant):
                if any(kw[k] != v for k, v in variant.items() if k in kw):
                    continue                             # the caller fixed this argument to another value
            try:
                ir = gen(topo.n, channels=channels, **{**variant, **kw})
            except (ValueError, TypeError):
                continue                                 # the world does not fit this algorithm (power of two, hosts, ...)
            if ir.collective != collective or ir.attrs.get("use"):
                continue
            est = estimate(ir, topo, nbytes)
            if est is not None:
                label = name + "".join(f"[{k}]" for k, v in variant.items() if v is True)
                out.append((label, est, ir))
    if include_milp:
        from .milp import synthesize
        res = synthesize(collective, topo, nbytes, chunks=channels, time_limit=20.0)
        est = estimate(res.ir, topo, nbytes)
        if est is not None:
            out.append((res.ir.name, est, res.ir))
    out.sort(key=lambda x: x[1].seconds)
    return out


__all__ = ["estimate", "choose", "Estimate", "bytes_per_unit"]
