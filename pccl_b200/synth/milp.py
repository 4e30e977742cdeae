"""MILP schedule synthesis (scipy.optimize.milp / HiGHS).

Decision variables, for every chunk k, directed link e = (u, v) and step s:
    x[k,e,s] in {0,1}   chunk k crosses link e during step s
    p[k,u,s] in {0,1}   chunk k is present on device u at the start of step s
    used[s]  in {0,1}   step s carries traffic
    T[s]     >= 0       duration of step s
subject to  x[k,(u,v),s] <= p[k,u,s]                      (send only what you hold)
            p[k,v,s+1]  <= p[k,v,s] + sum_u x[k,(u,v),s]  (data appears only by arriving)
            p[k,v,s+1]  >= p[k,v,s],  >= x[k,(u,v),s]
            sum_{u,s} x[k,(u,v),s] = 1 for every v that must receive k   (a tree per chunk: reversible into a reduction)
            T[s] >= alpha*used[s] + bytes * sum_{k,v} x[k,(u,v),s] / egress[u]     for every u   (port capacity, sending)
            T[s] >= alpha*used[s] + bytes * sum_{k,u} x[k,(u,v),s] / ingress[v]    for every v   (port capacity, receiving)
            T[s] >= alpha*used[s] + bytes * sum_k x[k,(u,v),s] / link[u,v]         for every link
minimise    sum_s T[s]  (+ a tiny cost per transfer).
On a rotation-symmetric topology only rank 0's chunks are variables; the other ranks run the same
pattern rotated, and every port then carries the step's whole transfer count.

The all-gather problem is what is solved; reduce-scatter is its time reversal (each chunk's
broadcast tree becomes a reduction tree), all-reduce is reduce-scatter followed by all-gather.
The result is a ``CollectiveIR`` (scratch-staged pushes) that the verifier checks and both
executors run.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
from scipy.optimize import Bounds, LinearConstraint, milp
from scipy.sparse import lil_matrix

from ..lang import Chunk, CollectiveIR, Device, DeviceType, verify
from ..lang.algorithms import allgather_conditions, allreduce_conditions, alltoall_conditions, reduce_scatter_conditions
from .topology import Topology


@dataclass
class SynthesisResult:
    ir: CollectiveIR
    objective_seconds: float
    steps_used: int
    transfers: List[Tuple[int, int, int, int]]    # (chunk owner rank, chunk index, u, v, ...) per step, see `sends`
    sends: List[List[Tuple[int, int, int, int]]]  # per step: (owner, chunk, u, v)
    status: str
    lower_bound_seconds: float


def _solve_allgather(topo: Topology, chunks: int, steps: int, chunk_bytes: float, symmetric: bool, time_limit: float,
                     alltoall: bool = False, only_owner: Optional[int] = None):
    """Spreading model.  All-gather: commodity (owner o, chunk c) starts on o and must reach everybody.  With
    ``alltoall`` a commodity is (o, destination d, c): it must reach d only, other devices may relay it (they
    receive it at most once).  With ``only_owner`` the chunks of that one rank are the only commodities: a broadcast
    (the rotation shortcut does not apply to it).  Returns per step the transfers (o, c, u, v), or (o, d, c, u, v) for
    all-to-all."""
    n = topo.n
    # Times inside the model are in microseconds: in seconds the coefficients (1e-6) would sit below
    # the solver's feasibility tolerance and it would accept schedules that overrun a port.
    alpha = topo.alpha * 1e6
    chunk_bytes = chunk_bytes * 1e6
    if only_owner is not None:
        symmetric = False
        owners = [only_owner]
    else:
        owners = [0] if symmetric else list(range(n))
    if alltoall:
        K = [(o, c, d) for o in owners for d in range(n) if d != o for c in range(chunks)]
    else:
        K = [(o, c, None) for o in owners for c in range(chunks)]
    E = sorted(topo.link_bw)
    nK, nE, S = len(K), len(E), steps
    ix = lambda k, e, s: (k * nE + e) * S + s                     # noqa: E731
    base_p = nK * nE * S
    ip = lambda k, u, s: base_p + (k * n + u) * (S + 1) + s        # noqa: E731
    base_u = base_p + nK * n * (S + 1)
    base_t = base_u + S
    nv = base_t + S
    rows, lo, hi = [], [], []

    def add(coeffs: Dict[int, float], l: float, h: float):
        rows.append(coeffs)
        lo.append(l)
        hi.append(h)

    lb = np.zeros(nv)
    ub = np.ones(nv)
    ub[base_t:] = np.inf
    integrality = np.ones(nv)
    integrality[base_t:] = 0
    for k, (o, c, dest) in enumerate(K):
        for u in range(n):
            v0 = 1.0 if u == o else 0.0
            lb[ip(k, u, 0)] = ub[ip(k, u, 0)] = v0
            if dest is None or u == dest:
                lb[ip(k, u, S)] = 1.0                                # everybody (all-to-all: the destination) has it at the end
        for s in range(S):
            for e, (u, v) in enumerate(E):
                add({ix(k, e, s): 1.0, ip(k, u, s): -1.0}, -np.inf, 0.0)
                add({ip(k, v, s + 1): 1.0, ix(k, e, s): -1.0}, 0.0, np.inf)
                add({ix(k, e, s): 1.0, base_u + s: -1.0}, -np.inf, 0.0)
            for v in range(n):
                co = {ip(k, v, s + 1): 1.0, ip(k, v, s): -1.0}
                add(dict(co), 0.0, np.inf)                           # monotone
                for e, (a, b) in enumerate(E):
                    if b == v:
                        co[ix(k, e, s)] = co.get(ix(k, e, s), 0.0) - 1.0
                add(co, -np.inf, 0.0)                                # appears only by arriving
        for v in range(n):
            if v == o:
                continue
            co = {}
            for s in range(S):
                for e, (a, b) in enumerate(E):
                    if b == v:
                        co[ix(k, e, s)] = 1.0
            # received exactly once (all-to-all: a relay at most once, the destination exactly once)
            add(co, 1.0 if (dest is None or v == dest) else 0.0, 1.0)
    for s in range(S):
        if symmetric:
            co = {base_t + s: 1.0, base_u + s: -alpha}
            for k in range(nK):
                for e in range(nE):
                    co[ix(k, e, s)] = -chunk_bytes / min(topo.egress_bw[0], topo.ingress_bw[0])
            add(co, 0.0, np.inf)
        else:
            for u in range(n):
                co = {base_t + s: 1.0, base_u + s: -alpha}
                for k in range(nK):
                    for e, (a, b) in enumerate(E):
                        if a == u:
                            co[ix(k, e, s)] = -chunk_bytes / topo.egress_bw[u]
                add(co, 0.0, np.inf)
                co = {base_t + s: 1.0, base_u + s: -alpha}
                for k in range(nK):
                    for e, (a, b) in enumerate(E):
                        if b == u:
                            co[ix(k, e, s)] = -chunk_bytes / topo.ingress_bw[u]
                add(co, 0.0, np.inf)
        for links, cap in getattr(topo, "shared_caps", []):
            if symmetric:
                raise ValueError("shared capacities need the general (non-rotation-symmetric) model")
            co = {base_t + s: 1.0, base_u + s: -alpha}
            members = set(links)
            for k in range(nK):
                for e, (a, b) in enumerate(E):
                    if (a, b) in members:
                        co[ix(k, e, s)] = -chunk_bytes / cap
            add(co, 0.0, np.inf)
        for e, (a, b) in enumerate(E):
            co = {base_t + s: 1.0, base_u + s: -alpha}
            mult = 1.0
            if symmetric:
                # the rotated copies put one transfer on link (a,b) for every variable of the same offset b-a
                for e2, (a2, b2) in enumerate(E):
                    if (b2 - a2) % n == (b - a) % n:
                        for k in range(nK):
                            co[ix(k, e2, s)] = co.get(ix(k, e2, s), 0.0) - chunk_bytes / topo.link_bw[(a, b)]
            else:
                for k in range(nK):
                    co[ix(k, e, s)] = -mult * chunk_bytes / topo.link_bw[(a, b)]
            add(co, 0.0, np.inf)
        if s + 1 < S:
            add({base_u + s: 1.0, base_u + s + 1: -1.0}, 0.0, np.inf)   # used steps come first
    A = lil_matrix((len(rows), nv))
    for i, co in enumerate(rows):
        for j, val in co.items():
            A[i, j] = val
    c = np.zeros(nv)
    c[base_t:] = 1.0
    c[:base_p] = 1e-9
    res = milp(c, constraints=LinearConstraint(A.tocsr(), np.array(lo), np.array(hi)), integrality=integrality,
               bounds=Bounds(lb, ub), options={"time_limit": time_limit, "disp": False})
    if res.x is None:
        return None, res
    sends: List[List[Tuple[int, int, int, int]]] = [[] for _ in range(S)]
    for k, (o, cidx, dest) in enumerate(K):
        for s in range(S):
            for e, (u, v) in enumerate(E):
                if res.x[ix(k, e, s)] > 0.5:
                    for r in (range(n) if symmetric else [0]):
                        if dest is None:
                            sends[s].append(((o + r) % n, cidx, (u + r) % n, (v + r) % n))
                        else:
                            sends[s].append(((o + r) % n, (dest + r) % n, cidx, (u + r) % n, (v + r) % n))
    return sends, res


def _build_allgather_ir(n: int, chunks: int, sends, name: str) -> CollectiveIR:
    sh = chunks
    ir = CollectiveIR(name, "allgather", sh, buffers={"input": sh, "output": n * sh, "scratch": n * sh})
    ir.attrs["block_units"] = sh
    for r in range(n):
        ir.add_device(Device(r, DeviceType.CUDA))
    ir.fully_connect()
    allgather_conditions(ir, n, sh)
    have: Dict[Tuple[int, int, int], int] = {}       # (owner, chunk, device) -> op that made it available in `output`
    for r in range(n):
        for c in range(sh):
            org = r * sh + c
            have[(r, c, r)] = ir.copy(Chunk({r}, r, 1, c, "input", origin=org), Chunk({r}, r, 1, org, "output", origin=org),
                                      step=0, channel=c % max(1, sh))
    for s, step_sends in enumerate(sends):
        new = {}
        for (o, c, u, v) in step_sends:
            org = o * sh + c
            push = ir.copy(Chunk({o}, u, 1, org, "output", origin=org), Chunk({o}, v, 1, org, "scratch", origin=org),
                           deps=[have[(o, c, u)]], step=1 + 2 * s, channel=c)
            new[(o, c, v)] = ir.copy(Chunk({o}, v, 1, org, "scratch", origin=org), Chunk({o}, v, 1, org, "output", origin=org),
                                     deps=[push], step=2 + 2 * s, channel=c)
        have.update(new)
    return ir


def _build_broadcast_ir(n: int, chunks: int, sends, name: str, root: int) -> CollectiveIR:
    """The root's vector in ``chunks`` pieces; every hop lands in the receiver's scratch slot of the piece and is copied
    into its output, from where it may be forwarded.  Ranks that only send get an acknowledgement at the end."""
    from ..lang import add_acknowledgements
    U = chunks
    ir = CollectiveIR(name, "broadcast", U, buffers={"input": U, "output": U, "scratch": U})
    ir.attrs["block_units"] = U
    ir.attrs["root"] = root
    for r in range(n):
        ir.add_device(Device(r, DeviceType.CUDA))
    ir.fully_connect()
    ir.set_precondition([Chunk({root}, root, U, 0, "input")])
    ir.set_postcondition([Chunk({root}, r, U, 0, "output") for r in range(n)])
    have: Dict[Tuple[int, int], int] = {}
    for c in range(U):
        have[(c, root)] = ir.copy(Chunk({root}, root, 1, c, "input"), Chunk({root}, root, 1, c, "output"), step=0, channel=c)
    for s, step_sends in enumerate(sends):
        new = {}
        for (_o, c, u, v) in step_sends:
            push = ir.copy(Chunk({root}, u, 1, c, "output"), Chunk({root}, v, 1, c, "scratch", origin=c),
                           deps=[have[(c, u)]], step=1 + 2 * s, channel=c)
            new[(c, v)] = ir.copy(Chunk({root}, v, 1, c, "scratch", origin=c), Chunk({root}, v, 1, c, "output"),
                                  deps=[push], step=2 + 2 * s, channel=c)
        have.update(new)
    add_acknowledgements(ir)
    return ir


def _build_alltoall_ir(n: int, chunks: int, sends, name: str) -> CollectiveIR:
    """Block d of rank o's input becomes block o of rank d's output.  Every hop lands in the receiver's scratch slot
    of its (o, d, c) -- relays forward from there, the destination copies it into its output -- so nobody writes a
    peer's input or output tensor and the program also runs on the host executor."""
    blk = chunks
    U = n * blk
    ir = CollectiveIR(name, "alltoall", U, buffers={"input": U, "output": U, "scratch": n * U})
    ir.attrs["block_units"] = blk
    for r in range(n):
        ir.add_device(Device(r, DeviceType.CUDA))
    ir.fully_connect()
    alltoall_conditions(ir, n, blk)
    held: Dict[Tuple[int, int, int, int], Tuple[str, int, Optional[int]]] = {}     # (o, d, c, device) -> (buffer, unit, producing op)
    for o in range(n):
        for c in range(blk):
            org = o * U + o * blk + c
            ir.copy(Chunk({o}, o, 1, o * blk + c, "input", origin=org), Chunk({o}, o, 1, o * blk + c, "output", origin=org), step=0, channel=c)
            for d in range(n):
                if d != o:
                    held[(o, d, c, o)] = ("input", d * blk + c, None)
    for s, step_sends in enumerate(sends):
        new = {}
        for (o, d, c, u, v) in step_sends:
            org = o * U + d * blk + c
            buf, unit, op = held[(o, d, c, u)]
            slot = o * U + d * blk + c
            push = ir.copy(Chunk({o}, u, 1, unit, buf, origin=org), Chunk({o}, v, 1, slot, "scratch", origin=org),
                           deps=[] if op is None else [op], step=1 + 2 * s, channel=c)
            new[(o, d, c, v)] = ("scratch", slot, push)
            if v == d:
                ir.copy(Chunk({o}, v, 1, slot, "scratch", origin=org), Chunk({o}, v, 1, o * blk + c, "output", origin=org),
                        deps=[push], step=2 + 2 * s, channel=c)
        held.update(new)
    return ir


def _build_reduce_scatter_ir(n: int, chunks: int, sends, name: str, redop: str) -> CollectiveIR:
    """Time reversal of an all-gather: the tree that spread chunk (o, c) from o now gathers it into o."""
    sh = chunks
    ir = CollectiveIR(name, "reduce_scatter", n * sh, redop=redop, buffers={"input": n * sh, "output": sh, "scratch": (n * n + n) * sh})
    ir.attrs["block_units"] = sh
    for r in range(n):
        ir.add_device(Device(r, DeviceType.CUDA))
    ir.fully_connect()
    reduce_scatter_conditions(ir, n, sh)
    # accumulators: device d keeps its running partial of shard (o, c) in scratch block (o), unit c, except o itself -> output
    acc_op: Dict[Tuple[int, int, int], int] = {}
    acc_set: Dict[Tuple[int, int, int], set] = {}

    def acc_chunk(o, c, d, ranks):
        if d == o:
            return Chunk(set(ranks), d, 1, c, "output", origin=o * sh + c)
        return Chunk(set(ranks), d, 1, o * sh + c, "scratch", origin=o * sh + c)

    for d in range(n):
        for o in range(n):
            for c in range(sh):
                acc_op[(o, c, d)] = ir.copy(Chunk({d}, d, 1, o * sh + c, "input"), acc_chunk(o, c, d, {d}), step=0, channel=c)
                acc_set[(o, c, d)] = {d}
    S = len(sends)
    for rs, s in enumerate(reversed(range(S))):
        for (o, c, u, v) in sends[s]:            # all-gather sent u -> v: now v hands its partial to u
            src = acc_chunk(o, c, v, acc_set[(o, c, v)])
            rslot = Chunk(set(acc_set[(o, c, v)]), u, 1, _recv_unit(n, sh, v, o, c), "scratch", origin=o * sh + c)
            push = ir.copy(src, rslot, deps=[acc_op[(o, c, v)]], step=1 + 2 * rs, channel=c)
            merged = acc_set[(o, c, u)] | acc_set[(o, c, v)]
            acc_op[(o, c, u)] = ir.reduce(rslot, acc_chunk(o, c, u, merged), deps=[push, acc_op[(o, c, u)]], step=2 + 2 * rs, channel=c)
            acc_set[(o, c, u)] = merged
    return ir


def _build_reduce_ir(n: int, chunks: int, sends, name: str, redop: str, root: int) -> CollectiveIR:
    """A broadcast schedule run backwards: where the broadcast sent piece c from u to v, v now hands its partial of
    piece c to u, which folds it in; the root ends with the reduction of everybody's vector in its output.  Scratch:
    block 0 holds a rank's running partials, block 1 + v the partials received from rank v."""
    from ..lang import add_acknowledgements
    U = chunks
    ir = CollectiveIR(name, "reduce", U, redop, buffers={"input": U, "output": U, "scratch": (n + 1) * U})
    ir.attrs["block_units"] = U
    ir.attrs["root"] = root
    for r in range(n):
        ir.add_device(Device(r, DeviceType.CUDA))
    ir.fully_connect()
    everyone = set(range(n))
    ir.set_precondition([Chunk({r}, r, U, 0, "input") for r in range(n)])
    ir.set_postcondition([Chunk(everyone, root, U, 0, "output")])

    def acc_chunk(c, d, ranks):
        return Chunk(set(ranks), d, 1, c, "output") if d == root else Chunk(set(ranks), d, 1, c, "scratch", origin=c)
    acc_op: Dict[Tuple[int, int], int] = {}
    acc_set: Dict[Tuple[int, int], set] = {}
    for d in range(n):
        for c in range(U):
            acc_op[(c, d)] = ir.copy(Chunk({d}, d, 1, c, "input"), acc_chunk(c, d, {d}), step=0, channel=c)
            acc_set[(c, d)] = {d}
    S = len(sends)
    for rs, s in enumerate(reversed(range(S))):
        for (_o, c, u, v) in sends[s]:
            rslot = Chunk(set(acc_set[(c, v)]), u, 1, (1 + v) * U + c, "scratch", origin=c)
            push = ir.copy(acc_chunk(c, v, acc_set[(c, v)]), rslot, deps=[acc_op[(c, v)]], step=1 + 2 * rs, channel=c)
            merged = acc_set[(c, u)] | acc_set[(c, v)]
            acc_op[(c, u)] = ir.reduce(rslot, acc_chunk(c, u, merged), deps=[push, acc_op[(c, u)]], step=2 + 2 * rs, channel=c)
            acc_set[(c, u)] = merged
    add_acknowledgements(ir)
    return ir


def _recv_unit(n: int, sh: int, v: int, o: int, c: int) -> int:
    """Scratch unit on a receiver for the partial of shard (o, c) sent by device v.  Scratch blocks
    (of `sh` units): [0, n) running partials per shard, [n, n + n*n) one receive slot per (sender, shard)."""
    return (n + v * n + o) * sh + c


def synthesize(collective: str, topo: Topology, nbytes: int, chunks: int = 1, max_steps: Optional[int] = None,
               redop: str = "sum", time_limit: float = 20.0, check: bool = True, root: int = 0) -> SynthesisResult:
    """Synthesise a schedule for `collective` in {"allgather", "reduce_scatter", "allreduce", "alltoall", "broadcast",
    "reduce"} (a rooted reduce is the broadcast's schedule run backwards) moving `nbytes` per rank (all-gather: bytes each rank contributes; reduce-scatter / all-reduce: bytes of the full
    vector; all-to-all: bytes of a rank's whole input, i.e. n blocks; broadcast: bytes of ``root``'s vector, which
    travels in ``chunks`` pieces -- with as many pieces as ranks the solver finds the scatter + all-gather form)."""
    n = topo.n
    if collective not in ("allgather", "reduce_scatter", "allreduce", "alltoall", "broadcast", "reduce"):
        raise ValueError("synthesize: unsupported collective")
    if not 0 <= root < n:
        raise ValueError("synthesize: root is not a rank of the topology")
    rooted = collective in ("broadcast", "reduce")
    shard_bytes = nbytes if (collective == "allgather" or rooted) else nbytes / n
    chunk_bytes = shard_bytes / chunks
    symmetric = topo.rotation_symmetric
    result = None
    steps_try = [max_steps] if max_steps else list(range(1, n + 1))
    best = None
    for S in steps_try:
        sends, res = _solve_allgather(topo, chunks, S, chunk_bytes, symmetric, time_limit, alltoall=collective == "alltoall",
                                      only_owner=root if rooted else None)
        if sends is None:
            continue
        obj = float(res.fun) * 1e-6
        if best is None or obj < best[0] - 1e-12:
            best = (obj, S, sends, res)
        elif best is not None and obj >= best[0] - 1e-12 and S > best[1] + 1:
            break                                   # more steps stopped helping
    if best is None:
        raise RuntimeError("synthesize: no feasible schedule (is the topology connected?)")
    obj, S, sends, res = best
    sends = [st for st in sends if st]
    name = f"milp_{collective}_{topo.name}_c{chunks}_s{len(sends)}"
    if collective == "allgather":
        ir = _build_allgather_ir(n, chunks, sends, name)
        total = obj
    elif collective == "reduce_scatter":
        ir = _build_reduce_scatter_ir(n, chunks, sends, name, redop)
        total = obj
    elif collective == "alltoall":
        ir = _build_alltoall_ir(n, chunks, sends, name)
        total = obj
    elif collective == "broadcast":
        ir = _build_broadcast_ir(n, chunks, sends, name, root)
        total = obj
    elif collective == "reduce":
        ir = _build_reduce_ir(n, chunks, sends, name, redop, root)
        total = obj
    else:
        ir = _compose_allreduce(n, chunks, sends, name, redop)
        total = 2 * obj
    ir.attrs.update({"synthesized": True, "topology": topo.fingerprint(), "objective_us": total * 1e6, "steps": len(sends)})
    if check:
        verify(ir).raise_if_failed()
    # lower bound: every rank must receive (n-1) shards through its ingress port, in at least one step
    lb = topo.alpha + (n - 1) * shard_bytes / min(min(topo.ingress_bw), min(topo.egress_bw))
    if collective == "allreduce":
        lb *= 2
    if rooted:                          # the vector has to leave (enter) the root and to enter (leave) every other rank once
        lb = topo.alpha + shard_bytes / min(topo.egress_bw[root], min(b for r, b in enumerate(topo.ingress_bw) if r != root))
    return SynthesisResult(ir, total, len(sends), [], sends, str(res.message), lb)


def _compose_allreduce(n: int, chunks: int, sends, name: str, redop: str) -> CollectiveIR:
    """Reduce-scatter (reversed trees) into the output, then all-gather (forward trees) of the reduced shards."""
    sh = chunks
    U = n * sh
    # scratch: n blocks of accumulators (block o holds partials of shard o), n*n - n receive blocks, n blocks for the gather
    ir = CollectiveIR(name, "allreduce", U, redop=redop, buffers={"input": U, "output": U, "scratch": (n * n + n) * U})
    ir.attrs["block_units"] = U
    for r in range(n):
        ir.add_device(Device(r, DeviceType.CUDA))
    ir.fully_connect()
    allreduce_conditions(ir, n, U)
    full = set(range(n))
    acc_op, acc_set = {}, {}

    def acc_chunk(o, c, d, ranks):
        u = o * sh + c
        if d == o:
            return Chunk(set(ranks), d, 1, u, "output")
        return Chunk(set(ranks), d, 1, u, "scratch", origin=u)       # block 0 of scratch mirrors the vector

    for d in range(n):
        for o in range(n):
            for c in range(sh):
                u = o * sh + c
                acc_op[(o, c, d)] = ir.copy(Chunk({d}, d, 1, u, "input"), acc_chunk(o, c, d, {d}), step=0, channel=c)
                acc_set[(o, c, d)] = {d}
    S = len(sends)
    step = 1
    for s in reversed(range(S)):
        for (o, c, u_dev, v_dev) in sends[s]:
            u = o * sh + c
            src = acc_chunk(o, c, v_dev, acc_set[(o, c, v_dev)])
            rslot = Chunk(set(acc_set[(o, c, v_dev)]), u_dev, 1, (1 + v_dev) * U + u, "scratch", origin=u)
            push = ir.copy(src, rslot, deps=[acc_op[(o, c, v_dev)]], step=step, channel=c)
            merged = acc_set[(o, c, u_dev)] | acc_set[(o, c, v_dev)]
            acc_op[(o, c, u_dev)] = ir.reduce(rslot, acc_chunk(o, c, u_dev, merged), deps=[push, acc_op[(o, c, u_dev)]],
                                              step=step + 1, channel=c)
            acc_set[(o, c, u_dev)] = merged
        step += 2
    have = {(o, c, o): acc_op[(o, c, o)] for o in range(n) for c in range(sh)}
    for s in range(S):
        new = {}
        for (o, c, u_dev, v_dev) in sends[s]:
            u = o * sh + c
            push = ir.copy(Chunk(full, u_dev, 1, u, "output"), Chunk(full, v_dev, 1, (n + 1) * U + u, "scratch", origin=u),
                           deps=[have[(o, c, u_dev)], acc_op[(o, c, v_dev)]], step=step, channel=c)
            new[(o, c, v_dev)] = ir.copy(Chunk(full, v_dev, 1, (n + 1) * U + u, "scratch", origin=u), Chunk(full, v_dev, 1, u, "output"),
                                         deps=[push], step=step + 1, channel=c)
        have.update(new)
        step += 2
    return ir
