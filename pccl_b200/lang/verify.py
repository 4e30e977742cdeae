"""Symbolic verifier and static race check for collective programs.

The reference gives chunks a symbolic ``reduced_ranks`` set and programs a pre/post-condition
(pccl/lang/chunk.py:17-23,60-61,110-114) but contains no code that uses them.  This module is the
abstract interpreter they imply: it runs the op DAG over *sets of contributing ranks* instead of
numbers and proves that a program implements its collective for any payload, and it rejects
programs whose memory accesses can race.

State: for every (device, buffer, unit) either ``None`` (undefined) or ``(origin, ranks)`` where
``origin`` identifies the logical datum and ``ranks`` is the frozenset of contributions in it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, FrozenSet, List, Optional, Tuple

from .ir import Chunk, CollectiveIR, PrimitiveOpType as T

Value = Optional[Tuple[int, FrozenSet[int]]]


class VerificationError(Exception):
    pass


@dataclass
class Report:
    ok: bool
    errors: List[str]
    num_ops: int
    num_steps: int
    critical_path: float
    bytes_moved_units: Dict[Tuple[int, int], int]   # (src,dst) -> units crossing that link

    def raise_if_failed(self) -> "Report":
        if not self.ok:
            raise VerificationError("; ".join(self.errors[:8]))
        return self


def _buf(ir: CollectiveIR, name: str) -> str:
    return "input" if (ir.in_place and name == "output") else name


def _key(ir: CollectiveIR, c: Chunk, device: Optional[int] = None):
    return (c.cur_device_id if device is None else device, _buf(ir, c.buffer))


def _accesses(ir: CollectiveIR, op) -> Tuple[List[tuple], List[tuple]]:
    """(reads, writes) as lists of (device, buffer, offset, size)."""
    reads, writes = [], []
    s, t = op.src_chunk, op.tgt_chunk
    devs = sorted(ir.devices)
    if op.op_type == T.COPY:
        reads.append((*_key(ir, s), s.offset, s.data_size))
        writes.append((*_key(ir, t), t.offset, t.data_size))
    elif op.op_type == T.REDUCE:
        reads.append((*_key(ir, s), s.offset, s.data_size))
        reads.append((*_key(ir, t), t.offset, t.data_size))
        writes.append((*_key(ir, t), t.offset, t.data_size))
    elif op.op_type == T.MM_LD_REDUCE:
        for d in devs:
            reads.append((*_key(ir, s, d), s.offset, s.data_size))
        writes.append((*_key(ir, t), t.offset, t.data_size))
    elif op.op_type == T.MM_ST:
        reads.append((*_key(ir, s), s.offset, s.data_size))
        for d in devs:
            writes.append((*_key(ir, t, d), t.offset, t.data_size))
    return reads, writes


def relaunch_hazards(ir: CollectiveIR) -> List[Tuple[int, int]]:
    """Pairs (s, r) such that rank s writes into rank r's workspace but nothing rank s executes depends on anything
    rank r executes.

    The engine alternates between two halves of the workspace from launch to launch and never clears a signal, so a
    program is run again without any barrier between launches.  That is safe as long as a writer cannot get two
    launches ahead of the rank it writes to.  If some op of s depends on some op of r, then s ends launch L+1 only
    after r has begun it, hence after r has finished launch L, and the half that s overwrites in launch L+2 is no
    longer read.  A rank that only ever sends has no such tie and needs an acknowledgement from its receiver."""
    if not ir.ops:
        return []
    anc = ir.op_dag.reachability()
    index = anc["__index__"]
    mask_of: Dict[int, int] = {}
    reach_of: Dict[int, int] = {}
    for op in ir.ops.values():
        e = op.executor
        mask_of[e] = mask_of.get(e, 0) | (1 << index[op.op_id])
        reach_of[e] = reach_of.get(e, 0) | anc[op.op_id]
    pairs = set()
    for op in ir.ops.values():
        _reads, writes = _accesses(ir, op)
        for dev, buf, _off, _size in writes:
            if buf == "scratch" and dev != op.executor:
                pairs.add((op.executor, dev))
    return sorted((s, r) for s, r in pairs if not (reach_of.get(s, 0) & mask_of.get(r, 0)))


def add_acknowledgements(ir: CollectiveIR) -> int:
    """Closes every relaunch hazard of ``ir`` in place and returns how many it closed: for a pair (s, r) the receiver r
    sends a NOTIFY to s once everything that consumes s's writes on r has run, and s ends with the matching
    GET_NOTIFIED.  A program that has none is left as it is."""
    added = 0
    for s_, r_ in relaunch_hazards(ir):
        pushes = []
        for op in ir.ops.values():
            if op.executor != s_:
                continue
            _reads, writes = _accesses(ir, op)
            if any(buf == "scratch" and dev == r_ for dev, buf, _o, _n in writes):
                pushes.append(op)
        consumers = sorted({c for p in pushes for c in ir.op_dag.get_successors(p.op_id) if ir.ops[c].executor == r_})
        after = consumers or [p.op_id for p in pushes]
        last = max(pushes, key=lambda o: (o.step, o.op_id))
        step = max(ir.ops[o].step for o in after) + 1
        nt = ir.notify(r_, s_, deps=after, step=step, channel=last.channel)
        ir.get_notified(r_, s_, deps=[nt], step=step, channel=last.channel)
        added += 1
    return added


def verify(ir: CollectiveIR, check_races: bool = True, check_remote_scratch_only: bool = False,
           check_annotations: bool = True, check_relaunch: bool = True) -> Report:
    errors: List[str] = []
    if not ir.validate_dag():
        return Report(False, ["op DAG has a cycle"], len(ir.ops), 0, 0.0, {})
    if not ir.validate_topology():
        errors.append("device topology is not connected")

    # ---- symbolic execution -----------------------------------------------------------------
    state: Dict[Tuple[int, str], List[Value]] = {}
    for d in ir.devices:
        for b, units in ir.buffers.items():
            state.setdefault((d, _buf(ir, b)), [None] * units)
            if len(state[(d, _buf(ir, b))]) < units:
                state[(d, _buf(ir, b))].extend([None] * (units - len(state[(d, _buf(ir, b))])))

    def cells(dev: int, buf: str, off: int, size: int, what: str) -> Optional[List[Value]]:
        arr = state.get((dev, buf))
        if arr is None or off < 0 or off + size > len(arr):
            errors.append(f"{what}: range [{off},{off+size}) outside buffer {buf!r} on device {dev}")
            return None
        return arr

    for c in ir.precondition:
        arr = cells(*_key(ir, c), c.offset, c.data_size, "precondition")
        if arr is None:
            continue
        base = c.offset if c.origin is None else c.origin
        for i in range(c.data_size):
            arr[c.offset + i] = (base + i, frozenset(c.reduced_ranks))

    links = set((l.src_device, l.dst_device) for l in ir.links)
    traffic: Dict[Tuple[int, int], int] = {}
    for op in ir.get_operation_sequence():
        s, t = op.src_chunk, op.tgt_chunk
        tag = f"op {op.op_id} ({op.op_type.name})"
        if op.op_type in (T.NOTIFY, T.GET_NOTIFIED, T.BARRIER):
            continue
        if s is None or t is None:
            errors.append(f"{tag}: missing chunk")
            continue
        if s.data_size != t.data_size:
            errors.append(f"{tag}: size mismatch {s.data_size} vs {t.data_size}")
            continue
        ex = op.executor
        for c in (s, t):
            if c.cur_device_id != ex:
                if op.op_type in (T.COPY, T.REDUCE):
                    pair = (s.cur_device_id, t.cur_device_id)
                    if pair[0] != pair[1] and pair not in links and (pair[1], pair[0]) not in links:
                        errors.append(f"{tag}: no link {pair[0]}->{pair[1]}")
                if check_remote_scratch_only and c.buffer != "scratch":
                    errors.append(f"{tag}: executor {ex} touches non-symmetric buffer "
                                  f"{c.buffer!r} of device {c.cur_device_id}")
        if s.cur_device_id != t.cur_device_id and op.op_type in (T.COPY, T.REDUCE):
            k = (s.cur_device_id, t.cur_device_id)
            traffic[k] = traffic.get(k, 0) + s.data_size

        if op.op_type == T.MM_LD_REDUCE:
            dst = cells(*_key(ir, t), t.offset, t.data_size, tag)
            srcs = [cells(*_key(ir, s, d), s.offset, s.data_size, tag) for d in sorted(ir.devices)]
            if dst is None or any(a is None for a in srcs):
                continue
            for i in range(s.data_size):
                vals = [a[s.offset + i] for a in srcs]
                if any(v is None for v in vals):
                    errors.append(f"{tag}: in-switch reduce reads undefined unit {s.offset+i}")
                    break
                org = {v[0] for v in vals}
                allr = [r for v in vals for r in v[1]]
                if len(org) != 1 or len(allr) != len(set(allr)):
                    errors.append(f"{tag}: replicas disagree on origin or overlap in ranks")
                    break
                dst[t.offset + i] = (vals[0][0], frozenset(allr))
                for d in ir.devices:
                    if d != ex:
                        traffic[(d, ex)] = traffic.get((d, ex), 0) + 1
            continue
        src = cells(*_key(ir, s), s.offset, s.data_size, tag)
        if src is None:
            continue
        if op.op_type == T.MM_ST:
            vals = [src[s.offset + i] for i in range(s.data_size)]
            if any(v is None for v in vals):
                errors.append(f"{tag}: multicast store of undefined data")
                continue
            for d in sorted(ir.devices):
                dst = cells(*_key(ir, t, d), t.offset, t.data_size, tag)
                if dst is not None:
                    dst[t.offset:t.offset + t.data_size] = vals
                    if d != ex:
                        traffic[(ex, d)] = traffic.get((ex, d), 0) + t.data_size
            continue
        dst = cells(*_key(ir, t), t.offset, t.data_size, tag)
        if dst is None:
            continue
        for i in range(s.data_size):
            v = src[s.offset + i]
            if v is None:
                errors.append(f"{tag}: reads undefined unit {s.offset+i} of {s.buffer!r}@{s.cur_device_id}")
                break
            if check_annotations and v[1] != frozenset(s.reduced_ranks):
                errors.append(f"{tag}: source annotated {sorted(s.reduced_ranks)} but holds {sorted(v[1])}")
                break
            if op.op_type == T.COPY:
                dst[t.offset + i] = v
            else:
                w = dst[t.offset + i]
                if w is None:
                    errors.append(f"{tag}: reduces into undefined unit {t.offset+i}")
                    break
                if w[0] != v[0]:
                    errors.append(f"{tag}: reduces different logical data ({w[0]} vs {v[0]})")
                    break
                if w[1] & v[1]:
                    errors.append(f"{tag}: contribution of ranks {sorted(w[1] & v[1])} counted twice")
                    break
                dst[t.offset + i] = (v[0], w[1] | v[1])

    for c in ir.postcondition:
        arr = cells(*_key(ir, c), c.offset, c.data_size, "postcondition")
        if arr is None:
            continue
        base = c.offset if c.origin is None else c.origin
        for i in range(c.data_size):
            v = arr[c.offset + i]
            want = (base + i, frozenset(c.reduced_ranks))
            if v != want:
                errors.append(f"postcondition: {c.buffer!r}@{c.cur_device_id} unit {c.offset+i} holds "
                              f"{None if v is None else (v[0], sorted(v[1]))}, wanted {(want[0], sorted(want[1]))}")
                break

    # ---- static race check --------------------------------------------------------------------
    if check_races and not errors:
        anc = ir.op_dag.reachability()
        index = anc["__index__"]
        touched: Dict[Tuple[int, str, int], List[Tuple[int, bool]]] = {}
        for op in ir.ops.values():
            reads, writes = _accesses(ir, op)
            for lst, is_w in ((reads, False), (writes, True)):
                for dev, buf, off, size in lst:
                    for u in range(off, off + size):
                        touched.setdefault((dev, buf, u), []).append((op.op_id, is_w))
        reported = set()
        for (dev, buf, u), lst in touched.items():
            for i in range(len(lst)):
                a, aw = lst[i]
                for j in range(i + 1, len(lst)):
                    b, bw = lst[j]
                    if a == b or not (aw or bw):
                        continue
                    ordered = (anc[b] >> index[a]) & 1 or (anc[a] >> index[b]) & 1
                    if not ordered and (a, b) not in reported:
                        reported.add((a, b))
                        errors.append(f"race: ops {a} and {b} touch {buf!r}@{dev} unit {u} "
                                      f"({'write' if aw else 'read'}/{'write' if bw else 'read'}) with no ordering")
            if len(errors) > 32:
                break

    # ---- repeated launches ----------------------------------------------------------------------
    if check_relaunch and not errors:
        for s_, r_ in relaunch_hazards(ir)[:8]:
            errors.append(f"relaunch: rank {s_} writes into rank {r_}'s workspace but waits for nothing from rank {r_}: "
                          f"launched repeatedly it can overwrite data that rank {r_} has not taken yet "
                          f"(end with an acknowledgement: NOTIFY from {r_}, GET_NOTIFIED on {s_})")

    return Report(not errors, errors, len(ir.ops), ir.num_steps(), ir.op_dag.critical_path(), traffic)


def port_load(ir: CollectiveIR) -> Dict[int, Tuple[int, int]]:
    """(egress, ingress) units per device: on NVSwitch the per-GPU port, not the pair, limits."""
    rep = verify(ir, check_races=False, check_annotations=False)
    out: Dict[int, List[int]] = {d: [0, 0] for d in ir.devices}
    for (a, b), u in rep.bytes_moved_units.items():
        out[a][0] += u
        out[b][1] += u
    return {d: (v[0], v[1]) for d, v in out.items()}
