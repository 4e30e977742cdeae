"""Lower a ``CollectiveIR`` DAG to per-(rank, channel) instruction streams.

This is the step the reference leaves between ``CollectiveIR`` (pccl/lang/chunk.py:57-135) and
``Engine::regOp(name, file)`` (csrc/engine.cc:102-104, empty body): the DAG becomes what an
executor can run without a scheduler.  The reference's runtime layout is a dependency-counted
graph with ready queues between executor kinds (include/base/operator.h:7-38); on a GPU that
costs a global atomic and a queue round-trip per op, so here dependencies are resolved at
lowering time instead:

* every op goes to the stream of (its executor rank, its channel), streams keep topological order;
* a dependency inside one stream is program order;
* a dependency between streams becomes a ``NOTIFY`` (after the producer) and a ``WAIT`` (before
  the consumer) on a counting signal slot owned by the consumer's rank.  Slots count up forever:
  launch ``e`` of a program expects ``e * notifies_per_launch + k``, so nothing is ever reset and
  a stale flag cannot satisfy a later wait;
* a ``BARRIER`` op uses one slot per channel that all ranks increment on all ranks.

Instruction = [opcode, src_rank, src_buf, src_off, dst_rank, dst_buf, dst_off, size, slot, value]
with offsets and sizes in units (the engine scales them to bytes for the message at hand).
"""
from __future__ import annotations

from typing import Any, Dict, List, Tuple

from .ir import BUFFER_KINDS, CollectiveIR, PrimitiveOpType as T

OPCODES = {"NOP": 0, "COPY": 1, "REDUCE": 2, "NOTIFY": 3, "WAIT": 4,
           "MM_LD_REDUCE": 5, "MM_ST": 6, "BARRIER": 7}
BUF_ID = {b: i for i, b in enumerate(BUFFER_KINDS)}


class LoweringError(Exception):
    pass


def lower(ir: CollectiveIR) -> Dict[str, Any]:
    order = ir.get_operation_sequence()
    if not order and ir.ops:
        raise LoweringError("op DAG has a cycle")
    ranks = sorted(ir.devices)
    if ranks != list(range(len(ranks))):
        raise LoweringError("device ids must be 0..n-1 to map onto ranks")
    n = len(ranks)
    C = ir.num_channels()
    anc = ir.op_dag.reachability()
    index = anc["__index__"]

    def stream_of(op) -> Tuple[int, int]:
        return (op.executor, op.channel)

    # barrier groups: k-th BARRIER op of a (rank, channel) belongs to group (channel, k)
    bar_group: Dict[int, Tuple[int, int]] = {}
    bar_of: Dict[Tuple[int, int, int], int] = {}    # (rank, channel, k) -> op id
    seen: Dict[Tuple[int, int], int] = {}
    for op in order:
        if op.op_type == T.BARRIER:
            k = seen.get(stream_of(op), 0) + 1
            seen[stream_of(op)] = k
            bar_group[op.op_id] = (op.channel, k)
            bar_of[(op.executor, op.channel, k)] = op.op_id
    for (ch, k) in set(bar_group.values()):
        for r in ranks:
            if (r, ch, k) not in bar_of:
                raise LoweringError(f"barrier {k} of channel {ch} is missing on rank {r}")

    streams: Dict[Tuple[int, int], List[list]] = {(r, c): [] for r in ranks for c in range(C)}
    slot_ids: Dict[Tuple[Tuple[int, int], Tuple[int, int]], int] = {}
    slot_counts: List[int] = []
    notified: Dict[Tuple[int, int], int] = {}        # (producer op, slot) -> ordinal
    # barrier slots first: one per channel
    bar_slot = {}
    for c in range(C):
        bar_slot[c] = len(slot_counts)
        slot_counts.append(0)
    for (ch, k) in bar_group.values():
        slot_counts[bar_slot[ch]] = max(slot_counts[bar_slot[ch]], k)

    # a producer's NOTIFY must directly follow it in its stream; since streams are appended in
    # topological order and the consumer comes later, we append the NOTIFY lazily at the
    # position right after the producer by recording insert points.
    emitted_at: Dict[int, Tuple[Tuple[int, int], int]] = {}   # op id -> (stream, index after op)
    pending_notifies: Dict[Tuple[int, int], List[Tuple[int, list]]] = {k: [] for k in streams}
    wait_fixups: List[Tuple[list, int, List[int]]] = []

    def chunk_fields(c):
        return [c.cur_device_id, BUF_ID["input" if (ir.in_place and c.buffer == "output") else c.buffer],
                c.offset, c.data_size]

    for op in order:
        me = stream_of(op)
        if me not in streams:
            raise LoweringError(f"op {op.op_id}: executor/channel {me} out of range")
        waits: Dict[int, List[int]] = {}
        for d in op.dependencies:
            dep = ir.ops[d]
            prod = stream_of(dep)
            if prod == me:
                continue
            if dep.op_type == T.BARRIER and dep.executor != op.executor:
                # ordering comes from this rank's own arrival at the same barrier
                mine = bar_of.get((op.executor, dep.channel, bar_group[d][1]))
                if mine is None or not ((anc[op.op_id] >> index[mine]) & 1 or mine == op.op_id):
                    raise LoweringError(f"op {op.op_id} depends on rank {dep.executor}'s barrier "
                                        f"without following its own")
                continue
            if op.op_type == T.BARRIER and dep.executor != op.executor:
                theirs = bar_of[(dep.executor, op.channel, bar_group[op.op_id][1])]
                if (anc[theirs] >> index[d]) & 1:
                    continue    # the peer arrives at this barrier only after dep
            key = (prod, me)
            if key not in slot_ids:
                slot_ids[key] = len(slot_counts)
                slot_counts.append(0)
            slot = slot_ids[key]
            notified.setdefault((d, slot), 0)
            waits.setdefault(slot, []).append(d)
        for slot, deps_ in sorted(waits.items()):
            ins = [OPCODES["WAIT"], 0, 0, 0, op.executor, 0, 0, 0, slot, 0]
            wait_fixups.append((ins, slot, deps_))
            streams[me].append(ins)
        t = op.op_type
        if t in (T.COPY, T.REDUCE, T.MM_LD_REDUCE, T.MM_ST):
            s, d_ = chunk_fields(op.src_chunk), chunk_fields(op.tgt_chunk)
            if s[3] != d_[3]:
                raise LoweringError(f"op {op.op_id}: size mismatch")
            streams[me].append([OPCODES[t.name], s[0], s[1], s[2], d_[0], d_[1], d_[2], s[3], 0, 0])
        elif t == T.BARRIER:
            ch, k = bar_group[op.op_id]
            streams[me].append([OPCODES["BARRIER"], 0, 0, 0, 0, 0, 0, 0, bar_slot[ch], k])
        else:   # NOTIFY / GET_NOTIFIED written by the user: ordering nodes only
            streams[me].append([OPCODES["NOP"], 0, 0, 0, 0, 0, 0, 0, 0, 0])
        emitted_at[op.op_id] = (me, len(streams[me]))

    # Ordinals follow the producer's program order, so that the k-th NOTIFY executed on a slot
    # is the one a WAIT for value k stands for; then splice the NOTIFYs in right after their
    # producers (back to front keeps the recorded positions valid).
    by_slot: Dict[int, List[int]] = {}
    for (d, slot) in notified:
        by_slot.setdefault(slot, []).append(d)
    prod_of_slot = {v: k[0] for k, v in slot_ids.items()}
    cons_of_slot = {v: k[1][0] for k, v in slot_ids.items()}
    for slot, ds in by_slot.items():
        ds.sort(key=lambda d: emitted_at[d][1])
        for k, d in enumerate(ds, 1):
            notified[(d, slot)] = k
            dep = ir.ops[d]
            cons_rank = cons_of_slot[slot]
            ins = [OPCODES["NOTIFY"], dep.executor, 0, 0, cons_rank, 0, 0, 0, slot, k]
            pending_notifies[prod_of_slot[slot]].append((emitted_at[d][1], ins))
        slot_counts[slot] = len(ds)
    for ins, slot, deps_ in wait_fixups:
        ins[9] = max(notified[(d, slot)] for d in deps_)
    for key, lst in pending_notifies.items():
        for pos, ins in sorted(lst, key=lambda x: -x[0]):
            streams[key].insert(pos, ins)
    for key in streams:
        streams[key] = [i for i in streams[key] if i[0] != OPCODES["NOP"]]

    programs = [[streams[(r, c)] for c in range(C)] for r in ranks]
    return {"num_ranks": n, "num_channels": C, "num_slots": len(slot_counts),
            "slot_counts": slot_counts, "programs": programs}


def to_schedule(ir: CollectiveIR) -> Dict[str, Any]:
    """Full schedule document: the IR plus its lowered programs (what ``regOp`` loads)."""
    d = ir.to_dict()
    d["lowered"] = lower(ir)
    return d


def check_lowered_deadlock_free(low: Dict[str, Any]) -> bool:
    """Simulate the streams with counting signals; True iff every stream runs to completion."""
    import copy
    low = copy.deepcopy(low)
    n, C = low["num_ranks"], low["num_channels"]
    pc = {(r, c): 0 for r in range(n) for c in range(C)}
    sig = [[0] * low["num_slots"] for _ in range(n)]
    progs = low["programs"]
    progress = True
    while progress:
        progress = False
        for (r, c), i in list(pc.items()):
            prog = progs[r][c]
            while i < len(prog):
                ins = prog[i]
                opc, slot, val = ins[0], ins[8], ins[9]
                if opc == OPCODES["WAIT"]:
                    if sig[r][slot] < val:
                        break
                elif opc == OPCODES["NOTIFY"]:
                    sig[ins[4]][slot] += 1
                elif opc == OPCODES["BARRIER"]:
                    if ins[7] == 0:          # not yet arrived: arrive, mark with size=1
                        for p in range(n):
                            sig[p][slot] += 1
                        ins = list(ins)
                        ins[7] = 1
                        prog[i] = ins
                        progress = True
                    if sig[r][slot] < n * val:
                        break
                    ins = list(prog[i]); ins[7] = 0; prog[i] = ins
                i += 1
                progress = True
            pc[(r, c)] = i
    return all(pc[(r, c)] == len(progs[r][c]) for r in range(n) for c in range(C))
