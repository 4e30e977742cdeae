"""Library of collective programs written in the IR.

The reference ships no program at all (example/collective/allreduce.py is empty); these are the
programs its vocabulary (pccl/lang/chunk.py:6-55) was evidently meant to express.  Each generator
returns a ``CollectiveIR`` whose pre/post-conditions the symbolic verifier can check and whose
JSON the CPU executor and the GPU interpreter kernel both run.

Conventions
-----------
* Remote ranks may only touch the ``scratch`` buffer (the engine's symmetric workspace) unless
  ``direct=True``, which states that the user's input/output tensors were themselves allocated
  from the symmetric heap and may be read or written by peers.
* ``channels`` splits every chunk ``channels`` ways; one channel = one executor worker (one CTA
  group on the GPU, one thread on the CPU).
* On NVSwitch every pair of GPUs has the same bandwidth and the limit is each GPU's port, so the
  one-step "direct" forms are the bandwidth-optimal ones; rings are kept for link-limited
  topologies, for the CPU/TCP transport and as verifier test material.
"""
from __future__ import annotations

from typing import Optional

from .ir import Chunk, CollectiveIR, Device, DeviceType, PrimitiveOpType


def _new(name: str, collective: str, n: int, units: int, buffers, device_type=DeviceType.CUDA,
         redop: str = "sum", in_place: bool = False, block_units: Optional[int] = None) -> CollectiveIR:
    """``block_units``: a buffer is a run of blocks of that many units, and a block is what maps
    onto an exact byte count at run time (a shard for gather/scatter/all-to-all, the whole vector
    for all-reduce); every buffer size is a multiple of it."""
    ir = CollectiveIR(name, collective, units, redop, buffers, in_place)
    ir.attrs["block_units"] = units if block_units is None else block_units
    for r in range(n):
        ir.add_device(Device(r, device_type))
    ir.fully_connect()
    ir.attrs["world_size"] = n
    return ir


def _all(n: int):
    return set(range(n))


# ---------------------------------------------------------------------------------------------
# pre/post-condition builders
# ---------------------------------------------------------------------------------------------
def allreduce_conditions(ir: CollectiveIR, n: int, units: int, out_buf: str = "output") -> None:
    ir.set_precondition([Chunk({r}, r, units, 0, "input") for r in range(n)])
    ir.set_postcondition([Chunk(_all(n), r, units, 0, out_buf) for r in range(n)])


def reduce_scatter_conditions(ir: CollectiveIR, n: int, shard: int) -> None:
    ir.set_precondition([Chunk({r}, r, n * shard, 0, "input") for r in range(n)])
    ir.set_postcondition([Chunk(_all(n), r, shard, 0, "output", origin=r * shard) for r in range(n)])


def allgather_conditions(ir: CollectiveIR, n: int, shard: int) -> None:
    # origin encodes (source rank, unit) as rank*shard + unit
    ir.set_precondition([Chunk({r}, r, shard, 0, "input", origin=r * shard) for r in range(n)])
    post = []
    for r in range(n):
        for s in range(n):
            post.append(Chunk({s}, r, shard, s * shard, "output", origin=s * shard))
    ir.set_postcondition(post)


def alltoall_conditions(ir: CollectiveIR, n: int, blk: int) -> None:
    # input unit u on rank r has origin r*(n*blk)+u ; output block s on rank d holds input block d of rank s
    U = n * blk
    ir.set_precondition([Chunk({r}, r, U, 0, "input", origin=r * U) for r in range(n)])
    post = []
    for d in range(n):
        for s in range(n):
            post.append(Chunk({s}, d, blk, s * blk, "output", origin=s * U + d * blk))
    ir.set_postcondition(post)


# ---------------------------------------------------------------------------------------------
# ring algorithms
# ---------------------------------------------------------------------------------------------
def ring_allreduce(n: int, channels: int = 1, device_type=DeviceType.CUDA, redop: str = "sum",
                   direct: bool = False) -> CollectiveIR:
    """Ring reduce-scatter followed by ring all-gather: 2(n-1) steps, n*channels chunks."""
    U = n * channels
    ir = _new(f"ring_allreduce_n{n}_c{channels}", "allreduce", n, U,
              {"input": U, "output": U, "scratch": U}, device_type, redop)
    allreduce_conditions(ir, n, U)
    if n == 1:
        ir.copy(Chunk({0}, 0, U, 0, "input"), Chunk({0}, 0, U, 0, "output"), step=0)
        return ir
    for ch in range(channels):
        unit = lambda c: c * channels + ch  # noqa: E731  chunk c of this channel
        # stage the input into the accumulator (output buffer)
        last = {}   # (rank, chunk) -> op id that last wrote output[chunk] on rank
        for r in range(n):
            for c in range(n):
                last[(r, c)] = ir.copy(Chunk({r}, r, 1, unit(c), "input"),
                                       Chunk({r}, r, 1, unit(c), "output"), step=0, channel=ch)
        # reduce-scatter: at step s rank r pushes chunk (r-s) to r+1, which folds it in
        for s in range(n - 1):
            new_last = {}
            for r in range(n):
                c, nxt = (r - s) % n, (r + 1) % n
                have = set(((r - k) % n) for k in range(s + 1))
                push = ir.copy(Chunk(have, r, 1, unit(c), "output"),
                               Chunk(have, nxt, 1, unit(c), "scratch"),
                               deps=[last[(r, c)]], step=1 + 2 * s, channel=ch)
                red = ir.reduce(Chunk(have, nxt, 1, unit(c), "scratch"),
                                Chunk(have | {nxt}, nxt, 1, unit(c), "output"),
                                deps=[push, last[(nxt, c)]], step=2 + 2 * s, channel=ch)
                new_last[(nxt, c)] = red
            last.update(new_last)
        # all-gather: rank r now owns chunk (r+1); at step s it forwards chunk (r+1-s)
        base = 1 + 2 * (n - 1)
        for s in range(n - 1):
            new_last = {}
            for r in range(n):
                c, nxt = (r + 1 - s) % n, (r + 1) % n
                if direct:
                    new_last[(nxt, c)] = ir.copy(Chunk(_all(n), r, 1, unit(c), "output"),
                                                 Chunk(_all(n), nxt, 1, unit(c), "output"),
                                                 deps=[last[(r, c)], last[(nxt, c)]],
                                                 step=base + 2 * s, channel=ch)
                else:
                    push = ir.copy(Chunk(_all(n), r, 1, unit(c), "output"),
                                   Chunk(_all(n), nxt, 1, unit(c), "scratch"),
                                   deps=[last[(r, c)], last[(nxt, c)]], step=base + 2 * s, channel=ch)
                    new_last[(nxt, c)] = ir.copy(Chunk(_all(n), nxt, 1, unit(c), "scratch"),
                                                 Chunk(_all(n), nxt, 1, unit(c), "output"),
                                                 deps=[push, last[(nxt, c)]],
                                                 step=base + 1 + 2 * s, channel=ch)
            last.update(new_last)
    return ir


def ring_allgather(n: int, channels: int = 1, device_type=DeviceType.CUDA,
                   explicit_signals: bool = False, name: Optional[str] = None) -> CollectiveIR:
    """Ring all-gather; with ``explicit_signals`` the hand-off uses NOTIFY / GET_NOTIFIED ops
    written into the program (the double-buffered block rotation of ring attention)."""
    sh = channels
    ir = _new(name or f"ring_allgather_n{n}_c{channels}", "allgather", n, sh,
              {"input": sh, "output": n * sh, "scratch": n * sh}, device_type, block_units=sh)
    allgather_conditions(ir, n, sh)
    for ch in range(channels):
        last = {}
        for r in range(n):
            last[(r, r)] = ir.copy(Chunk({r}, r, 1, ch, "input", origin=r * sh + ch),
                                   Chunk({r}, r, 1, r * sh + ch, "output", origin=r * sh + ch),
                                   step=0, channel=ch)
        for s in range(n - 1):
            new_last = {}
            for r in range(n):
                c, nxt = (r - s) % n, (r + 1) % n
                org = c * sh + ch
                push = ir.copy(Chunk({c}, r, 1, org, "output", origin=org),
                               Chunk({c}, nxt, 1, org, "scratch", origin=org),
                               deps=[last[(r, c)]], step=1 + 2 * s, channel=ch)
                dep = push
                if explicit_signals:
                    nt = ir.notify(r, nxt, deps=[push], step=1 + 2 * s, channel=ch)
                    dep = ir.get_notified(r, nxt, deps=[nt], step=2 + 2 * s, channel=ch)
                new_last[(nxt, c)] = ir.copy(Chunk({c}, nxt, 1, org, "scratch", origin=org),
                                             Chunk({c}, nxt, 1, org, "output", origin=org),
                                             deps=[dep], step=2 + 2 * s, channel=ch)
            last.update(new_last)
    return ir


def ring_kv_rotation(n: int, channels: int = 1, device_type=DeviceType.CUDA) -> CollectiveIR:
    """Ring-attention / blockwise context parallelism: every rank's KV block visits every rank
    in ring order, one hop per step, hand-offs by explicit NOTIFY / GET_NOTIFIED.  After step s
    rank r holds the block of rank (r-s-1) mod n in ``output`` at that block's slot."""
    ir = ring_allgather(n, channels, device_type, explicit_signals=True,
                        name=f"ring_kv_rotation_n{n}_c{channels}")
    ir.attrs["use"] = "ring_attention_kv"
    return ir


# ---------------------------------------------------------------------------------------------
# direct (one hop through the switch) algorithms
# ---------------------------------------------------------------------------------------------
def direct_reduce_scatter(n: int, channels: int = 1, device_type=DeviceType.CUDA,
                          redop: str = "sum", direct: bool = False) -> CollectiveIR:
    """Every rank sends shard d to rank d in one step; d folds the n contributions.

    ``direct=True`` is the pull form for symmetric inputs: rank d reads its shard straight out of every peer's input and
    reduces in registers; no scratch traffic.  A barrier before the reads says that every input is complete, one after
    them that every peer has finished reading this rank's input (which the caller may then overwrite)."""
    sh = channels
    ir = _new(f"direct_reduce_scatter_n{n}_c{channels}{'_pull' if direct else ''}", "reduce_scatter",
              n, n * sh, {"input": n * sh, "output": sh, "scratch": 0 if direct else n * sh},
              device_type, redop, block_units=sh)
    reduce_scatter_conditions(ir, n, sh)
    for ch in range(channels):
        bars = ([ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r, metadata={"step": 0, "channel": ch})
                 for r in range(n)] if direct else [])
        last = []
        for d in range(n):
            # (pull form: behind the barrier, so that the executor can take "copy, reduce, reduce, ..." as one pass)
            acc = ir.copy(Chunk({d}, d, 1, d * sh + ch, "input"),
                          Chunk({d}, d, 1, ch, "output", origin=d * sh + ch), deps=bars, step=0, channel=ch)
            have = {d}
            for k in range(1, n):
                r = (d + k) % n     # rotate so that the n ranks never all target one peer
                if direct:
                    acc = ir.reduce(Chunk({r}, r, 1, d * sh + ch, "input"),
                                    Chunk(have | {r}, d, 1, ch, "output", origin=d * sh + ch),
                                    deps=[acc] + (bars if k == 1 else []), step=k, channel=ch, executor=d)
                else:
                    push = ir.copy(Chunk({r}, r, 1, d * sh + ch, "input"),
                                   Chunk({r}, d, 1, r * sh + ch, "scratch", origin=d * sh + ch),
                                   step=0, channel=ch)
                    acc = ir.reduce(Chunk({r}, d, 1, r * sh + ch, "scratch", origin=d * sh + ch),
                                    Chunk(have | {r}, d, 1, ch, "output", origin=d * sh + ch),
                                    deps=[acc, push], step=k, channel=ch)
                have = have | {r}
            last.append(acc)
        if direct:
            for r in range(n):
                ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r, last, {"step": n, "channel": ch})
    return ir


def direct_allgather(n: int, channels: int = 1, device_type=DeviceType.CUDA,
                     direct: bool = False) -> CollectiveIR:
    """``direct=True``: for symmetric outputs every rank stores its shard straight into each peer's output, between a
    barrier that says the outputs may be written and one that says every store has landed."""
    sh = channels
    ir = _new(f"direct_allgather_n{n}_c{channels}{'_sym' if direct else ''}", "allgather", n, sh,
              {"input": sh, "output": n * sh, "scratch": 0 if direct else n * sh}, device_type,
              block_units=sh)
    allgather_conditions(ir, n, sh)
    for ch in range(channels):
        bars = ([ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r, metadata={"step": 0, "channel": ch})
                 for r in range(n)] if direct else [])
        stores = []
        for r in range(n):
            org = r * sh + ch
            src = Chunk({r}, r, 1, ch, "input", origin=org)
            ir.copy(src, Chunk({r}, r, 1, org, "output", origin=org), step=0, channel=ch)
            for k in range(1, n):
                d = (r + k) % n
                if direct:
                    stores.append(ir.copy(src, Chunk({r}, d, 1, org, "output", origin=org), deps=bars, step=1, channel=ch))
                else:
                    push = ir.copy(src, Chunk({r}, d, 1, org, "scratch", origin=org), step=0, channel=ch)
                    ir.copy(Chunk({r}, d, 1, org, "scratch", origin=org),
                            Chunk({r}, d, 1, org, "output", origin=org), deps=[push], step=1, channel=ch)
        if direct:
            for r in range(n):
                ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r, stores, {"step": 2, "channel": ch})
    return ir


def direct_allreduce(n: int, channels: int = 1, device_type=DeviceType.CUDA, redop: str = "sum",
                     direct: bool = False) -> CollectiveIR:
    """Two-shot: direct reduce-scatter into the output shard, then direct all-gather of shards.

    Scratch is n+1 images of the vector: image r receives rank r's contribution (each unit keeps its
    position inside the image, so source and target slices have the same length whatever the
    message size), image n receives the gathered results.

    ``direct=True`` is the form for symmetric inputs and outputs, with no scratch at all: rank d reduces its slice
    straight out of every peer's input into its own output and stores the result into every peer's output, between an
    entry barrier (inputs complete, outputs free) and an exit barrier (every store has landed, every read is over)."""
    sh = channels
    U = n * sh
    ir = _new(f"direct_allreduce_n{n}_c{channels}{'_pull' if direct else ''}", "allreduce", n, U,
              {"input": U, "output": U, "scratch": 0 if direct else (n + 1) * U}, device_type, redop)
    allreduce_conditions(ir, n, U)
    for ch in range(channels):
        bars = ([ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r, metadata={"step": 0, "channel": ch})
                 for r in range(n)] if direct else [])
        stores = []
        for d in range(n):
            u = d * sh + ch
            acc = ir.copy(Chunk({d}, d, 1, u, "input"), Chunk({d}, d, 1, u, "output"), deps=bars, step=0, channel=ch)
            have = {d}
            for k in range(1, n):
                r = (d + k) % n
                if direct:
                    acc = ir.reduce(Chunk({r}, r, 1, u, "input"), Chunk(have | {r}, d, 1, u, "output"),
                                    deps=[acc] + (bars if k == 1 else []), step=k, channel=ch, executor=d)
                else:
                    push = ir.copy(Chunk({r}, r, 1, u, "input"),
                                   Chunk({r}, d, 1, r * U + u, "scratch", origin=u), step=0, channel=ch)
                    acc = ir.reduce(Chunk({r}, d, 1, r * U + u, "scratch", origin=u),
                                    Chunk(have | {r}, d, 1, u, "output"), deps=[acc, push], step=k, channel=ch)
                have = have | {r}
            for k in range(1, n):
                t = (d + k) % n
                if direct:
                    stores.append(ir.copy(Chunk(_all(n), d, 1, u, "output"), Chunk(_all(n), t, 1, u, "output"),
                                          deps=[acc], step=n, channel=ch))
                else:
                    push = ir.copy(Chunk(_all(n), d, 1, u, "output"),
                                   Chunk(_all(n), t, 1, n * U + u, "scratch", origin=u),
                                   deps=[acc], step=n, channel=ch)
                    ir.copy(Chunk(_all(n), t, 1, n * U + u, "scratch", origin=u),
                            Chunk(_all(n), t, 1, u, "output"), deps=[push], step=n + 1, channel=ch)
        if direct:
            for r in range(n):
                ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r, stores, {"step": n + 1, "channel": ch})
    return ir


def oneshot_allreduce(n: int, channels: int = 1, device_type=DeviceType.CUDA,
                      redop: str = "sum") -> CollectiveIR:
    """Latency-optimal small-message form: everyone sends everything, everyone reduces."""
    U = channels
    ir = _new(f"oneshot_allreduce_n{n}_c{channels}", "allreduce", n, U,
              {"input": U, "output": U, "scratch": n * U}, device_type, redop)
    allreduce_conditions(ir, n, U)
    for ch in range(channels):
        for d in range(n):
            acc = ir.copy(Chunk({d}, d, 1, ch, "input"), Chunk({d}, d, 1, ch, "output"), step=0, channel=ch)
            have = {d}
            for k in range(1, n):
                r = (d + k) % n
                push = ir.copy(Chunk({r}, r, 1, ch, "input"),
                               Chunk({r}, d, 1, r * U + ch, "scratch", origin=ch), step=0, channel=ch)
                acc = ir.reduce(Chunk({r}, d, 1, r * U + ch, "scratch", origin=ch),
                                Chunk(have | {r}, d, 1, ch, "output"), deps=[acc, push], step=k, channel=ch)
                have = have | {r}
    return ir


def tree_allreduce(n: int, channels: int = 1, device_type=DeviceType.CUDA,
                   redop: str = "sum") -> CollectiveIR:
    """Binomial-tree reduce to rank 0 followed by binomial broadcast (log2 n steps each)."""
    U = channels
    ir = _new(f"tree_allreduce_n{n}_c{channels}", "allreduce", n, U,
              {"input": U, "output": U, "scratch": 2 * U * max(1, n.bit_length())}, device_type, redop)
    allreduce_conditions(ir, n, U)
    for ch in range(channels):
        last, have = {}, {}
        for r in range(n):
            last[r] = ir.copy(Chunk({r}, r, 1, ch, "input"), Chunk({r}, r, 1, ch, "output"), step=0, channel=ch)
            have[r] = {r}
        lvl, dist, step = 0, 1, 1
        while dist < n:
            for r in range(0, n, 2 * dist):
                s = r + dist
                if s >= n:
                    continue
                slot = lvl * U + ch
                push = ir.copy(Chunk(have[s], s, 1, ch, "output"),
                               Chunk(have[s], r, 1, slot, "scratch", origin=ch),
                               deps=[last[s]], step=step, channel=ch)
                last[r] = ir.reduce(Chunk(have[s], r, 1, slot, "scratch", origin=ch),
                                    Chunk(have[r] | have[s], r, 1, ch, "output"),
                                    deps=[push, last[r]], step=step + 1, channel=ch)
                have[r] = have[r] | have[s]
            dist *= 2
            lvl += 1
            step += 2
        nl = lvl
        dist //= 2
        while dist >= 1:
            lvl -= 1
            for r in range(0, n, 2 * dist):
                s = r + dist
                if s >= n:
                    continue
                slot = (nl + lvl) * U + ch
                push = ir.copy(Chunk(_all(n), r, 1, ch, "output"),
                               Chunk(_all(n), s, 1, slot, "scratch", origin=ch),
                               deps=[last[r], last[s]], step=step, channel=ch)
                last[s] = ir.copy(Chunk(_all(n), s, 1, slot, "scratch", origin=ch),
                                  Chunk(_all(n), s, 1, ch, "output"), deps=[push], step=step + 1, channel=ch)
            dist //= 2
            step += 2
    return ir


def alltoall(n: int, channels: int = 1, device_type=DeviceType.CUDA, direct: bool = False,
             name: Optional[str] = None) -> CollectiveIR:
    """Block d of rank s's input becomes block s of rank d's output."""
    blk = channels
    U = n * blk
    ir = _new(name or f"alltoall_n{n}_c{channels}", "alltoall", n, U,
              {"input": U, "output": U, "scratch": 0 if direct else U}, device_type, block_units=blk)
    alltoall_conditions(ir, n, blk)
    for ch in range(channels):
        for s in range(n):
            for k in range(n):
                d = (s + k) % n
                org = s * U + d * blk + ch
                src = Chunk({s}, s, 1, d * blk + ch, "input", origin=org)
                dst = Chunk({s}, d, 1, s * blk + ch, "output", origin=org)
                if d == s or direct:
                    ir.copy(src, dst, step=0, channel=ch)
                else:
                    mid = Chunk({s}, d, 1, s * blk + ch, "scratch", origin=org)
                    push = ir.copy(src, mid, step=0, channel=ch)
                    ir.copy(mid, dst, deps=[push], step=1, channel=ch)
    return ir


def ulysses_alltoall(n: int, channels: int = 1, device_type=DeviceType.CUDA) -> CollectiveIR:
    """DeepSpeed-Ulysses sequence<->head exchange: an all-to-all whose block d of rank s is the
    slice (sequence shard s, head group d); after it rank d holds every sequence shard of its
    head group."""
    ir = alltoall(n, channels, device_type, name=f"ulysses_alltoall_n{n}_c{channels}")
    ir.attrs["use"] = "ulysses_seq_to_head"
    return ir


# ---------------------------------------------------------------------------------------------
# more ring / recursive algorithms (latency-optimal shapes for switchless or power-of-two worlds)
# ---------------------------------------------------------------------------------------------
def ring_reduce_scatter(n: int, channels: int = 1, device_type=DeviceType.CUDA, redop: str = "sum") -> CollectiveIR:
    """Ring reduce-scatter: shard c starts on rank c+1 and travels the ring, every rank folding its own contribution
    in, until it reaches its owner c after n-1 steps."""
    sh = channels
    ir = _new(f"ring_reduce_scatter_n{n}_c{channels}", "reduce_scatter", n, n * sh,
              {"input": n * sh, "output": sh, "scratch": 2 * n * sh}, device_type, redop, block_units=sh)
    reduce_scatter_conditions(ir, n, sh)
    for ch in range(channels):
        # running partial of shard c on rank r: the output when r owns c, else scratch unit c*sh+ch
        def acc(r, c, ranks):
            if r == c:
                return Chunk(set(ranks), r, 1, ch, "output", origin=c * sh + ch)
            return Chunk(set(ranks), r, 1, c * sh + ch, "scratch", origin=c * sh + ch)
        last = {}
        for r in range(n):
            for c in range(n):
                last[(r, c)] = ir.copy(Chunk({r}, r, 1, c * sh + ch, "input"), acc(r, c, {r}), step=0, channel=ch)
        for s in range(n - 1):
            new_last = {}
            for r in range(n):
                c, nxt = (r - 1 - s) % n, (r + 1) % n
                have = {(r - k) % n for k in range(s + 1)}
                slot = Chunk(set(have), nxt, 1, (n + c) * sh + ch, "scratch", origin=c * sh + ch)
                push = ir.copy(acc(r, c, have), slot, deps=[last[(r, c)]], step=1 + 2 * s, channel=ch)
                new_last[(nxt, c)] = ir.reduce(slot, acc(nxt, c, have | {nxt}), deps=[push, last[(nxt, c)]], step=2 + 2 * s, channel=ch)
            last.update(new_last)
    return ir


def _log2_exact(n: int) -> int:
    k = n.bit_length() - 1
    if n < 1 or (1 << k) != n:
        raise ValueError(f"this algorithm needs a power-of-two world, not {n}")
    return k


def recursive_doubling_allgather(n: int, channels: int = 1, device_type=DeviceType.CUDA) -> CollectiveIR:
    """log2(n) exchange steps: at step k rank r swaps everything it holds (2^k blocks) with rank r xor 2^k."""
    steps = _log2_exact(n)
    sh = channels
    ir = _new(f"recursive_doubling_allgather_n{n}_c{channels}", "allgather", n, sh,
              {"input": sh, "output": n * sh, "scratch": n * sh}, device_type, block_units=sh)
    allgather_conditions(ir, n, sh)
    for ch in range(channels):
        last = {}
        held = {r: [r] for r in range(n)}
        for r in range(n):
            org = r * sh + ch
            last[(r, r)] = ir.copy(Chunk({r}, r, 1, ch, "input", origin=org), Chunk({r}, r, 1, org, "output", origin=org), step=0, channel=ch)
        for k in range(steps):
            new_last, new_held = {}, {r: list(held[r]) for r in range(n)}
            for r in range(n):
                p = r ^ (1 << k)
                for b in held[r]:
                    org = b * sh + ch
                    push = ir.copy(Chunk({b}, r, 1, org, "output", origin=org), Chunk({b}, p, 1, org, "scratch", origin=org),
                                   deps=[last[(r, b)]], step=1 + 2 * k, channel=ch)
                    new_last[(p, b)] = ir.copy(Chunk({b}, p, 1, org, "scratch", origin=org), Chunk({b}, p, 1, org, "output", origin=org),
                                               deps=[push], step=2 + 2 * k, channel=ch)
                    new_held[p].append(b)
            last.update(new_last)
            held = new_held
    return ir


def halving_doubling_allreduce(n: int, channels: int = 1, device_type=DeviceType.CUDA, redop: str = "sum") -> CollectiveIR:
    """Recursive halving reduce-scatter followed by recursive doubling all-gather: 2 log2(n) steps, each rank
    moves (n-1)/n of the vector per phase -- the bandwidth of the ring at the latency of a tree."""
    steps = _log2_exact(n)
    U = n * channels
    ir = _new(f"halving_doubling_allreduce_n{n}_c{channels}", "allreduce", n, U,
              {"input": U, "output": U, "scratch": max(1, 2 * steps) * U}, device_type, redop)
    allreduce_conditions(ir, n, U)
    for ch in range(channels):
        unit = lambda c: c * channels + ch  # noqa: E731
        last = {}
        for r in range(n):
            for c in range(n):
                last[(r, c)] = ir.copy(Chunk({r}, r, 1, unit(c), "input"), Chunk({r}, r, 1, unit(c), "output"), step=0, channel=ch)
        lo = {r: 0 for r in range(n)}
        hi = {r: n for r in range(n)}
        have = {r: {r} for r in range(n)}
        # reduce-scatter by halving: keep the half of the current range on your side of the split, send the other
        for k in range(steps):
            d = n >> (k + 1)
            new_last, new_have = {}, {}
            ranges = {}
            for r in range(n):
                mid = (lo[r] + hi[r]) // 2
                ranges[r] = (lo[r], mid) if (r & d) == 0 else (mid, hi[r])
            for r in range(n):
                p = r ^ d
                send_lo, send_hi = ranges[p]            # the partner keeps this part of the (common) range
                for c in range(send_lo, send_hi):
                    slot = Chunk(set(have[r]), p, 1, k * U + unit(c), "scratch")
                    push = ir.copy(Chunk(set(have[r]), r, 1, unit(c), "output"), slot, deps=[last[(r, c)]], step=1 + 2 * k, channel=ch)
                    new_last[(p, c)] = ir.reduce(slot, Chunk(have[r] | have[p], p, 1, unit(c), "output"), deps=[push, last[(p, c)]],
                                                 step=2 + 2 * k, channel=ch)
                new_have[r] = have[r] | have[p]
            last.update(new_last)
            for r in range(n):
                lo[r], hi[r] = ranges[r]
            have = new_have
        # all-gather by doubling: the ranges merge back in the opposite order
        base = 1 + 2 * steps
        everyone = _all(n)
        for j, k in enumerate(reversed(range(steps))):
            d = n >> (k + 1)
            new_last = {}
            new_lo, new_hi = dict(lo), dict(hi)
            for r in range(n):
                p = r ^ d
                for c in range(lo[r], hi[r]):
                    slot = Chunk(set(everyone), p, 1, (steps + j) * U + unit(c), "scratch")
                    push = ir.copy(Chunk(set(everyone), r, 1, unit(c), "output"), slot, deps=[last[(r, c)], last[(p, c)]],
                                   step=base + 2 * j, channel=ch)
                    new_last[(p, c)] = ir.copy(slot, Chunk(set(everyone), p, 1, unit(c), "output"), deps=[push], step=base + 1 + 2 * j, channel=ch)
                new_lo[p], new_hi[p] = min(new_lo[p], lo[r]), max(new_hi[p], hi[r])
            last.update(new_last)
            lo, hi = new_lo, new_hi
    return ir


def hierarchical_allgather(n: int, channels: int = 1, device_type=DeviceType.CUDA, per_host: int = 2) -> CollectiveIR:
    """All-gather for hosts of ``per_host`` ranks: every rank first swaps its shard with the ranks of the same local
    index on the other hosts (the only traffic between hosts: each shard crosses once per remote host), then the
    ranks of a host hand one another everything they hold."""
    L = per_host
    if L < 1 or n % L:
        raise ValueError(f"hierarchical_allgather: {n} ranks do not split into hosts of {L}")
    H = n // L
    sh = channels
    ir = _new(f"hierarchical_allgather_n{n}_h{H}x{L}_c{channels}", "allgather", n, sh,
              {"input": sh, "output": n * sh, "scratch": n * sh}, device_type, block_units=sh)
    allgather_conditions(ir, n, sh)
    rank_of = lambda g, l: g * L + l  # noqa: E731
    for ch in range(channels):
        last = {}
        for r in range(n):
            org = r * sh + ch
            last[(r, r)] = ir.copy(Chunk({r}, r, 1, ch, "input", origin=org), Chunk({r}, r, 1, org, "output", origin=org), step=0, channel=ch)

        def hand_over(src, dst, b, step):
            org = b * sh + ch
            push = ir.copy(Chunk({b}, src, 1, org, "output", origin=org), Chunk({b}, dst, 1, org, "scratch", origin=org),
                           deps=[last[(src, b)]], step=step, channel=ch)
            return ir.copy(Chunk({b}, dst, 1, org, "scratch", origin=org), Chunk({b}, dst, 1, org, "output", origin=org),
                           deps=[push], step=step + 1, channel=ch)
        new_last = {}
        for l in range(L):                       # between hosts, same local index
            for g in range(H):
                for gp in range(H):
                    if gp != g:
                        new_last[(rank_of(gp, l), rank_of(g, l))] = hand_over(rank_of(g, l), rank_of(gp, l), rank_of(g, l), 1)
        last.update(new_last)
        new_last = {}
        for g in range(H):                       # inside a host: rank (g, l) holds the shards of local index l from every host
            for l in range(L):
                for lp in range(L):
                    if lp == l:
                        continue
                    for gg in range(H):
                        new_last[(rank_of(g, lp), rank_of(gg, l))] = hand_over(rank_of(g, l), rank_of(g, lp), rank_of(gg, l), 3)
        last.update(new_last)
    return ir


def hierarchical_allreduce(n: int, channels: int = 1, device_type=DeviceType.CUDA, redop: str = "sum",
                           per_host: int = 2) -> CollectiveIR:
    """All-reduce for ``n / per_host`` hosts of ``per_host`` ranks (rank r on host r // per_host): reduce-scatter inside
    each host, all-reduce of every part among the ranks with the same local index (one per host), all-gather inside
    each host.  Only the middle phase crosses hosts, and it moves 2 (hosts-1)/n of the vector per rank."""
    L = per_host
    if L < 1 or n % L:
        raise ValueError(f"hierarchical_allreduce: {n} ranks do not split into hosts of {L}")
    H = n // L
    U = n * channels
    ir = _new(f"hierarchical_allreduce_n{n}_h{H}x{L}_c{channels}", "allreduce", n, U,
              {"input": U, "output": U, "scratch": (L + H + 1) * U}, device_type, redop)
    allreduce_conditions(ir, n, U)
    rank_of = lambda g, l: g * L + l  # noqa: E731
    for ch in range(channels):
        unit = lambda c: c * channels + ch  # noqa: E731      chunk c = l * H + h: part l, sub-chunk h
        last, have = {}, {}
        for r in range(n):
            for c in range(n):
                last[(r, c)] = ir.copy(Chunk({r}, r, 1, unit(c), "input"), Chunk({r}, r, 1, unit(c), "output"), step=0, channel=ch)
                have[(r, c)] = {r}
        # A: inside a host, local rank l collects part l
        new_last, new_have = {}, {}
        for g in range(H):
            for l in range(L):
                owner = rank_of(g, l)
                for lp in range(L):
                    if lp == l:
                        continue
                    src = rank_of(g, lp)
                    for h in range(H):
                        c = l * H + h
                        slot = Chunk({src}, owner, 1, (lp * n + c) * channels + ch, "scratch")
                        push = ir.copy(Chunk({src}, src, 1, unit(c), "output"), slot, deps=[last[(src, c)]], step=1, channel=ch)
                        got = new_have.get((owner, c), {owner}) | {src}
                        new_last[(owner, c)] = ir.reduce(slot, Chunk(set(got), owner, 1, unit(c), "output"),
                                                         deps=[push, new_last.get((owner, c), last[(owner, c)])], step=2, channel=ch)
                        new_have[(owner, c)] = got
        last.update(new_last)
        have.update(new_have)
        # B1: among the hosts, rank (g, l) collects sub-chunk g of part l
        new_last, new_have = {}, {}
        for l in range(L):
            for g in range(H):
                owner, c = rank_of(g, l), l * H + g
                for gp in range(H):
                    if gp == g:
                        continue
                    src = rank_of(gp, l)
                    slot = Chunk(set(have[(src, c)]), owner, 1, ((L + gp) * n + c) * channels + ch, "scratch")
                    push = ir.copy(Chunk(set(have[(src, c)]), src, 1, unit(c), "output"), slot, deps=[last[(src, c)]], step=3, channel=ch)
                    got = new_have.get((owner, c), have[(owner, c)]) | have[(src, c)]
                    new_last[(owner, c)] = ir.reduce(slot, Chunk(set(got), owner, 1, unit(c), "output"),
                                                     deps=[push, new_last.get((owner, c), last[(owner, c)])], step=4, channel=ch)
                    new_have[(owner, c)] = got
        last.update(new_last)
        have.update(new_have)
        everyone = _all(n)
        gather_slot = lambda c: ((L + H) * n + c) * channels + ch  # noqa: E731

        def hand_over(src, dst, c, step):
            slot = Chunk(set(everyone), dst, 1, gather_slot(c), "scratch")
            push = ir.copy(Chunk(set(everyone), src, 1, unit(c), "output"), slot, deps=[last[(src, c)], last[(dst, c)]], step=step, channel=ch)
            return ir.copy(slot, Chunk(set(everyone), dst, 1, unit(c), "output"), deps=[push], step=step + 1, channel=ch)
        # B2: the finished sub-chunks go back to the other hosts
        new_last = {}
        for l in range(L):
            for g in range(H):
                c = l * H + g
                for gp in range(H):
                    if gp != g:
                        new_last[(rank_of(gp, l), c)] = hand_over(rank_of(g, l), rank_of(gp, l), c, 5)
        last.update(new_last)
        # C: inside a host, every rank hands its finished part to its neighbours
        new_last = {}
        for g in range(H):
            for l in range(L):
                for lp in range(L):
                    if lp == l:
                        continue
                    for h in range(H):
                        c = l * H + h
                        new_last[(rank_of(g, lp), c)] = hand_over(rank_of(g, l), rank_of(g, lp), c, 7)
        last.update(new_last)
    return ir


# ---------------------------------------------------------------------------------------------
# NVLS (in-switch) algorithms — GPU only, symmetric input/output bound to a multicast object
# ---------------------------------------------------------------------------------------------
def nvls_allreduce(n: int, channels: int = 1, redop: str = "sum") -> CollectiveIR:
    """Two-shot through the switch: rank r ld_reduce's slice r (the switch sums the n replicas)
    and multicast-stores the result into every replica of the output."""
    sh = channels
    U = n * sh
    ir = _new(f"nvls_allreduce_n{n}_c{channels}", "allreduce", n, U,
              {"input": U, "output": U, "scratch": 0}, DeviceType.CUDA, redop, in_place=True)
    ir.attrs["requires"] = "multicast"
    allreduce_conditions(ir, n, U)
    for ch in range(channels):
        bars = [ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r,
                                    metadata={"step": 0, "channel": ch}) for r in range(n)]
        sts = []
        for r in range(n):
            u = r * sh + ch
            ld = ir.create_operation(PrimitiveOpType.MM_LD_REDUCE, Chunk(_all(n), r, 1, u, "input"),
                                     Chunk(_all(n), r, 1, u, "output"), r, r, bars,
                                     {"step": 1, "channel": ch})
            sts.append(ir.create_operation(PrimitiveOpType.MM_ST, Chunk(_all(n), r, 1, u, "output"),
                                           Chunk(_all(n), r, 1, u, "output"), r, r, [ld],
                                           {"step": 2, "channel": ch}))
        for r in range(n):
            ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r, sts,
                                {"step": 3, "channel": ch})
    return ir


def nvls_reduce_scatter(n: int, channels: int = 1, redop: str = "sum") -> CollectiveIR:
    sh = channels
    ir = _new(f"nvls_reduce_scatter_n{n}_c{channels}", "reduce_scatter", n, n * sh,
              {"input": n * sh, "output": sh, "scratch": 0}, DeviceType.CUDA, redop, block_units=sh)
    ir.attrs["requires"] = "multicast"
    reduce_scatter_conditions(ir, n, sh)
    for ch in range(channels):
        bars = [ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r,
                                    metadata={"step": 0, "channel": ch}) for r in range(n)]
        lds = [ir.create_operation(PrimitiveOpType.MM_LD_REDUCE,
                                   Chunk(_all(n), r, 1, r * sh + ch, "input"),
                                   Chunk(_all(n), r, 1, ch, "output", origin=r * sh + ch), r, r, bars,
                                   {"step": 1, "channel": ch}) for r in range(n)]
        for r in range(n):
            ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r, lds, {"step": 2, "channel": ch})
    return ir


def nvls_allgather(n: int, channels: int = 1) -> CollectiveIR:
    sh = channels
    ir = _new(f"nvls_allgather_n{n}_c{channels}", "allgather", n, sh,
              {"input": sh, "output": n * sh, "scratch": 0}, DeviceType.CUDA, block_units=sh)
    ir.attrs["requires"] = "multicast"
    allgather_conditions(ir, n, sh)
    for ch in range(channels):
        bars = [ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r,
                                    metadata={"step": 0, "channel": ch}) for r in range(n)]
        sts = [ir.create_operation(PrimitiveOpType.MM_ST,
                                   Chunk({r}, r, 1, ch, "input", origin=r * sh + ch),
                                   Chunk({r}, r, 1, r * sh + ch, "output", origin=r * sh + ch), r, r, bars,
                                   {"step": 1, "channel": ch}) for r in range(n)]
        for r in range(n):
            ir.create_operation(PrimitiveOpType.BARRIER, None, None, r, r, sts, {"step": 2, "channel": ch})
    return ir


# ---------------------------------------------------------------------------------------------
# rooted and point-to-point programs
# ---------------------------------------------------------------------------------------------
def _check_rank(n: int, **ranks) -> None:
    for what, r in ranks.items():
        if not 0 <= r < n:
            raise ValueError(f"{what}={r} is not a rank of a world of {n}")


def _ack(ir: CollectiveIR, consumer: int, producer: int, after: int, step: int, ch: int) -> int:
    """The consumer tells the producer that it has taken the data out of its workspace, and the producer waits for
    that before it ends.  In the symmetric collectives every rank needs something from every other rank in every
    launch, so nobody gets ahead; a rank that ONLY sends could otherwise run two launches ahead and overwrite a
    workspace half (the halves alternate by launch) that the receiver of the launch before last still reads."""
    nt = ir.notify(consumer, producer, deps=[after], step=step, channel=ch)
    return ir.get_notified(consumer, producer, deps=[nt], step=step, channel=ch)


def send_recv(n: int, channels: int = 1, device_type=DeviceType.CUDA, src: int = 0, dst: int = 1) -> CollectiveIR:
    """Point to point: rank ``src``'s input becomes rank ``dst``'s output.  The sender stores into the receiver's
    workspace and the receiver copies out, so neither tensor needs to come from the symmetric heap; the other
    ranks have empty programs."""
    _check_rank(n, src=src, dst=dst)
    U = channels
    ir = _new(f"send_recv_n{n}_c{channels}_{src}to{dst}", "send_recv", n, U,
              {"input": U, "output": U, "scratch": U}, device_type)
    ir.attrs.update(src=src, dst=dst)
    ir.set_precondition([Chunk({src}, src, U, 0, "input")])
    ir.set_postcondition([Chunk({src}, dst, U, 0, "output")])
    for ch in range(channels):
        if src == dst:
            ir.copy(Chunk({src}, src, 1, ch, "input"), Chunk({src}, src, 1, ch, "output"), step=0, channel=ch)
            continue
        push = ir.copy(Chunk({src}, src, 1, ch, "input"), Chunk({src}, dst, 1, ch, "scratch", origin=ch),
                       step=0, channel=ch)
        took = ir.copy(Chunk({src}, dst, 1, ch, "scratch", origin=ch), Chunk({src}, dst, 1, ch, "output"),
                       deps=[push], step=1, channel=ch)
        _ack(ir, dst, src, took, 2, ch)
    return ir


def ring_shift(n: int, channels: int = 1, device_type=DeviceType.CUDA, shift: int = 1) -> CollectiveIR:
    """Permutation: rank r's input becomes the output of rank (r + shift) mod n.  One hop of ring attention's KV
    rotation when the attention of a block is computed between two hops; each receiver acknowledges, because a
    rank's sends depend on nothing that its receiver does."""
    U = channels
    shift %= n
    ir = _new(f"ring_shift_n{n}_c{channels}_s{shift}", "permute", n, U, {"input": U, "output": U, "scratch": U}, device_type)
    ir.attrs["shift"] = shift
    ir.set_precondition([Chunk({r}, r, U, 0, "input", origin=r * U) for r in range(n)])
    ir.set_postcondition([Chunk({r}, (r + shift) % n, U, 0, "output", origin=r * U) for r in range(n)])
    for ch in range(channels):
        for r in range(n):
            d = (r + shift) % n
            org = r * U + ch
            if d == r:
                ir.copy(Chunk({r}, r, 1, ch, "input", origin=org), Chunk({r}, r, 1, ch, "output", origin=org), step=0, channel=ch)
                continue
            push = ir.copy(Chunk({r}, r, 1, ch, "input", origin=org), Chunk({r}, d, 1, ch, "scratch", origin=org),
                           step=0, channel=ch)
            took = ir.copy(Chunk({r}, d, 1, ch, "scratch", origin=org), Chunk({r}, d, 1, ch, "output", origin=org),
                           deps=[push], step=1, channel=ch)
            _ack(ir, d, r, took, 2, ch)
    return ir


def broadcast(n: int, channels: int = 1, device_type=DeviceType.CUDA, root: int = 0, tree: bool = False) -> CollectiveIR:
    """``root``'s input reaches every rank's output.  Default: the root stores to every peer in one step (on a switch
    its port is the limit either way and one hop is the shortest path); ``tree=True`` relays along a binomial tree,
    log2(n) rounds in which every holder sends once, for links where the root's fan-out is the bottleneck."""
    _check_rank(n, root=root)
    U = channels
    ir = _new(f"broadcast_n{n}_c{channels}_r{root}{'_tree' if tree else ''}", "broadcast", n, U,
              {"input": U, "output": U, "scratch": U}, device_type)
    ir.attrs["root"] = root
    ir.set_precondition([Chunk({root}, root, U, 0, "input")])
    ir.set_postcondition([Chunk({root}, r, U, 0, "output") for r in range(n)])
    real = lambda v: (v + root) % n        # the tree is laid over ranks counted from the root
    for ch in range(channels):
        got = {root: ir.copy(Chunk({root}, root, 1, ch, "input"), Chunk({root}, root, 1, ch, "output"), step=0, channel=ch)}
        if not tree:
            for v in range(1, n):
                d = real(v)
                push = ir.copy(Chunk({root}, root, 1, ch, "input"), Chunk({root}, d, 1, ch, "scratch", origin=ch),
                               step=0, channel=ch)
                took = ir.copy(Chunk({root}, d, 1, ch, "scratch", origin=ch), Chunk({root}, d, 1, ch, "output"),
                               deps=[push], step=1, channel=ch)
                _ack(ir, d, root, took, 2, ch)
            continue
        dist = 1
        while dist * 2 < n:
            dist *= 2
        step = 1
        parent = {}
        while dist >= 1:
            for v in range(0, n, 2 * dist):
                if v + dist >= n:
                    continue
                a, b = real(v), real(v + dist)
                push = ir.copy(Chunk({root}, a, 1, ch, "output"), Chunk({root}, b, 1, ch, "scratch", origin=ch),
                               deps=[got[a]], step=step, channel=ch)
                got[b] = ir.copy(Chunk({root}, b, 1, ch, "scratch", origin=ch), Chunk({root}, b, 1, ch, "output"),
                                 deps=[push], step=step + 1, channel=ch)
                parent[b] = a
            dist //= 2
            step += 2
        for b, a in parent.items():         # after the last round, so that no parent's later sends wait for an ack
            _ack(ir, b, a, got[b], step, ch)
    return ir


def scatter_allgather_broadcast(n: int, channels: int = 1, device_type=DeviceType.CUDA, root: int = 0) -> CollectiveIR:
    """Broadcast of a long vector in two steps: the root sends piece d to rank d, then every rank sends its piece to
    all the others.  The root's port carries the vector once instead of n-1 times, and so does every other port."""
    _check_rank(n, root=root)
    sh = channels
    U = n * sh
    ir = _new(f"scatter_allgather_broadcast_n{n}_c{channels}_r{root}", "broadcast", n, U,
              {"input": U, "output": U, "scratch": U}, device_type)
    ir.attrs["root"] = root
    ir.set_precondition([Chunk({root}, root, U, 0, "input")])
    ir.set_postcondition([Chunk({root}, r, U, 0, "output") for r in range(n)])
    for ch in range(channels):
        have = {}
        for k in range(n):                  # step 0-1: piece d -> rank d
            d = (root + k) % n
            u = d * sh + ch
            if d == root:
                for v in range(n):          # the root keeps everything
                    own = ir.copy(Chunk({root}, root, 1, v * sh + ch, "input"), Chunk({root}, root, 1, v * sh + ch, "output"),
                                  step=0, channel=ch)
                    if v == root:
                        have[root] = own
                continue
            push = ir.copy(Chunk({root}, root, 1, u, "input"), Chunk({root}, d, 1, u, "scratch", origin=u), step=0, channel=ch)
            have[d] = ir.copy(Chunk({root}, d, 1, u, "scratch", origin=u), Chunk({root}, d, 1, u, "output"),
                              deps=[push], step=1, channel=ch)
            _ack(ir, d, root, have[d], 4, ch)           # the root receives nothing else from d
        for d in range(n):                  # step 2-3: every other rank hands its piece round (the root has them all)
            if d == root:
                continue
            u = d * sh + ch
            for k in range(1, n):
                e = (d + k) % n
                if e == root:
                    continue
                push = ir.copy(Chunk({root}, d, 1, u, "output"), Chunk({root}, e, 1, u, "scratch", origin=u),
                               deps=[have[d]], step=2, channel=ch)
                ir.copy(Chunk({root}, e, 1, u, "scratch", origin=u), Chunk({root}, e, 1, u, "output"),
                        deps=[push], step=3, channel=ch)
        for e in range(n):                  # the root's own piece reaches the others from the root
            if e == root:
                continue
            u = root * sh + ch
            push = ir.copy(Chunk({root}, root, 1, u, "input"), Chunk({root}, e, 1, u, "scratch", origin=u), step=2, channel=ch)
            ir.copy(Chunk({root}, e, 1, u, "scratch", origin=u), Chunk({root}, e, 1, u, "output"), deps=[push], step=3, channel=ch)
    return ir


def reduce(n: int, channels: int = 1, device_type=DeviceType.CUDA, redop: str = "sum", root: int = 0) -> CollectiveIR:
    """Rooted reduction along a binomial tree: log2(n) rounds, after which ``root``'s output holds the reduction of
    every rank's input.  The other ranks accumulate in their workspace; their outputs are left alone."""
    _check_rank(n, root=root)
    U = channels
    levels = max(1, (n - 1).bit_length())
    ir = _new(f"reduce_n{n}_c{channels}_r{root}", "reduce", n, U,
              {"input": U, "output": U, "scratch": U * (levels + 1)}, device_type, redop)
    ir.attrs["root"] = root
    ir.set_precondition([Chunk({r}, r, U, 0, "input") for r in range(n)])
    ir.set_postcondition([Chunk(_all(n), root, U, 0, "output")])
    real = lambda v: (v + root) % n

    def acc(r: int, have, ch: int) -> Chunk:        # where rank r keeps its partial result
        if r == root:
            return Chunk(have, r, 1, ch, "output")
        return Chunk(have, r, 1, levels * U + ch, "scratch", origin=ch)
    for ch in range(channels):
        last, have = {}, {}
        for r in range(n):
            have[r] = {r}
            last[r] = ir.copy(Chunk({r}, r, 1, ch, "input"), acc(r, {r}, ch), step=0, channel=ch)
        lvl, dist, step = 0, 1, 1
        while dist < n:
            for v in range(0, n, 2 * dist):
                if v + dist >= n:
                    continue
                a, b = real(v), real(v + dist)
                slot = lvl * U + ch
                push = ir.copy(acc(b, have[b], ch), Chunk(have[b], a, 1, slot, "scratch", origin=ch),
                               deps=[last[b]], step=step, channel=ch)
                last[a] = ir.reduce(Chunk(have[b], a, 1, slot, "scratch", origin=ch), acc(a, have[a] | have[b], ch),
                                    deps=[push, last[a]], step=step + 1, channel=ch)
                _ack(ir, a, b, last[a], step + 2, ch)        # b has sent its only message: waiting costs it nothing
                have[a] = have[a] | have[b]
            dist *= 2
            lvl += 1
            step += 2
    return ir


def reduce_scatter_gather_reduce(n: int, channels: int = 1, device_type=DeviceType.CUDA, redop: str = "sum",
                                 root: int = 0) -> CollectiveIR:
    """Rooted reduction of a long vector in two steps: piece d is reduced on rank d (every rank sends it its
    contribution), then every rank hands its reduced piece to the root.  Every port carries the vector about once,
    where the tree form sends the whole vector log2(n) times in a row.  Scratch: block 0 holds a rank's own reduced
    piece (on the root: the pieces that come back), block 1 + r the contribution received from rank r."""
    _check_rank(n, root=root)
    sh = channels
    U = n * sh
    ir = _new(f"reduce_scatter_gather_reduce_n{n}_c{channels}_r{root}", "reduce", n, U,
              {"input": U, "output": U, "scratch": (n + 1) * U}, device_type, redop)
    ir.attrs["root"] = root
    ir.set_precondition([Chunk({r}, r, U, 0, "input") for r in range(n)])
    ir.set_postcondition([Chunk(_all(n), root, U, 0, "output")])
    for ch in range(channels):
        for d in range(n):
            u = d * sh + ch

            def acc(ranks):
                return Chunk(set(ranks), d, 1, u, "output") if d == root else Chunk(set(ranks), d, 1, u, "scratch", origin=u)
            last = ir.copy(Chunk({d}, d, 1, u, "input"), acc({d}), step=0, channel=ch)
            have = {d}
            for k in range(1, n):
                r = (d + k) % n
                slot = Chunk({r}, d, 1, (1 + r) * U + u, "scratch", origin=u)
                push = ir.copy(Chunk({r}, r, 1, u, "input"), slot, step=0, channel=ch)
                last = ir.reduce(slot, acc(have | {r}), deps=[push, last], step=k, channel=ch)
                have = have | {r}
            if d != root:
                back = ir.copy(acc(have), Chunk(set(have), root, 1, u, "scratch", origin=u), deps=[last], step=n, channel=ch)
                ir.copy(Chunk(set(have), root, 1, u, "scratch", origin=u), Chunk(set(have), root, 1, u, "output"),
                        deps=[back], step=n + 1, channel=ch)
    return ir


def scatter(n: int, channels: int = 1, device_type=DeviceType.CUDA, root: int = 0) -> CollectiveIR:
    """Block d of ``root``'s input becomes rank d's output."""
    _check_rank(n, root=root)
    blk = channels
    ir = _new(f"scatter_n{n}_c{channels}_r{root}", "scatter", n, n * blk,
              {"input": n * blk, "output": blk, "scratch": blk}, device_type, block_units=blk)
    ir.attrs["root"] = root
    ir.set_precondition([Chunk({root}, root, n * blk, 0, "input")])
    ir.set_postcondition([Chunk({root}, d, blk, 0, "output", origin=d * blk) for d in range(n)])
    for ch in range(channels):
        acks = []
        for k in range(n):
            d = (root + k) % n
            src = Chunk({root}, root, 1, d * blk + ch, "input")
            if d == root:
                ir.copy(src, Chunk({root}, d, 1, ch, "output", origin=d * blk + ch), step=0, channel=ch)
                continue
            push = ir.copy(src, Chunk({root}, d, 1, ch, "scratch", origin=d * blk + ch), step=0, channel=ch)
            took = ir.copy(Chunk({root}, d, 1, ch, "scratch", origin=d * blk + ch),
                           Chunk({root}, d, 1, ch, "output", origin=d * blk + ch), deps=[push], step=1, channel=ch)
            acks.append((d, took))
        for d, took in acks:                # after all the sends
            _ack(ir, d, root, took, 2, ch)
    return ir


def gather(n: int, channels: int = 1, device_type=DeviceType.CUDA, root: int = 0) -> CollectiveIR:
    """Rank s's input becomes block s of ``root``'s output."""
    _check_rank(n, root=root)
    blk = channels
    ir = _new(f"gather_n{n}_c{channels}_r{root}", "gather", n, blk,
              {"input": blk, "output": n * blk, "scratch": n * blk}, device_type, block_units=blk)
    ir.attrs["root"] = root
    ir.set_precondition([Chunk({s}, s, blk, 0, "input", origin=s * blk) for s in range(n)])
    ir.set_postcondition([Chunk({s}, root, blk, s * blk, "output", origin=s * blk) for s in range(n)])
    for ch in range(channels):
        for s in range(n):
            src = Chunk({s}, s, 1, ch, "input", origin=s * blk + ch)
            if s == root:
                ir.copy(src, Chunk({s}, root, 1, s * blk + ch, "output", origin=s * blk + ch), step=0, channel=ch)
                continue
            push = ir.copy(src, Chunk({s}, root, 1, s * blk + ch, "scratch", origin=s * blk + ch), step=0, channel=ch)
            took = ir.copy(Chunk({s}, root, 1, s * blk + ch, "scratch", origin=s * blk + ch),
                           Chunk({s}, root, 1, s * blk + ch, "output", origin=s * blk + ch), deps=[push], step=1, channel=ch)
            _ack(ir, root, s, took, 2, ch)
    return ir


ALGORITHMS = {
    "ring_allreduce": ring_allreduce,
    "ring_allgather": ring_allgather,
    "ring_kv_rotation": ring_kv_rotation,
    "direct_reduce_scatter": direct_reduce_scatter,
    "direct_allgather": direct_allgather,
    "direct_allreduce": direct_allreduce,
    "oneshot_allreduce": oneshot_allreduce,
    "tree_allreduce": tree_allreduce,
    "alltoall": alltoall,
    "ulysses_alltoall": ulysses_alltoall,
    "nvls_allreduce": nvls_allreduce,
    "nvls_reduce_scatter": nvls_reduce_scatter,
    "nvls_allgather": nvls_allgather,
    "ring_reduce_scatter": ring_reduce_scatter,
    "recursive_doubling_allgather": recursive_doubling_allgather,
    "halving_doubling_allreduce": halving_doubling_allreduce,
    "hierarchical_allreduce": hierarchical_allreduce,
    "hierarchical_allgather": hierarchical_allgather,
    "send_recv": send_recv,
    "ring_shift": ring_shift,
    "broadcast": broadcast,
    "scatter_allgather_broadcast": scatter_allgather_broadcast,
    "reduce": reduce,
    "reduce_scatter_gather_reduce": reduce_scatter_gather_reduce,
    "scatter": scatter,
    "gather": gather,
}


def build(name: str, n: int, **kw) -> CollectiveIR:
    """The library algorithm ``name`` for ``n`` ranks.  ``channels`` defaults to the environment variable
    ``PCCL_CHANNELS`` (1 when unset)."""
    if name not in ALGORITHMS:
        raise KeyError(f"unknown algorithm {name!r}; have {sorted(ALGORITHMS)}")
    if "channels" not in kw:
        import os
        env = os.environ.get("PCCL_CHANNELS", "")
        if env.isdigit() and int(env) > 0:
            kw["channels"] = int(env)
    return ALGORITHMS[name](n, **kw)
