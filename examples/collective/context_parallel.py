#!/usr/bin/env python
"""Long-context attention over ranks, two ways, with the library's collective programs and plain torch math.

* ring attention: every rank keeps its block of queries; the key/value blocks travel round the ring one hop at a
  time (`ring_shift`), and between two hops each rank folds the block it holds into a running softmax.
* Ulysses: an all-to-all turns "my slice of the sequence, all heads" into "the whole sequence, my heads", attention
  runs locally per head, and a second all-to-all turns it back.

Both are checked against attention over the whole sequence on one process.  CPU ranks, no GPU needed:

    python examples/collective/context_parallel.py --world 4          # spawns the ranks itself

On GPUs the same calls run through the interpreter kernel (engine initialised with device="cuda").
"""
import argparse
import math
import os
import socket
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def reference_attention(q, k, v):
    """q, k, v: [heads, seq, dim]; softmax(q k^T / sqrt(dim)) v, no mask."""
    s = torch.einsum("hqd,hkd->hqk", q, k) / math.sqrt(q.shape[-1])
    return torch.einsum("hqk,hkd->hqd", torch.softmax(s, dim=-1), v)


def ring_attention(eng, C, q, k, v):
    """Blockwise attention with a running maximum and denominator; K and V hop to the next rank between blocks."""
    world = eng.world
    scale = 1.0 / math.sqrt(q.shape[-1])
    m = torch.full(q.shape[:2], -float("inf"))          # running row maximum      [heads, q]
    den = torch.zeros(q.shape[:2])                       # running softmax sum
    acc = torch.zeros_like(q)                            # running weighted values
    kv = torch.stack([k, v]).contiguous()
    nxt = torch.empty_like(kv)
    for hop in range(world):
        kb, vb = kv[0], kv[1]
        s = torch.einsum("hqd,hkd->hqk", q, kb) * scale
        m_new = torch.maximum(m, s.amax(dim=-1))
        p = torch.exp(s - m_new.unsqueeze(-1))
        fix = torch.exp(m - m_new)
        den = den * fix + p.sum(dim=-1)
        acc = acc * fix.unsqueeze(-1) + torch.einsum("hqk,hkd->hqd", p, vb)
        m = m_new
        if hop + 1 < world:
            C.ring_shift(eng, kv, nxt, shift=1)          # my block goes to rank+1, rank-1's block comes here
            kv, nxt = nxt, kv
    return acc / den.unsqueeze(-1)


def ulysses_attention(eng, C, q, k, v):
    """q, k, v: [heads, seq/world, dim] -> all-to-all -> [heads/world, seq, dim] -> attention -> all-to-all back."""
    world = eng.world
    H, S, D = q.shape
    hp = H // world

    def alltoall(send, recv):
        eng.exeOp("ulysses", send.view(-1), recv.view(-1))

    def seq_to_heads(x):
        send = x.reshape(world, hp, S, D).contiguous()            # block d = the heads that rank d will own
        recv = torch.empty_like(send)
        alltoall(send, recv)                                      # block s = my heads for rank s's slice of the sequence
        return recv.permute(1, 0, 2, 3).reshape(hp, world * S, D).contiguous()

    def heads_to_seq(x):
        send = x.reshape(hp, world, S, D).permute(1, 0, 2, 3).contiguous()   # block d = rank d's slice of the sequence
        recv = torch.empty_like(send)
        alltoall(send, recv)                                      # block s = the heads rank s owns
        return recv.reshape(H, S, D)

    return heads_to_seq(reference_attention(seq_to_heads(q), seq_to_heads(k), seq_to_heads(v)))


def rank_main(rank, world, port, heads, seq, dim, out):
    from pccl.engine import Engine
    from pccl.lang import DeviceType, build
    from pccl_b200.ops import collectives as C
    torch.manual_seed(0)
    q, k, v = (torch.randn(heads, seq, dim) for _ in range(3))    # the same on every rank; each takes its slice
    blk = seq // world
    mine = slice(rank * blk, (rank + 1) * blk)
    want = reference_attention(q, k, v)[:, mine]

    eng = Engine(rank, world)
    eng.initEngine("cpu")
    if world > 1:
        eng.joinCluster(f"127.0.0.1:{port}")
    eng.regOp("ulysses", build("ulysses_alltoall", world, device_type=DeviceType.CPU))
    ql, kl, vl = (t[:, mine].contiguous() for t in (q, k, v))
    ring = ring_attention(eng, C, ql, kl, vl)
    uly = ulysses_attention(eng, C, ql, kl, vl)
    errs = ((ring - want).abs().max().item(), (uly - want).abs().max().item())
    eng.exitCluster()
    if out is not None:
        out.put((rank, errs))
    return errs


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--dim", type=int, default=32)
    args = ap.parse_args()
    assert args.seq % args.world == 0 and args.heads % args.world == 0, "sequence and heads must divide by the world size"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=rank_main, args=(r, args.world, port, args.heads, args.seq, args.dim, q)) for r in range(args.world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(30)
    for r in sorted(results):
        ring, uly = results[r]
        print(f"rank {r}: ring attention max error {ring:.2e}, Ulysses max error {uly:.2e}")
        assert ring < 1e-4 and uly < 1e-4
    print("context parallel attention matches attention over the whole sequence")


if __name__ == "__main__":
    main()
