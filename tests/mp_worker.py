"""Worker run by tests/test_multigpu.py under torch.distributed.run (one process per GPU).

Every case ends with a barrier and an orderly teardown, also when an assertion fails, so that no
rank leaves while its memory is still bound to the multicast object or while a peer's kernel waits.
"""
from __future__ import annotations

import json
import os
import sys
import traceback

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def case_heap(eng, rank, world):
    """Peer mapping: every rank writes a pattern into its symmetric tensor and reads its neighbour's."""
    t = eng.symmetric_tensor((1024,), torch.float32)
    t.fill_(float(rank + 1))
    torch.cuda.synchronize(); dist.barrier()
    nxt = (rank + 1) % world
    peer = eng.read_peer(nxt, eng.heap_offset(t), (1024,), torch.float32)
    assert torch.all(peer == float(nxt + 1)), "peer read returned the wrong data"
    eng.write_peer(nxt, eng.heap_offset(t), torch.full((8,), 100.0 + rank, device="cuda"))
    torch.cuda.synchronize(); dist.barrier()
    prev = (rank - 1) % world
    assert torch.all(t[:8] == 100.0 + prev) and torch.all(t[8:] == float(rank + 1))
    return {"nvls": eng.has_nvls}


def _coll_checks(eng, rank, world, algo):
    from pccl_b200.ops import collectives as C
    res = {}
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        for n in (8, 1024, 1 << 20, (1 << 20) + 24):
            g = torch.Generator(device="cuda").manual_seed(7)
            xs = [torch.randn(n, generator=g, device="cuda").to(dtype) for _ in range(world)]
            mark = eng.symmetric_mark()
            inp = eng.symmetric_tensor((n,), dtype); out = eng.symmetric_tensor((n,), dtype)
            for it in range(2):
                inp.copy_(xs[rank] * (it + 1))
                C.all_reduce(eng, inp, out, algo=algo)
                torch.cuda.synchronize()
                ref = torch.stack([x.float() * (it + 1) for x in xs]).sum(0)
                err = (out.float() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
                assert err <= tol * world, f"allreduce {algo} {dtype} n={n}: {err}"
            # in place (two-shot)
            inp.copy_(xs[rank]); C.all_reduce(eng, inp, algo=algo); torch.cuda.synchronize()
            ref = torch.stack([x.float() for x in xs]).sum(0)
            assert (inp.float() - ref).abs().max().item() / max(1.0, ref.abs().max().item()) <= tol * world
            # reduce-scatter with scale and fp32 output into a plain tensor
            if n % world == 0:
                inp.copy_(xs[rank])
                shard = torch.empty(n // world, dtype=torch.float32, device="cuda")
                C.reduce_scatter(eng, inp, shard, scale=1.0 / world, algo=algo); torch.cuda.synchronize()
                ref = (torch.stack([x.float() for x in xs]).sum(0) / world)[rank * (n // world):(rank + 1) * (n // world)]
                assert (shard - ref).abs().max().item() <= tol
                # all-gather of the shards back
                src = xs[rank][: n // world].contiguous()
                C.all_gather(eng, src, out, algo=algo); torch.cuda.synchronize()
                ref = torch.cat([x[: n // world] for x in xs])
                assert torch.equal(out, ref), f"allgather {algo} n={n}"
                # all-to-all
                C.all_to_all(eng, xs[rank], out); torch.cuda.synchronize()
                blk = n // world
                ref = torch.cat([x[rank * blk:(rank + 1) * blk] for x in xs])
                assert torch.equal(out, ref), "alltoall"
            eng.symmetric_reset(mark)
            dist.barrier()
    eng.raise_on_status(8, "collectives")
    res["ok"] = True
    return res


def case_coll_p2p(eng, rank, world):
    return _coll_checks(eng, rank, world, "p2p")


def case_coll_nvls(eng, rank, world):
    if not eng.has_nvls:
        return {"skipped": "no multicast"}
    return _coll_checks(eng, rank, world, "nvls")


def case_coll_fp8(eng, rank, world):
    """Block-scaled fp8 all-reduce and reduce-scatter through the Python API."""
    from pccl_b200.ops import collectives as C
    from pccl_b200.ops.gemm import dequant_rows, quant_rows
    blocks = 64 * world
    n = 128 * blocks
    g = torch.Generator(device="cuda").manual_seed(41)
    xs = [(torch.randn(blocks, 128, generator=g, device="cuda") * (1 + r)).bfloat16() for r in range(world)]
    qs = [quant_rows(x) for x in xs]
    ref = torch.stack([dequant_rows(q, s) for q, s in qs]).sum(0)
    q = eng.symmetric_tensor((n,), torch.uint8); s = eng.symmetric_tensor((blocks,), torch.float32)
    oq = eng.symmetric_tensor((n,), torch.uint8); os_ = eng.symmetric_tensor((blocks,), torch.float32)
    rq = eng.symmetric_tensor((n // world,), torch.uint8); rs = eng.symmetric_tensor((blocks // world,), torch.float32)
    for it in range(2):
        q.copy_(qs[rank][0].view(-1)); s.copy_(qs[rank][1].view(-1))
        torch.cuda.synchronize(); dist.barrier()
        C.all_reduce_fp8(eng, q, s, oq, os_)
        C.reduce_scatter_fp8(eng, q, s, rq, rs, lane=1)
        torch.cuda.synchronize()
        got = dequant_rows(oq.view(blocks, 128), os_.view(blocks, 1))
        assert (got - ref).abs().max().item() <= 0.0625 * ref.abs().max().item() + 1e-6, "all_reduce_fp8"
        assert torch.allclose(os_, ref.abs().amax(-1) / 448.0, rtol=1e-5, atol=0)
        mine = ref[rank * (blocks // world):(rank + 1) * (blocks // world)]
        got = dequant_rows(rq.view(blocks // world, 128), rs.view(blocks // world, 1))
        assert (got - mine).abs().max().item() <= 0.0625 * mine.abs().max().item() + 1e-6, "reduce_scatter_fp8"
        dist.barrier()
    eng.raise_on_status(8, "fp8 all-reduce"); eng.raise_on_status(9, "fp8 reduce-scatter")
    return {"ok": True}


def case_rooted(eng, rank, world):
    """Rooted and point-to-point library programs through the interpreter kernel (ordinary device tensors: the data
    travels through the engine's workspace).  Run on demand, it is not in the list of test_multigpu.py:
    `python -m torch.distributed.run --nproc-per-node N tests/mp_worker.py rooted out.json`."""
    from pccl_b200.ops import collectives as C
    n = 48 * 1024 + 8
    base = torch.arange(n, dtype=torch.float32, device="cuda")
    mine = base + 1000 * rank
    root = world - 1
    for it in range(3):
        for algo in ("direct", "tree", "scatter_allgather"):
            t = mine + it
            C.broadcast(eng, t, root=root, algo=algo, width=2)
            torch.cuda.synchronize()
            assert torch.equal(t, base + 1000 * root + it), f"broadcast {algo}"
        for algo in ("tree", "pieces"):
            out = torch.full((n,), -1.0, device="cuda")
            C.reduce(eng, mine + it, out, root=root, algo=algo, channels=2)
            torch.cuda.synchronize()
            want = sum(base + 1000 * r + it for r in range(world)) if rank == root else torch.full((n,), -1.0, device="cuda")
            assert torch.allclose(out, want, rtol=1e-6), f"reduce {algo}"
        big = torch.arange(n * world, dtype=torch.float32, device="cuda") + 7 * rank + it
        part = torch.zeros(n, device="cuda")
        C.scatter(eng, big, part, root=0)
        allv = torch.full((n * world,), -1.0, device="cuda")
        C.gather(eng, mine + it, allv, root=root)
        got = torch.full((n,), -1.0, device="cuda")
        C.send_recv(eng, mine + it, got, src=0, dst=world - 1)
        nxt = torch.zeros(n, device="cuda")
        C.ring_shift(eng, mine + it, nxt, shift=1)
        torch.cuda.synchronize()
        assert torch.equal(part, (torch.arange(n * world, dtype=torch.float32, device="cuda") + it)[rank * n:(rank + 1) * n]), "scatter"
        want = torch.cat([base + 1000 * r + it for r in range(world)]) if rank == root else torch.full((n * world,), -1.0, device="cuda")
        assert torch.equal(allv, want), "gather"
        assert torch.equal(got, base + it if rank == world - 1 else torch.full((n,), -1.0, device="cuda")), "send_recv"
        assert torch.equal(nxt, base + 1000 * ((rank - 1) % world) + it), "ring_shift"
    eng.raise_on_status(0, "rooted programs")
    return {"ok": True}


def case_trace(eng, rank, world):
    """Device-side instruction trace of the interpreter kernel.  Run on demand with PCCL_TRACE=1 in the environment
    (the engine reads it when it is initialised): `PCCL_TRACE=1 python -m torch.distributed.run --nproc-per-node N
    tests/mp_worker.py trace out.json`."""
    from pccl_b200.lang import build
    from pccl_b200.utils.trace import summarize
    eng.regOp("traced_ar", build("direct_allreduce", world, channels=2))
    n = 1 << 20
    x = eng.symmetric_tensor((n,), torch.float32); y = eng.symmetric_tensor((n,), torch.float32)
    x.fill_(float(rank + 1))
    torch.cuda.synchronize(); dist.barrier()
    eng.exeOp("traced_ar", x, y, width=2)
    torch.cuda.synchronize()
    assert torch.all(y == world * (world + 1) / 2)
    doc = eng.trace()
    ev = [e for e in doc["traceEvents"] if e["ph"] == "X"]
    assert ev, "no device stamps came back (was PCCL_TRACE=1 set before the engine was initialised?)"
    assert all(e["dur"] >= 0 and e["pid"] == rank for e in ev)
    stats = summarize(doc)
    assert stats["REDUCE"]["count"] >= 1 and stats["COPY"]["bytes"] > 0
    return {"events": len(ev), "copy_gbs": stats["COPY"]["gbs"]}


def case_interp(eng, rank, world):
    """Lowered programs through the interpreter kernel, including the NVLS ones."""
    from pccl_b200.lang import build
    names = ["ring_allreduce", "direct_allreduce", "direct_reduce_scatter", "direct_allgather", "alltoall", "tree_allreduce"]
    if eng.has_nvls:
        names += ["nvls_allreduce", "nvls_reduce_scatter", "nvls_allgather"]
    n = 64 * 1024
    for name in names:
        ir = build(name, world, channels=2)
        eng.regOp(name, ir)
        coll = ir.collective
        n_in = {"allreduce": n, "reduce_scatter": n * world, "allgather": n, "alltoall": n * world}[coll]
        n_out = {"allreduce": n, "reduce_scatter": n, "allgather": n * world, "alltoall": n * world}[coll]
        g = torch.Generator(device="cuda").manual_seed(11)
        xs = [torch.randn(n_in, generator=g, device="cuda") for _ in range(world)]
        mark = eng.symmetric_mark()
        inp = eng.symmetric_tensor((n_in,), torch.float32); out = eng.symmetric_tensor((n_out,), torch.float32)
        for it in range(2):
            inp.copy_(xs[rank] + it)
            if name.startswith("nvls"):
                torch.cuda.synchronize(); dist.barrier()
            eng.exeOp(name, inp, out, width=4, check=True)
            full = torch.stack([x + it for x in xs])
            res = inp if ir.in_place else out
            if coll == "allreduce":
                ref = full.sum(0)
            elif coll == "reduce_scatter":
                ref = full.sum(0)[rank * n:(rank + 1) * n]
            elif coll == "allgather":
                ref = torch.cat(list(full))
            else:
                ref = torch.cat([f[rank * n:(rank + 1) * n] for f in full])
            err = (res - ref).abs().max().item()
            assert err < 1e-3, f"{name} iteration {it}: {err}"
            dist.barrier()
        eng.symmetric_reset(mark)
    return {"programs": names}


def case_dp(eng, rank, world):
    """Two steps of sharded data-parallel training give every rank the same parameters, equal to a
    single-process run on the concatenated batch (up to bf16 rounding)."""
    from pccl_b200.models import GPT, GPTConfig
    from pccl_b200.parallel import ShardedDataParallel
    cfg = GPTConfig.tiny()
    torch.manual_seed(0)
    model = GPT(cfg, device="cuda")
    dp = ShardedDataParallel(model, eng, lr=1e-3, bucket_mb=0.25)
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, cfg.vocab_size, (2 * world, cfg.seq_len + 1), generator=g)
    mine = data[2 * rank:2 * rank + 2].cuda()
    losses = [float(dp.train_step(mine[:, :-1], mine[:, 1:])) for _ in range(3)]
    torch.cuda.synchronize()
    flat = dp.flat_params.float()
    ref = flat.clone()
    dist.broadcast(ref, 0)
    assert torch.equal(ref, flat), "ranks disagree on the parameters after the all-gather"
    lt = torch.tensor(losses, device="cuda"); dist.all_reduce(lt); lt /= world
    assert lt[-1] < lt[0], f"mean loss did not go down: {lt.tolist()}"
    eng.raise_on_status(9, "dp reduce-scatter"); eng.raise_on_status(10, "dp all-gather")
    return {"losses": lt.tolist()}


def case_dp_milp_ring(eng, rank, world):
    """Gradient reduce-scatter by a MILP-synthesised multi-step schedule (ring topology forced) that the
    interpreter kernel executes: training proceeds and every rank ends with the same parameters."""
    from pccl_b200.models import GPT, GPTConfig
    from pccl_b200.parallel import ShardedDataParallel
    from pccl_b200.synth import Topology
    cfg = GPTConfig.tiny()
    torch.manual_seed(0)
    model = GPT(cfg, device="cuda")
    dp = ShardedDataParallel(model, eng, lr=1e-3, bucket_mb=0.25, topology=Topology.ring(world))
    assert dp.schedule["source"] == ("milp" if world > 1 else "none")
    if world > 2:
        assert dp.interpreted and dp.schedule["steps"] > 1, dp.schedule
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, cfg.vocab_size, (2 * world, cfg.seq_len + 1), generator=g)
    mine = data[2 * rank:2 * rank + 2].cuda()
    losses = [float(dp.train_step(mine[:, :-1], mine[:, 1:])) for _ in range(3)]
    torch.cuda.synchronize()
    eng.raise_on_status(1, "interpreted reduce-scatter")
    flat = dp.flat_params.float()
    ref = flat.clone()
    dist.broadcast(ref, 0)
    assert torch.equal(ref, flat), "ranks disagree on the parameters after the all-gather"
    lt = torch.tensor(losses, device="cuda"); dist.all_reduce(lt); lt /= world
    assert lt[-1] < lt[0], f"mean loss did not go down: {lt.tolist()}"
    return {"losses": lt.tolist(), "schedule": dp.schedule}


def case_fused_tp(eng, rank, world):
    """all-gather -> GEMM and GEMM -> reduce-scatter against gathered/reduced fp32 references."""
    from pccl_b200.ops import check_status
    from pccl_b200.ops.fused_tp import AllGatherGemm, GemmReduceScatter
    M_local, K, N = 256, 1024, 768
    M = M_local * world
    g = torch.Generator(device="cuda").manual_seed(21)
    xs = [(torch.randn(M_local, K, generator=g, device="cuda") * 0.5).bfloat16() for _ in range(world)]
    ws = [(torch.randn(N, K, generator=g, device="cuda") * 0.05).bfloat16() for _ in range(world)]
    ag = AllGatherGemm(eng, M, K, n_copy=8)
    for it in range(3):
        ag.x_local.copy_(xs[rank] * (it + 1))
        out = ag(ws[rank])
        torch.cuda.synchronize()
        check_status("ag_gemm")
        X = torch.cat([x * (it + 1) for x in xs]).float()      # scaled in bf16, like the shards
        ref = X @ ws[rank].float().t()
        err = (out.float() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
        assert err < 0.03, f"ag_gemm iteration {it}: {err}"
        assert torch.equal(ag.x_full.float(), X), "gathered X differs"
        dist.barrier()
    # GEMM -> RS: y differs per rank (each rank holds its K-slice of the activations)
    K2, N2 = 512, 1024
    ys = [(torch.randn(M, K2, generator=g, device="cuda") * 0.5).bfloat16() for _ in range(world)]
    w2 = [(torch.randn(N2, K2, generator=g, device="cuda") * 0.05).bfloat16() for _ in range(world)]
    rs = GemmReduceScatter(eng, M, N2)
    dist.barrier()
    for it in range(3):
        out = rs(ys[rank] if it % 2 == 0 else ys[rank] * 0.5, w2[rank])
        torch.cuda.synchronize()
        check_status("gemm_rs")
        sc = 1.0 if it % 2 == 0 else 0.5
        total = sum((ys[r].float() * sc).bfloat16().float() @ w2[r].float().t() for r in range(world))
        ref = total[rank * M_local:(rank + 1) * M_local]
        err = (out.float() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
        assert err < 0.03, f"gemm_rs iteration {it}: {err}"
        dist.barrier()
    return {"ok": True}


def case_fused_tp_fp8(eng, rank, world):
    """Block-scaled fp8 forms of the two fused paths, chained like an MLP: AG->GEMM (+GELU, quantised output) -> GEMM->RS."""
    from pccl_b200.ops import check_status
    from pccl_b200.ops.fused_tp import AllGatherGemmFp8, GemmReduceScatterFp8
    from pccl_b200.ops.gemm import dequant_blocks, dequant_rows, quant_blocks, quant_rows
    M_local, K, N = 256, 1024, 512
    M = M_local * world
    g = torch.Generator(device="cuda").manual_seed(23)
    xs = [(torch.randn(M_local, K, generator=g, device="cuda") * 0.5).bfloat16() for _ in range(world)]
    w1 = [(torch.randn(N, K, generator=g, device="cuda") * 0.05).bfloat16() for _ in range(world)]
    w2 = [(torch.randn(K, N, generator=g, device="cuda") * 0.05).bfloat16() for _ in range(world)]
    w1q, w1s = quant_blocks(w1[rank])
    w2q, w2s = quant_blocks(w2[rank])
    ag = AllGatherGemmFp8(eng, M, K, n_copy=4)
    rs = GemmReduceScatterFp8(eng, M, K)
    for it in range(3):
        ag.quantize_local((xs[rank].float() * (it + 1)).bfloat16())
        y = ag(w1q, w1s)
        hq, hs = ag(w1q, w1s, gelu=True, quant_out=True)
        z = rs(hq, hs, w2q, w2s)
        torch.cuda.synchronize()
        check_status("fused fp8")
        X = torch.cat([dequant_rows(*quant_rows((x.float() * (it + 1)).bfloat16())) for x in xs])
        assert torch.equal(dequant_rows(ag.xq_full, ag.xs_full), X), "gathered fp8 X differs"
        ref = X @ dequant_blocks(w1q, w1s).t()
        err = (y.float() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
        assert err < 0.02, f"ag_gemm fp8 iteration {it}: {err}"
        # second GEMM: every rank's partial from ITS quantised hidden activations, summed over ranks
        mine = dequant_rows(hq, hs) @ dequant_blocks(w2q, w2s).t()
        total = mine.clone()
        dist.all_reduce(total)
        refz = total[rank * M_local:(rank + 1) * M_local]
        errz = (z.float() - refz).abs().max().item() / max(1.0, refz.abs().max().item())
        assert errz < 0.03, f"gemm_rs fp8 iteration {it}: {errz}"
        href = torch.nn.functional.gelu(ref, approximate="tanh")
        errh = (dequant_rows(hq, hs) - href).abs().max().item() / max(1.0, href.abs().max().item())
        assert errh < 0.07, f"quantised hidden iteration {it}: {errh}"
        dist.barrier()
    # the same all-gather GEMM on the hardware block-scaled pipeline (power-of-two scale bytes)
    from pccl_b200.ops.gemm import quant_blocks_mx, quant_rows_mx, ue8m0_to_float
    agx = AllGatherGemmFp8(eng, M, K, n_copy=4, mx=True)
    wxq, wxs = quant_blocks_mx(w1[rank])
    for it in range(2):
        agx.quantize_local((xs[rank].float() * (it + 1)).bfloat16())
        y = agx(wxq, wxs)
        torch.cuda.synchronize()
        check_status("ag_gemm mx8")
        X = torch.cat([dequant_rows(q, ue8m0_to_float(s)) for q, s in (quant_rows_mx((x.float() * (it + 1)).bfloat16()) for x in xs)])
        ref = X @ dequant_blocks(wxq, ue8m0_to_float(wxs)).t()
        err = (y.float() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
        assert err < 0.02, f"ag_gemm mx8 iteration {it}: {err}"
        dist.barrier()
    return {"ok": True}


def case_tp_mlp(eng, rank, world):
    """Sequence/tensor-parallel MLP (fused forward and backward) against the single-device network."""
    from pccl_b200.ops import check_status
    from pccl_b200.parallel.tp import TensorParallelMLP
    tokens, d, ff = 256 * world, 512, 1024 * world
    torch.manual_seed(40)
    mlp = TensorParallelMLP(eng, tokens, d, ff, n_copy=4)
    # every rank builds the full reference weights from all shards
    def gather(p):
        parts = [torch.empty_like(p.data) for _ in range(world)]
        dist.all_gather(parts, p.data.contiguous())
        return parts
    w1 = torch.cat(gather(mlp.fc1.weight), 0).float().requires_grad_(True)       # [ff, d]
    b1 = torch.cat(gather(mlp.fc1.bias), 0).float().requires_grad_(True)
    w2 = torch.cat(gather(mlp.fc2.weight), 1).float().requires_grad_(True)       # [d, ff]
    g = torch.Generator(device="cuda").manual_seed(41)
    X = torch.randn(tokens, d, generator=g, device="cuda").bfloat16()
    G = (torch.randn(tokens, d, generator=g, device="cuda") * 0.1).bfloat16()
    ml = tokens // world
    x_local = X[rank * ml:(rank + 1) * ml].clone().requires_grad_(True)
    z = mlp(x_local)
    z.backward(G[rank * ml:(rank + 1) * ml])
    torch.cuda.synchronize()
    check_status("tp mlp")
    Xr = X.float().requires_grad_(True)
    zr = torch.nn.functional.gelu(Xr @ w1.t() + b1, approximate="tanh") @ w2.t() + mlp.fc2.bias.float()
    zr.backward(G.float())
    def rel(a, b):
        return (a.float() - b).abs().max().item() / max(1e-6, b.abs().max().item())
    n1 = ff // world
    assert rel(z, zr[rank * ml:(rank + 1) * ml].detach()) < 0.03
    assert rel(x_local.grad, Xr.grad[rank * ml:(rank + 1) * ml]) < 0.04
    assert rel(mlp.fc1.weight.grad, w1.grad[rank * n1:(rank + 1) * n1]) < 0.04
    assert rel(mlp.fc2.weight.grad, w2.grad[:, rank * n1:(rank + 1) * n1]) < 0.04
    assert rel(mlp.fc1.bias.grad, b1.grad[rank * n1:(rank + 1) * n1]) < 0.04
    return {"ok": True}


def case_moe(eng, rank, world):
    """Expert-parallel MoE layer against a dense reference that every rank computes from the gathered inputs."""
    from pccl_b200.ops import check_status
    from pccl_b200.ops.moe import MoEExchange
    T, H, F, E, Kt = 512, 512, 256, 4 * world, 4
    epr = E // world
    g = torch.Generator(device="cuda").manual_seed(31)
    xs = [torch.randn(T, H, generator=g, device="cuda").bfloat16() for _ in range(world)]
    logits = [torch.randn(T, E, generator=g, device="cuda") for _ in range(world)]
    w1 = (torch.randn(E * F, H, generator=g, device="cuda") * 0.05).bfloat16()
    w2 = (torch.randn(E * H, F, generator=g, device="cuda") * 0.05).bfloat16()
    moe = MoEExchange(eng, T, H, E, Kt)
    my_w1 = w1[rank * epr * F:(rank + 1) * epr * F].contiguous()
    my_w2 = w2[rank * epr * H:(rank + 1) * epr * H].contiguous()
    for it in range(2):
        out = moe.forward(xs[rank], logits[rank] + it, my_w1, my_w2)
        torch.cuda.synchronize()
        check_status("moe")
        ids, probs = MoEExchange.route(logits[rank] + it, Kt)
        x = xs[rank]
        xq = x.float().view(T, H // 128, 128)
        sc = xq.abs().amax(-1, keepdim=True) / 448.0
        xd = ((xq / sc).to(torch.float8_e4m3fn).float() * sc).view(T, H).bfloat16().float()
        ref = torch.zeros(T, H, device="cuda")
        for e in range(E):
            h = torch.nn.functional.gelu(xd @ w1[e * F:(e + 1) * F].float().t(), approximate="tanh").bfloat16().float()
            y = (h @ w2[e * H:(e + 1) * H].float().t()).bfloat16().float()
            for k in range(Kt):
                m = ids[:, k] == e
                ref[m] += probs[m, k, None] * y[m]
        err = (out.float() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
        assert err < 0.03, f"moe iteration {it}: {err}"
        dist.barrier()
    eng.raise_on_status(8 + 5, "moe exchange")
    return {"ok": True}


def case_mixed_hosts(eng, rank, world):
    """CUDA ranks that do not share one host (emulated: every rank, or every pair of ranks, claims its own host id).
    Peers of the same "host" keep their NVLink mapping for data; the others are reached over the host/TCP transport
    through a pinned host shadow of the workspace; programs run on the host-driven executor.  A second engine is built
    for this, the worker's own engine is not touched."""
    from pccl_b200.engine import Engine, LaunchEnvironments
    from pccl_b200.lang import build
    per_host = 2 if world >= 4 and world % 2 == 0 else 1
    LaunchEnvironments.setOverride("PCCL_HOST_ID", f"emulated-host-{rank // per_host}")
    e2 = Engine(rank, world)
    try:
        e2.initEngine("cuda", heap_bytes=512 << 20)
        e2.connect(nvls=False)
    finally:
        LaunchEnvironments.setOverride("PCCL_HOST_ID", "")
    st = e2.stats()
    assert st["mixed_hosts"] and not st["multicast"], st
    n = 96 * 1024
    g = torch.Generator(device="cuda").manual_seed(21)
    xs = [torch.randn(n, generator=g, device="cuda") for _ in range(world)]
    info = {}
    e2.regOp("ring", build("ring_allreduce", world, channels=2))
    e2.regOp("hier", build("hierarchical_allreduce", world, channels=1, per_host=per_host))
    e2.regOp("ag", build("direct_allgather", world, channels=1))
    for it in range(3):
        for name in ("ring", "hier"):
            y = torch.full((n,), -1.0, device="cuda")
            stc = e2.exeOp(name, xs[rank] + it, y, width=2)
            assert stc == 0, (name, stc)
            ref = torch.stack(xs).sum(0) + it * world
            assert torch.allclose(y, ref, rtol=1e-5, atol=1e-4), f"{name} launch {it}: {(y - ref).abs().max().item()}"
        out = torch.zeros(world * 4096, device="cuda")
        assert e2.exeOp("ag", xs[rank][:4096].contiguous() + it, out) == 0
        assert torch.equal(out, torch.cat([x[:4096] + it for x in xs])), "allgather"
    st = e2.stats()
    info["tcp_bytes_sent"] = st.get("tcp_bytes_sent", 0)
    assert info["tcp_bytes_sent"] > n * 4 // world
    # kernels that address every peer directly are refused on such a world instead of dereferencing an unmapped peer
    from pccl_b200.ops import collectives as C
    t = e2.symmetric_tensor((1024,), torch.float32)
    try:
        C.all_reduce(e2, t)
        raise AssertionError("a direct kernel ran on a world that spans hosts")
    except RuntimeError as ex:
        assert "span several hosts" in str(ex)
    torch.cuda.synchronize(); dist.barrier()
    del e2
    return info


def case_jit(eng, rank, world):
    """Programs compiled at run time for this world (NVRTC), launched next to the interpreter on the same lane."""
    from pccl_b200.jit import JitOp
    from pccl_b200.lang import build
    names = {"jit_direct_ar": "direct_allreduce", "jit_direct_rs": "direct_reduce_scatter", "jit_ag": "direct_allgather"}
    if eng.has_nvls:
        names["jit_nvls_ar"] = "nvls_allreduce"
    for name, algo in names.items():
        eng.regOp(name, build(algo, world, channels=2))
    ops = {name: JitOp(eng, name) for name in names}
    n = world * 2 * 8192
    g = torch.Generator(device="cuda").manual_seed(33)
    xs = [torch.randn(n, generator=g, device="cuda") for _ in range(world)]
    x = eng.symmetric_tensor((n,), torch.float32)
    y = eng.symmetric_tensor((n,), torch.float32)
    total = torch.stack(xs).sum(0)
    for it in range(3):
        for name in [k for k in names if k.endswith("_ar")]:
            res = x if ops[name].in_place else y                # the in-switch program reduces in place
            x.copy_(xs[rank] + it); y.fill_(-1.0)
            torch.cuda.synchronize(); dist.barrier()
            ops[name](x, y, width=2)
            torch.cuda.synchronize()
            assert torch.allclose(res, total + it * world, rtol=1e-5, atol=1e-4), f"{name} launch {it}"
            dist.barrier()
            x.copy_(xs[rank] + it); y.fill_(-1.0)
            torch.cuda.synchronize(); dist.barrier()
            eng.exeOp(name, x, y, width=2)                      # interpreter launch of the same program in between
            torch.cuda.synchronize()
            assert torch.allclose(res, total + it * world, rtol=1e-5, atol=1e-4), f"{name} interpreted {it}"
            dist.barrier()
        shard = torch.full((n // world,), -1.0, device="cuda")
        x.copy_(xs[rank] + it)
        torch.cuda.synchronize(); dist.barrier()
        ops["jit_direct_rs"](x, shard, width=2)
        gath = torch.zeros(n, device="cuda")
        ops["jit_ag"](xs[rank][: n // world].contiguous(), gath)
        torch.cuda.synchronize()
        assert torch.allclose(shard, (total + it * world)[rank * (n // world):(rank + 1) * (n // world)], rtol=1e-5, atol=1e-4), "reduce-scatter"
        assert torch.equal(gath, torch.cat([v[: n // world] for v in xs])), "all-gather"
    eng.raise_on_status(0, "jit")
    return {"compiled": {k: v.compiled for k, v in ops.items()}}


def case_resident(eng, rank, world):
    """The resident interpreter kernel on every rank: a run of all-reduces and all-gathers queued without a kernel
    launch each; the ranks' kernels wait on one another through the usual signal words (each on its own GPU)."""
    from pccl_b200.lang import build
    eng.regOp("res_ar", build("direct_allreduce", world, channels=2))
    eng.regOp("res_ag", build("direct_allgather", world, channels=1))
    n = 256 * 1024
    xs = [torch.full((n,), float(rank + 1) * (i + 1), device="cuda") for i in range(12)]
    ys = [torch.zeros(n, device="cuda") for _ in range(12)]
    gs = [torch.zeros(world * 1024, device="cuda") for _ in range(12)]
    torch.cuda.synchronize(); dist.barrier()
    eng.start_resident(width=4)
    tickets = []
    for i in range(12):
        tickets.append(eng.enqueue("res_ar", xs[i], ys[i], sync_inputs=False))
        tickets.append(eng.enqueue("res_ag", xs[i][:1024], gs[i], sync_inputs=False))
    eng.wait(tickets[-1], timeout_ms=30000)
    st = eng.check_status(0)
    assert st[0] == 0, list(st)
    for i in range(12):
        want = sum(float(r + 1) * (i + 1) for r in range(world))
        assert torch.all(ys[i] == want), f"all-reduce {i}"
        ref = torch.cat([torch.full((1024,), float(r + 1) * (i + 1), device="cuda") for r in range(world)])
        assert torch.equal(gs[i], ref), f"all-gather {i}"
    stats = eng.stats()
    dist.barrier()
    eng.stop_resident()
    return {"resident_kernel_launches": stats["resident_kernel_launches"], "resident_ops": stats["resident_ops"]}


def case_overlap(eng, rank, world):
    """Two collectives at once on two CUDA streams with disjoint CTA budgets and separate flag lanes (an all-reduce on
    lane 0, an all-gather on lane 1), against the same two back to back on one stream.  Checks both results and
    reports the two times; device-timed, maximum over ranks."""
    from pccl_b200.ops import collectives as C
    n = (32 << 20) // 2                                   # 32 MiB of bf16 per collective
    a_in = eng.symmetric_tensor((n,), torch.bfloat16); a_out = eng.symmetric_tensor((n,), torch.bfloat16)
    g_in = torch.full((n // world,), float(rank + 1), device="cuda", dtype=torch.bfloat16)
    g_out = eng.symmetric_tensor((n,), torch.bfloat16)
    a_in.fill_(1.0)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize(); dist.barrier()

    def together():
        cur = torch.cuda.current_stream()
        s1.wait_stream(cur); s2.wait_stream(cur)
        C.all_reduce(eng, a_in, a_out, blocks=32, lane=0, stream=s1)
        C.all_gather(eng, g_in, g_out, blocks=32, lane=1, stream=s2)
        cur.wait_stream(s1); cur.wait_stream(s2)

    def in_turn():
        C.all_reduce(eng, a_in, a_out, blocks=32, lane=0)
        C.all_gather(eng, g_in, g_out, blocks=32, lane=1)

    def timed(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record(); e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e3

    t_seq = timed(in_turn)
    t_par = timed(together)
    torch.cuda.synchronize()
    assert torch.all(a_out == float(world)), "all-reduce result"
    want = torch.cat([torch.full((n // world,), float(r + 1), dtype=torch.bfloat16) for r in range(world)]).cuda()
    assert torch.equal(g_out, want), "all-gather result"
    eng.raise_on_status(8, "overlap lane 0"); eng.raise_on_status(9, "overlap lane 1")
    return {"back_to_back_us": t_seq, "two_streams_us": t_par, "ratio": t_seq / t_par}


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}


def main():
    case = sys.argv[1]
    out_path = sys.argv[2]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=__import__("datetime").timedelta(seconds=180))
    from pccl_b200.engine import Engine
    os.environ.setdefault("PCCL_WORKSPACE_MB", "256")
    eng = Engine(rank, world)
    result = {"ok": False}
    try:
        eng.initEngine("cuda", heap_bytes=2 << 30)
        eng.connect(nvls=os.environ.get("PCCL_TEST_NVLS", "1") == "1")
        info = {}
        for one in case.split(","):         # several cases may share one launch (start-up dominates their cost)
            mark = eng.symmetric_mark()
            info[one] = CASES[one](eng, rank, world)
            torch.cuda.synchronize()
            dist.barrier()
            eng.symmetric_reset(mark)
        result = {"ok": True, "info": info}
    except BaseException as e:  # noqa: BLE001
        result = {"ok": False, "error": f"{type(e).__name__}: {e}", "trace": traceback.format_exc()}
    try:
        torch.cuda.synchronize()
    except Exception:  # noqa: BLE001
        pass
    flags = [None] * world
    dist.all_gather_object(flags, result)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(flags, f)
    dist.barrier()
    del eng
    dist.destroy_process_group()
    sys.exit(0 if all(f["ok"] for f in flags) else 1)


if __name__ == "__main__":
    main()
