"""Hand-written collectives and the interpreter kernel, all ranks emulated on one GPU (one
cooperative launch plays every rank; 'heaps' are buffers of that GPU)."""
import json

import pytest
import torch

pytestmark = pytest.mark.gpu

SIGNAL_OFF = 0            # layout of each emulated heap: [signals 64 KiB | flags 256 KiB | data]
FLAG_OFF = 64 * 1024
DATA_OFF = 512 * 1024
NAMES = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}


def _heaps(world, data_bytes):
    hs = [torch.zeros(DATA_OFF + data_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    return hs, st


def _view(h, off, n, dtype):
    es = torch.empty((), dtype=dtype).element_size()
    return h[DATA_OFF + off: DATA_OFF + off + n * es].view(dtype)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("count", [1, 7, 1024, 256 * 1024 + 17])
def test_allreduce_emulated(native, world, dtype, count):
    es = torch.empty((), dtype=dtype).element_size()
    size = (count * es + 255) // 256 * 256
    hs, st = _heaps(world, 2 * size)
    g = torch.Generator(device="cuda").manual_seed(0)
    xs = [torch.randn(count, generator=g, device="cuda").to(dtype) for _ in range(world)]
    for epoch in (1, 2):
        for r in range(world):
            _view(hs[r], 0, count, dtype).copy_(xs[r] * epoch)
        native.emu_collective("allreduce", [h.data_ptr() for h in hs], SIGNAL_OFF, FLAG_OFF, NAMES[dtype], "sum",
                              DATA_OFF, DATA_OFF + size, count, epoch, 0, 1.0, "", 4, 256,
                              torch.cuda.current_stream().cuda_stream, [s.data_ptr() for s in st], [], [], 0)
        torch.cuda.synchronize()
        assert all(s[0].item() == 0 for s in st)
        ref = torch.stack([x.float() * epoch for x in xs]).sum(0)
        tol = 1e-5 * world if dtype == torch.float32 else 0.04 * world
        for r in range(world):
            got = _view(hs[r], size, count, dtype).float()
            assert (got - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype,redop", [(torch.float32, "sum"), (torch.bfloat16, "sum"), (torch.bfloat16, "max")])
@pytest.mark.parametrize("count", [2, 1024, 16 * 1024])
def test_allreduce_low_latency_path_emulated(native, world, dtype, redop, count):
    """All-reduce of up to 64 KiB with the flag travelling in the data (8-byte packets {word, launch number}): no barrier,
    out of place and in place, several launches on alternating receive areas."""
    es = torch.empty((), dtype=dtype).element_size()
    size = (count * es + 255) // 256 * 256
    ll_off = DATA_OFF + 2 * size
    hs = [torch.zeros(ll_off + native.LL_LANE_BYTES, dtype=torch.uint8, device="cuda") for _ in range(world)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    g = torch.Generator(device="cuda").manual_seed(1)
    xs = [torch.randn(count, generator=g, device="cuda").to(dtype) for _ in range(world)]
    for epoch in (1, 2, 3, 4):
        in_place = epoch == 4
        for r in range(world):
            _view(hs[r], 0, count, dtype).copy_(xs[r] * epoch)
        native.emu_collective("allreduce", [h.data_ptr() for h in hs], SIGNAL_OFF, FLAG_OFF, NAMES[dtype], redop,
                              DATA_OFF, DATA_OFF if in_place else DATA_OFF + size, count, epoch, 0, 1.0, "", 4, 256,
                              torch.cuda.current_stream().cuda_stream, [s.data_ptr() for s in st], [], [], 0, 0, 0, ll_off)
        torch.cuda.synchronize()
        assert all(s[0].item() == 0 for s in st), [s.tolist() for s in st]
        stack = torch.stack([(x * epoch).float() for x in xs])
        ref = stack.sum(0) if redop == "sum" else stack.max(0).values
        tol = 1e-5 * world if dtype == torch.float32 else 0.04 * world
        for r in range(world):
            got = _view(hs[r], 0 if in_place else size, count, dtype).float()
            assert (got - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item()), (epoch, r)
        # the packets of this launch are in the receive area of its parity: the path was taken
        slot = native.LL_LANE_BYTES // 2 // native.MAX_RANKS                      # rank 1's packets in rank 0's area
        first = hs[0][ll_off + (epoch & 1) * (native.LL_LANE_BYTES // 2) + slot:][:8].view(torch.int64)[0].item()
        assert first >> 32 == epoch, "the low-latency path was not taken"


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("redop", ["max", "min"])
def test_allreduce_minmax_in_place(native, world, redop):
    count, dtype = 5000, torch.bfloat16
    hs, st = _heaps(world, 1 << 16)
    g = torch.Generator(device="cuda").manual_seed(1)
    xs = [torch.randn(count, generator=g, device="cuda").to(dtype) for _ in range(world)]
    for r in range(world):
        _view(hs[r], 0, count, dtype).copy_(xs[r])
    native.emu_collective("allreduce", [h.data_ptr() for h in hs], SIGNAL_OFF, FLAG_OFF, "bf16", redop, DATA_OFF, DATA_OFF,
                          count, 1, 1, 1.0, "", 3, 128, torch.cuda.current_stream().cuda_stream,
                          [s.data_ptr() for s in st], [], [], 0)
    torch.cuda.synchronize()
    ref = torch.stack(xs).float().max(0).values if redop == "max" else torch.stack(xs).float().min(0).values
    for r in range(world):
        assert torch.equal(_view(hs[r], 0, count, dtype).float(), ref)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("count", [16, 4096 + 8, 100003])
def test_reduce_scatter_scale_cast_emulated(native, world, count):
    """Gradient-bucket form: bf16 in, sum over ranks, x 1/world, fp32 out into a plain tensor."""
    dtype = torch.bfloat16
    size = (world * count * 2 + 255) // 256 * 256
    hs, st = _heaps(world, size)
    g = torch.Generator(device="cuda").manual_seed(2)
    xs = [torch.randn(world * count, generator=g, device="cuda").to(dtype) for _ in range(world)]
    outs = [torch.zeros(count, dtype=torch.float32, device="cuda") for _ in range(world)]
    for r in range(world):
        _view(hs[r], 0, world * count, dtype).copy_(xs[r])
    native.emu_collective("reduce_scatter", [h.data_ptr() for h in hs], SIGNAL_OFF, FLAG_OFF, "bf16", "sum", DATA_OFF, 0,
                          count, 1, 2, 1.0 / world, "f32", 4, 256, torch.cuda.current_stream().cuda_stream,
                          [s.data_ptr() for s in st], [], [o.data_ptr() for o in outs], 0)
    torch.cuda.synchronize()
    assert all(s[0].item() == 0 for s in st)
    full = torch.stack([x.float() for x in xs]).sum(0) / world
    for r in range(world):
        assert (outs[r] - full[r * count:(r + 1) * count]).abs().max().item() < 1e-5


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("kind", ["allgather", "alltoall"])
@pytest.mark.parametrize("nbytes", [16, 1000, 64 * 1024 + 48])
def test_allgather_alltoall_emulated(native, world, kind, nbytes):
    size = (world * nbytes + 255) // 256 * 256
    hs, st = _heaps(world, size)
    g = torch.Generator(device="cuda").manual_seed(3)
    n_in = nbytes if kind == "allgather" else world * nbytes
    xs = [torch.randint(0, 255, (n_in,), generator=g, device="cuda", dtype=torch.uint8) for _ in range(world)]
    native.emu_collective(kind, [h.data_ptr() for h in hs], SIGNAL_OFF, FLAG_OFF, "f32", "sum", 0, DATA_OFF, nbytes, 1, 3,
                          1.0, "", 2, 256, torch.cuda.current_stream().cuda_stream, [s.data_ptr() for s in st],
                          [x.data_ptr() for x in xs], [], 0)
    torch.cuda.synchronize()
    assert all(s[0].item() == 0 for s in st)
    for r in range(world):
        got = hs[r][DATA_OFF:DATA_OFF + world * nbytes]
        if kind == "allgather":
            ref = torch.cat(xs)
        else:
            ref = torch.cat([x[r * nbytes:(r + 1) * nbytes] for x in xs])
        assert torch.equal(got, ref)


@pytest.mark.parametrize("algo", ["ring_allreduce", "direct_allreduce", "oneshot_allreduce", "tree_allreduce",
                                  "direct_reduce_scatter", "direct_allgather", "ring_kv_rotation", "alltoall"])
@pytest.mark.parametrize("world,width", [(2, 1), (4, 2)])
def test_interpreter_runs_lowered_programs(native, algo, world, width):
    from pccl_b200.lang import build, to_schedule
    ir = build(algo, world, channels=2)
    doc = json.dumps(to_schedule(ir))
    dtype, n = torch.float32, 3000 + 5
    coll = ir.collective
    n_in = {"allreduce": n, "reduce_scatter": n * world, "allgather": n, "alltoall": n * world}[coll]
    n_out = {"allreduce": n, "reduce_scatter": n, "allgather": n * world, "alltoall": n * world}[coll]
    hs, st = _heaps(world, 16 << 20)
    g = torch.Generator(device="cuda").manual_seed(4)
    xs = [torch.randn(n_in, generator=g, device="cuda") for _ in range(world)]
    ys = [torch.full((n_out,), -5.0, device="cuda") for _ in range(world)]
    for epoch in (0, 1):
        native.emu_program(doc, [h.data_ptr() for h in hs], SIGNAL_OFF, [x.data_ptr() for x in xs],
                           [y.data_ptr() for y in ys], n_in * 4, "f32", width, DATA_OFF + epoch * (8 << 20), 0, epoch,
                           0, [s.data_ptr() for s in st], [], torch.cuda.current_stream().cuda_stream)
        assert all(s[0].item() == 0 for s in st), [s.tolist() for s in st]
        full = torch.stack(xs)
        for r in range(world):
            if coll == "allreduce":
                ref = full.sum(0)
            elif coll == "reduce_scatter":
                ref = full.sum(0)[r * n:(r + 1) * n]
            elif coll == "allgather":
                ref = torch.cat(xs)
            else:
                ref = torch.cat([x[r * n:(r + 1) * n] for x in xs])
            assert (ys[r] - ref).abs().max().item() < 1e-4, (algo, r)


@pytest.mark.parametrize("algo", ["direct_allreduce", "direct_reduce_scatter", "direct_allgather"])
@pytest.mark.parametrize("world,width", [(2, 1), (4, 2), (8, 2)])
def test_interpreter_runs_pull_forms_on_symmetric_buffers(native, algo, world, width):
    """``direct=True``: peers' inputs are read and peers' outputs written in place (same heap offset on every rank), no
    scratch; three launches in a row with changing inputs, so a rank that ran ahead of the barriers would be seen."""
    from pccl_b200.lang import build, to_schedule
    ir = build(algo, world, channels=2, direct=True)
    assert ir.buffers["scratch"] == 0
    doc = json.dumps(to_schedule(ir))
    n = 2048 + 8
    coll = ir.collective
    n_in = {"allreduce": n, "reduce_scatter": n * world, "allgather": n}[coll]
    n_out = {"allreduce": n, "reduce_scatter": n, "allgather": n * world}[coll]
    hs, st = _heaps(world, 4 << 20)
    in_off, out_off = DATA_OFF + (1 << 20), DATA_OFF + (2 << 20)
    g = torch.Generator(device="cuda").manual_seed(14)
    for epoch in range(3):
        xs = [torch.randn(n_in, generator=g, device="cuda") for _ in range(world)]
        for r in range(world):
            _view(hs[r], in_off - DATA_OFF, n_in, torch.float32).copy_(xs[r])
            _view(hs[r], out_off - DATA_OFF, n_out, torch.float32).fill_(-5.0)
        native.emu_program(doc, [h.data_ptr() for h in hs], SIGNAL_OFF, [h.data_ptr() + in_off for h in hs],
                           [h.data_ptr() + out_off for h in hs], n_in * 4, "f32", width, DATA_OFF, 0, epoch,
                           0, [s.data_ptr() for s in st], [], torch.cuda.current_stream().cuda_stream)
        assert all(s[0].item() == 0 for s in st), [s.tolist() for s in st]
        full = torch.stack(xs)
        for r in range(world):
            got = _view(hs[r], out_off - DATA_OFF, n_out, torch.float32)
            ref = full.sum(0) if coll == "allreduce" else (full.sum(0)[r * n:(r + 1) * n] if coll == "reduce_scatter" else torch.cat(xs))
            assert (got - ref).abs().max().item() < 1e-4, (algo, r, epoch)


def test_bounded_wait_returns_timeout_status(native):
    """A wait on a flag nobody sets comes back with ST_TIMEOUT; the context stays usable."""
    flag = torch.zeros(1, dtype=torch.int64, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    native.wait_timeout_probe(flag.data_ptr(), 200_000, st.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st[0].item() == 1
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_interpreter_peer_never_arrives(native):
    """Rank 1's streams are left out: rank 0 gives up after its time limit and reports where."""
    from pccl_b200.lang import build, to_schedule
    doc = json.dumps(to_schedule(build("ring_allreduce", 2)))
    hs, st = _heaps(2, 1 << 20)
    xs = [torch.ones(1024, device="cuda") for _ in range(2)]
    ys = [torch.zeros(1024, device="cuda") for _ in range(2)]
    native.emu_program(doc, [h.data_ptr() for h in hs], SIGNAL_OFF, [x.data_ptr() for x in xs], [y.data_ptr() for y in ys],
                       4096, "f32", 1, DATA_OFF, 0, 0, 100_000, [s.data_ptr() for s in st], [1],
                       torch.cuda.current_stream().cuda_stream)
    assert st[0][0].item() == 1 and st[1][0].item() == 0
    assert torch.ones(4, device="cuda").sum().item() == 4.0


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("kind,redop", [("allreduce_fp8", "sum"), ("allreduce_fp8", "max"), ("reduce_scatter_fp8", "sum")])
def test_fp8_block_scaled_reduce_emulated(native, world, kind, redop):
    """Block-scaled fp8 all-reduce / reduce-scatter: dequantise, accumulate in fp32, requantise with a fresh scale."""
    from pccl_b200.ops.gemm import dequant_rows, quant_rows
    shard_blocks = 24
    n = 128 * shard_blocks * world            # elements of the whole vector
    g = torch.Generator(device="cuda").manual_seed(33)
    xs = [(torch.randn(n // 128, 128, generator=g, device="cuda") * (1 + r)).bfloat16() for r in range(world)]
    qs = [quant_rows(x) for x in xs]
    q_in, s_in = DATA_OFF, DATA_OFF + n
    q_out, s_out = s_in + (n // 128) * 4, s_in + (n // 128) * 4 + n
    hs = [torch.zeros(s_out + (n // 128) * 4 + 256, dtype=torch.uint8, device="cuda") for _ in range(world)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    for r in range(world):
        hs[r][q_in:q_in + n] = qs[r][0].view(-1)
        hs[r][s_in:s_in + (n // 128) * 4].view(torch.float32)[:] = qs[r][1].view(-1)
    count = n if kind == "allreduce_fp8" else n // world
    native.emu_collective(kind, [h.data_ptr() for h in hs], SIGNAL_OFF, FLAG_OFF, "e4m3", redop, q_in, q_out, count, 1, 2, 1.0, "",
                          4, 256, torch.cuda.current_stream().cuda_stream, [s.data_ptr() for s in st], [], [], 0, s_in, s_out)
    torch.cuda.synchronize()
    assert all(s[0].item() == 0 for s in st), [s.tolist() for s in st]
    vals = torch.stack([dequant_rows(q, s) for q, s in qs])       # [world, n/128, 128] exact inputs
    ref = vals.sum(0) if redop == "sum" else vals.amax(0)
    for r in range(world):
        if kind == "allreduce_fp8":
            oq = hs[r][q_out:q_out + n].view(n // 128, 128)
            os_ = hs[r][s_out:s_out + (n // 128) * 4].view(torch.float32).view(n // 128, 1)
            want = ref
        else:
            m = n // world
            oq = hs[r][q_out:q_out + m].view(m // 128, 128)
            os_ = hs[r][s_out:s_out + (m // 128) * 4].view(torch.float32).view(m // 128, 1)
            want = ref[r * shard_blocks:(r + 1) * shard_blocks]
        # the fresh scale is the block maximum over 448, and the payload is the e4m3 rounding of value / scale
        assert torch.allclose(os_.view(-1), want.abs().amax(-1) / 448.0, rtol=1e-5, atol=0)
        got = dequant_rows(oq, os_)
        assert (got - want).abs().max().item() <= 0.0625 * want.abs().max().item() + 1e-6
        want_q = (want / os_).to(torch.float8_e4m3fn).float()
        assert (oq.view(torch.float8_e4m3fn).float() - want_q).abs().max().item() <= 32.0     # at most one e4m3 step at the top of the range


# ---------------------------------------------------------------------------------------------
# fused collective + GEMM kernels, ranks emulated on one GPU
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("world,tail", [(2, -1), (4, -1), (2, 0), (2, 2), (2, 100), (4, 5)])
def test_ag_gemm_emulated(native, world, tail):
    """`tail`: tiles at the end of the tile order that the copy CTAs compute after sending their rows (-1: cost model,
    0: none, a number beyond the tile count: all of them)."""
    M_local, K, N = 256, 512, 520
    M = M_local * world
    g = torch.Generator(device="cuda").manual_seed(9)
    xs = [(torch.randn(M_local, K, generator=g, device="cuda") * 0.5).bfloat16() for _ in range(world)]
    ws = [(torch.randn(N, K, generator=g, device="cuda") * 0.1).bfloat16() for _ in range(world)]
    x_off = DATA_OFF
    ready_off = DATA_OFF + M * K * 2
    heaps = [torch.zeros(ready_off + 4096, dtype=torch.uint8, device="cuda") for _ in range(world)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    outs = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ctas = 148 // world
    for epoch in (1, 2):
        for r in range(world):
            full = heaps[r][x_off:x_off + M * K * 2].view(torch.bfloat16).view(M, K)
            full.zero_()
            full[r * M_local:(r + 1) * M_local] = xs[r] * epoch
        native.emu_ag_gemm([h.data_ptr() for h in heaps], FLAG_OFF, x_off, M, N, K, [w.data_ptr() for w in ws], K,
                           [o.data_ptr() for o in outs], N, ready_off, epoch, 4, ctas,
                           [s.data_ptr() for s in st], 0, torch.cuda.current_stream().cuda_stream, tail)
        torch.cuda.synchronize()
        assert all(s[0].item() == 0 for s in st), [s.tolist() for s in st]
        X = torch.cat(xs).float() * epoch
        for r in range(world):
            ref = X @ ws[r].float().t()
            assert (outs[r].float() - ref).abs().max().item() < 0.03 * max(1.0, ref.abs().max().item())
            gathered = heaps[r][x_off:x_off + M * K * 2].view(torch.bfloat16).view(M, K)
            assert torch.equal(gathered.float(), X)


@pytest.mark.parametrize("world,M_local", [(2, 128), (2, 256), (4, 128), (2, 512)])
def test_gemm_rs_emulated(native, world, M_local):
    K, N = 448, 512     # 256 rows per rank and an even CTA count take the CTA-pair pipeline (whole rows staged per tile)
    M = M_local * world
    g = torch.Generator(device="cuda").manual_seed(10)
    ys = [(torch.randn(M, K, generator=g, device="cuda") * 0.5).bfloat16() for _ in range(world)]
    ws = [(torch.randn(N, K, generator=g, device="cuda") * 0.1).bfloat16() for _ in range(world)]
    stage_bytes = world * M_local * N * 2
    n_flags = world * (M_local // 128) * (N // 256)
    heaps = [torch.zeros(DATA_OFF + stage_bytes + n_flags * 8, dtype=torch.uint8, device="cuda") for _ in range(world)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    outs = [torch.zeros(M_local, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for epoch in (1, 2):
        native.emu_gemm_rs([h.data_ptr() for h in heaps], [y.data_ptr() for y in ys], K, [w.data_ptr() for w in ws], K,
                           [o.data_ptr() for o in outs], N, M, N, K, DATA_OFF, DATA_OFF + stage_bytes, epoch, 148 // world,
                           [s.data_ptr() for s in st], 0, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert all(s[0].item() == 0 for s in st), [s.tolist() for s in st]
        total = sum(ys[r].float() @ ws[r].float().t() for r in range(world))
        for r in range(world):
            ref = total[r * M_local:(r + 1) * M_local]
            assert (outs[r].float() - ref).abs().max().item() < 0.03 * max(1.0, ref.abs().max().item())
        for y in ys:
            y.mul_(0.5)


@pytest.mark.parametrize("world,quant_out", [(2, False), (4, False), (2, True)])
def test_ag_gemm_fp8_emulated(native, world, quant_out):
    from pccl_b200.ops.gemm import dequant_blocks, dequant_rows, quant_blocks, quant_rows
    M_local, K, N = 256, 1024, 512
    M = M_local * world
    g = torch.Generator(device="cuda").manual_seed(19)
    xs = [(torch.randn(M_local, K, generator=g, device="cuda") * 0.5).bfloat16() for _ in range(world)]
    ws = [quant_blocks((torch.randn(N, K, generator=g, device="cuda") * 0.1).bfloat16()) for _ in range(world)]
    x_off = DATA_OFF
    xs_off = x_off + M * K
    ready_off = xs_off + M * (K // 128) * 4
    heaps = [torch.zeros(ready_off + 4096, dtype=torch.uint8, device="cuda") for _ in range(world)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    outs = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    oq = [torch.zeros(M, N, dtype=torch.uint8, device="cuda") for _ in range(world)]
    os_ = [torch.zeros(M, N // 128, dtype=torch.float32, device="cuda") for _ in range(world)]
    ctas = 148 // world
    for epoch in (1, 2):
        X = []
        for r in range(world):
            q, s = quant_rows((xs[r].float() * epoch).bfloat16())
            X.append(dequant_rows(q, s))
            fq = heaps[r][x_off:x_off + M * K].view(M, K)
            fs = heaps[r][xs_off:xs_off + M * (K // 128) * 4].view(torch.float32).view(M, K // 128)
            fq.zero_()
            fs.zero_()
            fq[r * M_local:(r + 1) * M_local] = q
            fs[r * M_local:(r + 1) * M_local] = s
        native.ag_gemm_fp8(None, [h.data_ptr() for h in heaps], FLAG_OFF, x_off, xs_off, M, N, K, [w[0].data_ptr() for w in ws], K,
                           [w[1].data_ptr() for w in ws], K // 128, [] if quant_out else [o.data_ptr() for o in outs], N,
                           [o.data_ptr() for o in oq] if quant_out else [], [o.data_ptr() for o in os_] if quant_out else [], N,
                           0, native.GEMM_GELU_INPLACE if quant_out else 0, ready_off, epoch, 4, ctas, 0,
                           [s.data_ptr() for s in st], 0, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert all(s[0].item() == 0 for s in st), [s.tolist() for s in st]
        X = torch.cat(X)
        for r in range(world):
            ref = X @ dequant_blocks(*ws[r]).t()
            if quant_out:
                ref = torch.nn.functional.gelu(ref, approximate="tanh")
                got = dequant_rows(oq[r], os_[r])
                # e4m3 keeps 3 mantissa bits: half a unit in the last place of the block maximum
                assert (got - ref).abs().max().item() <= 0.07 * max(1.0, ref.abs().max().item())
                assert torch.allclose(os_[r], ref.view(M, N // 128, 128).abs().amax(-1) / 448.0, rtol=2e-2, atol=1e-6)
            else:
                assert (outs[r].float() - ref).abs().max().item() < 0.02 * max(1.0, ref.abs().max().item())
            gq = heaps[r][x_off:x_off + M * K].view(M, K)
            gs = heaps[r][xs_off:xs_off + M * (K // 128) * 4].view(torch.float32).view(M, K // 128)
            assert torch.equal(dequant_rows(gq, gs), X)


@pytest.mark.parametrize("world", [2, 4])
def test_ag_gemm_mx8_emulated(native, world):
    """All-gather -> GEMM on the hardware block-scaled pipeline: e4m3 rows and UE8M0 scale bytes are gathered."""
    from pccl_b200.ops.gemm import dequant_blocks, dequant_rows, quant_blocks_mx, quant_rows_mx, ue8m0_to_float
    M_local, K, N = 256, 1024, 640
    M = M_local * world
    g = torch.Generator(device="cuda").manual_seed(29)
    xs = [(torch.randn(M_local, K, generator=g, device="cuda") * (0.5 + r)).bfloat16() for r in range(world)]
    ws = [quant_blocks_mx((torch.randn(N, K, generator=g, device="cuda") * 0.1).bfloat16()) for _ in range(world)]
    x_off = DATA_OFF
    xs_off = x_off + M * K
    ready_off = xs_off + M * (K // 128)
    heaps = [torch.zeros(ready_off + 4096, dtype=torch.uint8, device="cuda") for _ in range(world)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    outs = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ctas = 148 // world
    for epoch in (1, 2):
        X = []
        for r in range(world):
            q, s = quant_rows_mx((xs[r].float() * epoch).bfloat16())
            X.append(dequant_rows(q, ue8m0_to_float(s)))
            fq = heaps[r][x_off:x_off + M * K].view(M, K)
            fs = heaps[r][xs_off:xs_off + M * (K // 128)].view(M, K // 128)
            fq.zero_()
            fs.zero_()
            fq[r * M_local:(r + 1) * M_local] = q
            fs[r * M_local:(r + 1) * M_local] = s
        native.ag_gemm_fp8(None, [h.data_ptr() for h in heaps], FLAG_OFF, x_off, xs_off, M, N, K, [w[0].data_ptr() for w in ws], K,
                           [w[1].data_ptr() for w in ws], K // 128, [o.data_ptr() for o in outs], N, [], [], 0, 0, 0, ready_off, epoch,
                           4, ctas, 0, [s.data_ptr() for s in st], 0, torch.cuda.current_stream().cuda_stream, True)
        torch.cuda.synchronize()
        assert all(s[0].item() == 0 for s in st), [s.tolist() for s in st]
        X = torch.cat(X)
        for r in range(world):
            ref = X @ dequant_blocks(ws[r][0], ue8m0_to_float(ws[r][1])).t()
            assert (outs[r].float() - ref).abs().max().item() < 0.02 * max(1.0, ref.abs().max().item())
            gs = heaps[r][xs_off:xs_off + M * (K // 128)].view(M, K // 128)
            assert torch.equal(dequant_rows(heaps[r][x_off:x_off + M * K].view(M, K), ue8m0_to_float(gs)), X)


@pytest.mark.parametrize("world,M_local", [(2, 128), (2, 256), (4, 128)])
def test_gemm_rs_fp8_emulated(native, world, M_local):
    from pccl_b200.ops.gemm import dequant_blocks, dequant_rows, quant_blocks, quant_rows
    K, N = 512, 512
    M = M_local * world
    g = torch.Generator(device="cuda").manual_seed(20)
    ys = [quant_rows((torch.randn(M, K, generator=g, device="cuda") * 0.5).bfloat16()) for _ in range(world)]
    ws = [quant_blocks((torch.randn(N, K, generator=g, device="cuda") * 0.1).bfloat16()) for _ in range(world)]
    stage_bytes = world * M_local * N * 2
    n_flags = world * (M_local // 128) * (N // 256)
    heaps = [torch.zeros(DATA_OFF + stage_bytes + n_flags * 8, dtype=torch.uint8, device="cuda") for _ in range(world)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    outs = [torch.zeros(M_local, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    total = sum(dequant_rows(*ys[r]) @ dequant_blocks(*ws[r]).t() for r in range(world))
    for epoch in (1, 2):
        native.gemm_rs_fp8(None, [h.data_ptr() for h in heaps], [y[0].data_ptr() for y in ys], K, [y[1].data_ptr() for y in ys], K // 128,
                           [w[0].data_ptr() for w in ws], K, [w[1].data_ptr() for w in ws], K // 128, [o.data_ptr() for o in outs], N,
                           M, N, K, DATA_OFF, DATA_OFF + stage_bytes, epoch, 148 // world, [s.data_ptr() for s in st], 0,
                           torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert all(s[0].item() == 0 for s in st), [s.tolist() for s in st]
        for r in range(world):
            ref = total[r * M_local:(r + 1) * M_local]
            assert (outs[r].float() - ref).abs().max().item() < 0.03 * max(1.0, ref.abs().max().item())
        for o in outs:
            o.zero_()


# ---------------------------------------------------------------------------------------------
# MoE kernels
# ---------------------------------------------------------------------------------------------
def test_fp8_quantisers_match_reference(native):
    from pccl_b200.ops.moe import quant_fp8_blocks, quant_fp8_rows
    torch.manual_seed(3)
    x = (torch.randn(300, 1024, device="cuda") * 3).bfloat16()
    q, s = quant_fp8_rows(x)
    xf = x.float().view(300, 8, 128)
    ref_s = xf.abs().amax(-1) / 448.0
    assert torch.allclose(s, ref_s, rtol=1e-6, atol=0)
    ref_q = (xf / ref_s[..., None]).to(torch.float8_e4m3fn).view(300, 1024).float()
    got_q = q.view(torch.float8_e4m3fn).float()
    # the kernel multiplies by a reciprocal: a value that sits on a rounding boundary may land one
    # fp8 step away from the divide-then-round reference, never further
    assert (got_q == ref_q).float().mean().item() > 0.999
    assert ((got_q - ref_q).abs() <= 0.0625 * ref_q.abs() + 2 ** -9).all()
    w = (torch.randn(256, 384, device="cuda")).bfloat16()
    qw, sw = quant_fp8_blocks(w)
    wf = w.float().view(2, 128, 3, 128).permute(0, 2, 1, 3)
    ref_sw = wf.abs().amax((-1, -2)) / 448.0
    assert torch.allclose(sw, ref_sw, rtol=1e-6, atol=0)
    deq = qw.view(torch.float8_e4m3fn).float().view(2, 128, 3, 128) * sw[:, None, :, None]
    assert (deq.view(256, 384) - w.float()).abs().max().item() <= 0.07 * w.float().abs().max().item()


@pytest.mark.parametrize("N,gelu", [(384, False), (512, False), (768, True)])
def test_grouped_gemm_matches_per_group_reference(native, N, gelu):
    """N = 384 takes the single-CTA row-major kernel; multiples of 256 take the CTA-pair kernel with the operands exchanged,
    whose tiles end where a group's rows end (group sizes around and off the multiples of 16 and 256)."""
    from pccl_b200.ops import check_status
    from pccl_b200.ops.moe import grouped_gemm
    torch.manual_seed(4)
    K = 512
    sizes = [130, 0, 257, 5, 128, 64, 513, 16, 300, 1]
    off = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
    total = int(off[-1])
    a = (torch.randn(total + 200, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(len(sizes) * N, K, device="cuda") * 0.1).bfloat16()
    out = torch.full((total + 200, N), 7.0, device="cuda", dtype=torch.bfloat16)
    grouped_gemm(a, b, off, N, out=out, gelu=gelu)
    check_status("grouped gemm")
    for g, n in enumerate(sizes):
        lo = int(off[g])
        ref = a[lo:lo + n].float() @ b[g * N:(g + 1) * N].float().t()
        if gelu:
            ref = torch.nn.functional.gelu(ref, approximate="tanh")
        assert (out[lo:lo + n].float() - ref).abs().max().item() < 0.05 if n else True
    assert torch.all(out[total:] == 7.0)        # rows past the last group are untouched


def test_moe_dispatch_combine_emulated(native):
    """Two emulated ranks: fp8 dispatch lands in the right rows with the right scales; combine pulls
    rows back from both ranks and weights them."""
    world, T, H, Kt, epr = 2, 64, 256, 2, 2
    cap = 512
    q_off, s_off, y_off = DATA_OFF, DATA_OFF + cap * H, DATA_OFF + cap * H + cap * (H // 128) * 4
    heaps = [torch.zeros(y_off + cap * H * 2, dtype=torch.uint8, device="cuda") for _ in range(world)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    g = torch.Generator(device="cuda").manual_seed(5)
    xs = [(torch.randn(T, H, generator=g, device="cuda") * 2).bfloat16() for _ in range(world)]
    ids = [torch.randint(0, world * epr, (T, Kt), generator=g, device="cuda", dtype=torch.int32) for _ in range(world)]
    # every (rank, token, k) gets a unique row on its destination: rank r uses rows r*T*Kt + t*Kt + k
    rows = [(torch.arange(T * Kt, device="cuda", dtype=torch.int32) + r * T * Kt).view(T, Kt).contiguous() for r in range(world)]
    probs = [torch.rand(T, Kt, generator=g, device="cuda") for _ in range(world)]
    outs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    stream = torch.cuda.current_stream().cuda_stream
    native.moe_exchange("dispatch", None, [h.data_ptr() for h in heaps], FLAG_OFF, T, H, Kt, epr, q_off, s_off, y_off, 1, 0,
                        [x.data_ptr() for x in xs], [i.data_ptr() for i in ids], [r.data_ptr() for r in rows], [], [],
                        [s.data_ptr() for s in st], 8, 0, stream)
    torch.cuda.synchronize()
    assert all(s[0].item() == 0 for s in st)
    from pccl_b200.ops.moe import quant_fp8_rows
    for r in range(world):
        q_ref, s_ref = quant_fp8_rows(xs[r])
        for t in range(0, T, 7):
            for k in range(Kt):
                d, row = int(ids[r][t, k]) // epr, int(rows[r][t, k])
                got_q = heaps[d][q_off + row * H: q_off + (row + 1) * H]
                got_s = heaps[d][s_off + row * (H // 128) * 4: s_off + (row + 1) * (H // 128) * 4].view(torch.float32)
                assert torch.equal(got_q, q_ref[t]) and torch.equal(got_s, s_ref[t])
    # expert outputs: fill y on both ranks with a known function of (rank, row)
    ys = []
    for d in range(world):
        y = heaps[d][y_off:y_off + cap * H * 2].view(torch.bfloat16).view(cap, H)
        y.copy_((torch.randn(cap, H, generator=g, device="cuda")).bfloat16())
        ys.append(y)
    native.moe_exchange("combine", None, [h.data_ptr() for h in heaps], FLAG_OFF, T, H, Kt, epr, q_off, s_off, y_off, 2, 0,
                        [], [i.data_ptr() for i in ids], [r.data_ptr() for r in rows], [p.data_ptr() for p in probs],
                        [o.data_ptr() for o in outs], [s.data_ptr() for s in st], 8, 0, stream)
    torch.cuda.synchronize()
    assert all(s[0].item() == 0 for s in st)
    for r in range(world):
        ref = torch.zeros(T, H, device="cuda")
        for k in range(Kt):
            d = (ids[r][:, k] // epr).long()
            picked = torch.stack([ys[int(d[t])][int(rows[r][t, k])] for t in range(T)]).float()
            ref += probs[r][:, k, None] * picked
        assert (outs[r].float() - ref).abs().max().item() < 0.05


def test_moe_deduplicated_exchange_emulated(native):
    """Two emulated ranks, four assignments per token over four experts: most tokens have several assignments on one
    rank.  The dispatch sends the row once per rank and tells the others where it is; the conversion to bf16 fills every
    row; the ranks add up each token's weighted expert outputs locally and the combine pulls one row per rank."""
    world, T, H, Kt, epr = 2, 64, 256, 4, 2
    cap = 1024
    G = H // 128
    q_off = DATA_OFF
    s_off = q_off + cap * H
    y_off = s_off + cap * G * 4
    alias_off = y_off + cap * H * 2
    group_off = alias_off + cap * 4
    z_off = group_off + cap * 64
    heaps = [torch.zeros(z_off + cap * H * 2, dtype=torch.uint8, device="cuda") for _ in range(world)]
    st = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(world)]
    g = torch.Generator(device="cuda").manual_seed(15)
    xs = [(torch.randn(T, H, generator=g, device="cuda") * 2).bfloat16() for _ in range(world)]
    ids = [torch.randint(0, world * epr, (T, Kt), generator=g, device="cuda", dtype=torch.int32) for _ in range(world)]
    ids[0][3, 1] = -1                                   # a dropped assignment takes no part in any group
    rows = [(torch.arange(T * Kt, device="cuda", dtype=torch.int32) + r * T * Kt).view(T, Kt).contiguous() for r in range(world)]
    probs = [torch.rand(T, Kt, generator=g, device="cuda") for _ in range(world)]
    outs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    stream = torch.cuda.current_stream().cuda_stream
    hp = [h.data_ptr() for h in heaps]
    native.moe_exchange("dispatch", None, hp, FLAG_OFF, T, H, Kt, epr, q_off, s_off, y_off, 1, 0,
                        [x.data_ptr() for x in xs], [i.data_ptr() for i in ids], [r.data_ptr() for r in rows], [], [],
                        [s.data_ptr() for s in st], 8, 0, stream, alias_off=alias_off, group_off=group_off, z_off=z_off,
                        gate=[p.data_ptr() for p in probs], dedupe=True)
    torch.cuda.synchronize()
    assert all(s[0].item() == 0 for s in st)
    from pccl_b200.ops.moe import quant_fp8_rows
    n_rows = torch.tensor([world * T * Kt], dtype=torch.int32, device="cuda")
    sent = skipped = 0
    xb = []
    for d in range(world):
        out = torch.zeros(cap, H, dtype=torch.bfloat16, device="cuda")
        native.moe_dequant(heaps[d].data_ptr() + q_off, heaps[d].data_ptr() + s_off, out.data_ptr(), n_rows.data_ptr(), cap, H, stream,
                           alias=heaps[d].data_ptr() + alias_off)
        xb.append(out)
    torch.cuda.synchronize()
    for r in range(world):
        q_ref, s_ref = quant_fp8_rows(xs[r])
        deq = (q_ref.view(torch.float8_e4m3fn).float().view(T, G, 128) * s_ref.view(T, G, 1)).view(T, H).bfloat16()
        for t in range(T):
            seen = set()
            for k in range(Kt):
                e = int(ids[r][t, k])
                if e < 0:
                    continue
                d, row = e // epr, int(rows[r][t, k])
                payload = heaps[d][q_off + row * H: q_off + (row + 1) * H]
                if d in seen:
                    skipped += 1
                    assert not payload.any()                      # never sent
                else:
                    sent += 1
                    assert torch.equal(payload, q_ref[t])
                seen.add(d)
                assert torch.equal(xb[d][row], deq[t]), (r, t, k)   # every row is there after the conversion
    assert skipped > T and sent > T
    ys = []
    for d in range(world):
        y = heaps[d][y_off:y_off + cap * H * 2].view(torch.bfloat16).view(cap, H)
        y.copy_((torch.randn(cap, H, generator=g, device="cuda")).bfloat16())
        ys.append(y)
        native.moe_reduce_groups(heaps[d].data_ptr() + y_off, heaps[d].data_ptr() + z_off, heaps[d].data_ptr() + alias_off,
                                 heaps[d].data_ptr() + group_off, n_rows.data_ptr(), cap, H, stream)
    native.moe_exchange("combine", None, hp, FLAG_OFF, T, H, Kt, epr, q_off, s_off, y_off, 2, 0,
                        [], [i.data_ptr() for i in ids], [r.data_ptr() for r in rows], [p.data_ptr() for p in probs],
                        [o.data_ptr() for o in outs], [s.data_ptr() for s in st], 8, 0, stream, alias_off=alias_off,
                        group_off=group_off, z_off=z_off, dedupe=True)
    torch.cuda.synchronize()
    assert all(s[0].item() == 0 for s in st)
    for r in range(world):
        ref = torch.zeros(T, H, device="cuda")
        for t in range(T):
            for k in range(Kt):
                e = int(ids[r][t, k])
                if e >= 0:
                    ref[t] += probs[r][t, k] * ys[e // epr][int(rows[r][t, k])].float()
        assert (outs[r].float() - ref).abs().max().item() < 0.06, r


def test_moe_layer_world_of_one_matches_dense_reference(native):
    from pccl_b200.engine import Engine
    from pccl_b200.ops import check_status
    from pccl_b200.ops.moe import MoEExchange
    torch.manual_seed(6)
    T, H, F, E, Kt = 256, 512, 256, 8, 2
    eng = Engine(0, 1)
    eng.initEngine("cuda", heap_bytes=512 << 20)
    moe = MoEExchange(eng, T, H, E, Kt)
    x = torch.randn(T, H, device="cuda").bfloat16()
    logits = torch.randn(T, E, device="cuda")
    w1 = (torch.randn(E * F, H, device="cuda") * 0.05).bfloat16()
    w2 = (torch.randn(E * H, F, device="cuda") * 0.05).bfloat16()
    out = moe.forward(x, logits, w1, w2)
    check_status("moe")
    ids, probs = MoEExchange.route(logits, Kt)
    ref = torch.zeros(T, H, device="cuda")
    xq = x.float().view(T, H // 128, 128)
    sc = xq.abs().amax(-1, keepdim=True) / 448.0
    xd = ((xq / sc).to(torch.float8_e4m3fn).float() * sc).view(T, H).bfloat16().float()   # what the experts see
    for e in range(E):
        h = torch.nn.functional.gelu(xd @ w1[e * F:(e + 1) * F].float().t(), approximate="tanh").bfloat16().float()
        y = (h @ w2[e * H:(e + 1) * H].float().t()).bfloat16().float()
        for k in range(Kt):
            m = (ids[:, k] == e)
            ref[m] += probs[m, k, None] * y[m]
    assert (out.float() - ref).abs().max().item() < 0.03 * max(1.0, ref.abs().max().item())
    del moe, eng


def test_moe_route_and_plan_kernels_match_tensor_ops(native):
    from pccl_b200.engine import Engine
    from pccl_b200.ops.moe import MoEExchange
    torch.manual_seed(8)
    T, H, E, Kt = 1000, 256, 64, 6
    eng = Engine(0, 1); eng.initEngine("cuda", heap_bytes=256 << 20)
    moe = MoEExchange(eng, T, H, E, Kt)
    logits = torch.randn(T, E, device="cuda")
    ids, probs, plan = moe.route_and_plan(logits)
    ref_ids, ref_probs = MoEExchange.route(logits, Kt)
    ref_plan = moe.plan(ref_ids)
    assert torch.equal(ids, ref_ids)
    assert torch.allclose(probs, ref_probs, rtol=1e-4, atol=1e-7)
    assert torch.equal(plan["row_off"], ref_plan["row_off"])
    # rows are a permutation within each expert's segment: same multiset per expert, all distinct
    rows, ref_rows = plan["rows"].view(-1).long(), ref_plan["rows"].view(-1).long()
    assert rows.unique().numel() == rows.numel()
    off = plan["row_off"].long()
    flat = ids.view(-1).long()
    assert ((rows >= off[flat]) & (rows < off[flat + 1])).all()
    assert torch.equal(rows.sort().values, ref_rows.sort().values)
    del moe, eng


@pytest.mark.parametrize("algo", ["ring_allreduce", "direct_allreduce", "direct_reduce_scatter", "direct_allgather", "alltoall"])
def test_engine_regop_exeop_on_a_cuda_engine_with_alternating_widths(native, algo):
    """The public path initEngine("cuda") -> regOp -> exeOp on a world of one: the program is materialised per width,
    every (program, width) pair gets its own signal words and launch count, the scratch half alternates per launch, and
    the interpreter kernel runs it on the GPU.  A world of one keeps every wait inside one launch."""
    from pccl_b200.engine import Engine
    from pccl_b200.lang import build
    eng = Engine(0, 1)
    eng.initEngine("cuda", heap_bytes=512 << 20)       # the default 256 MiB workspace and some room for tensors
    eng.regOp("op", build(algo, 1, channels=2))
    n = 3 * 8192 + 16
    for it, width in enumerate([1, 4, 1, 4, 2, 4]):
        x = torch.arange(n, device="cuda", dtype=torch.float32) + it
        y = torch.full((n,), -1.0, device="cuda")
        eng.exeOp("op", x, y, width=width, check=True)
        assert torch.equal(y, x), (algo, it, width)
    st = eng.stats()
    assert st["ops"]["op"]["launches"] == 6 and st["device"] == "cuda" and st["signals_used"] > 0
    # a symmetric (heap) tensor works as well, and in place
    z = eng.symmetric_tensor((n,), torch.float32)
    z.copy_(torch.arange(n, device="cuda", dtype=torch.float32))
    if algo.endswith("allreduce"):
        eng.exeOp("op", z, width=2, check=True)
        assert torch.equal(z, torch.arange(n, device="cuda", dtype=torch.float32))
    del eng


def test_resident_executor_takes_queued_launches_without_a_kernel_launch_each(native):
    """startResident -> enqueue x N -> wait: the interpreter kernel stays on the GPU and takes its work from a queue in
    pinned host memory (a world of one keeps every wait inside the one kernel).  It leaves by itself when idle and is
    started again by the next submission."""
    import time
    from pccl_b200.engine import Engine
    from pccl_b200.lang import build
    eng = Engine(0, 1)
    eng.initEngine("cuda", heap_bytes=512 << 20)
    eng.regOp("ar", build("ring_allreduce", 1, channels=2))
    eng.regOp("ag", build("direct_allgather", 1, channels=1))
    eng.start_resident(width=2)
    n = 64 * 1024
    xs = [torch.arange(n, device="cuda", dtype=torch.float32) + i for i in range(24)]
    ys = [torch.full((n,), -1.0, device="cuda") for _ in range(24)]
    torch.cuda.current_stream().synchronize()
    t0 = time.perf_counter()
    tickets = [eng.enqueue("ar" if i % 3 else "ag", xs[i], ys[i], sync_inputs=False) for i in range(24)]
    eng.wait(tickets[-1], timeout_ms=20000)
    per_op_us = (time.perf_counter() - t0) / 24 * 1e6
    for i in range(24):
        assert torch.equal(ys[i], xs[i]), i
    st = eng.stats()
    assert st["resident_ops"] == 24 and st["resident_kernel_launches"] >= 1
    first_launches = st["resident_kernel_launches"]
    assert first_launches <= 3, st            # not one launch per operation
    assert eng.check_status(0)[0] == 0
    # idle: the kernel leaves (a device-wide synchronize returns), the next submission brings it back
    time.sleep(0.1)
    torch.cuda.synchronize()
    y = torch.zeros(n, device="cuda")
    eng.wait(eng.enqueue("ar", xs[3], y), timeout_ms=20000)
    assert torch.equal(y, xs[3])
    assert eng.stats()["resident_kernel_launches"] > first_launches
    eng.stop_resident()
    eng.exeOp("ar", xs[5], y, check=True)          # the launch-per-call path still works afterwards
    assert torch.equal(y, xs[5])
    print(f"resident executor: {per_op_us:.1f} us per queued operation (host clock, 24 operations)")
    del eng


def test_moe_layer_backward_matches_dense_reference(native):
    """The expert-parallel layer as an autograd node (world of one): gradients of the input, the gate logits and both
    expert weights against a dense fp32 reference that sees the same e4m3 round trips as the kernels."""
    from pccl_b200.engine import Engine
    from pccl_b200.ops import check_status
    from pccl_b200.ops.moe import MoEExchange
    from pccl_b200.parallel.ep import _MoEFn
    torch.manual_seed(16)
    T, H, Fd, E, Kt = 256, 512, 256, 8, 2
    eng = Engine(0, 1)
    eng.initEngine("cuda", heap_bytes=512 << 20)
    moe = MoEExchange(eng, T, H, E, Kt)
    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True)
    logits = torch.randn(T, E, device="cuda").requires_grad_(True)
    w1 = (torch.randn(E * Fd, H, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    w2 = (torch.randn(E * H, Fd, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    g = (torch.randn(T, H, device="cuda") * 0.1).bfloat16()
    out = _MoEFn.apply(x, logits, w1, w2, moe)
    out.backward(g)
    check_status("moe backward")

    def e4m3_round_trip(t):      # what a row looks like after the dispatch (1 x 128 blocks)
        q = t.view(t.shape[0], -1, 128)
        sc = (q.abs().amax(-1, keepdim=True) / 448.0).clamp_min(1e-30)
        return ((q / sc).to(torch.float8_e4m3fn).float() * sc).view_as(t)

    xr = x.detach().float().requires_grad_(True)
    lr = logits.detach().float().requires_grad_(True)
    w1r, w2r = w1.detach().float().requires_grad_(True), w2.detach().float().requires_grad_(True)
    pf = torch.softmax(lr, -1)
    p, ids = pf.topk(Kt, -1)
    xs = xr + (e4m3_round_trip(xr.detach()) - xr.detach())            # straight-through: forward sees the quantised rows
    ref = torch.zeros(T, H, device="cuda")
    for e in range(E):
        y = torch.nn.functional.gelu(xs @ w1r[e * Fd:(e + 1) * Fd].t(), approximate="tanh") @ w2r[e * H:(e + 1) * H].t()
        for k in range(Kt):
            m = (ids[:, k] == e).float()[:, None]
            ref = ref + m * p[:, k, None] * y
    ref.backward(g.float())
    assert (out.float() - ref.detach()).abs().max().item() < 0.03 * max(1.0, ref.abs().max().item())
    for got, want, name, tol in ((x.grad, xr.grad, "dx", 0.08), (logits.grad, lr.grad, "dlogits", 0.08), (w1.grad, w1r.grad, "dw1", 0.08),
                                 (w2.grad, w2r.grad, "dw2", 0.08)):
        err = (got.float() - want).abs().max().item()
        assert err <= tol * max(1e-6, want.abs().max().item()), (name, err, want.abs().max().item())
    del moe, eng


def test_run_time_compiled_program_launches_and_mixes_with_the_interpreter(native):
    """JitOp on a world of one: the generated kernel (NVRTC -> cubin -> driver launch) gives the program's result, at two
    widths and two sizes, interleaved with interpreter launches of the same program on the same lane."""
    from pccl_b200.engine import Engine
    from pccl_b200.jit import JitOp
    from pccl_b200.lang import build
    eng = Engine(0, 1)
    eng.initEngine("cuda", heap_bytes=512 << 20)
    eng.regOp("ar", build("ring_allreduce", 1, channels=2))
    eng.regOp("ag", build("direct_allgather", 1, channels=1))
    ar, ag = JitOp(eng, "ar"), JitOp(eng, "ag")
    for it, (n, width) in enumerate([(4096, 1), (4096, 2), (3 * 8192 + 16, 2), (4096, 1)]):
        x = torch.arange(n, device="cuda", dtype=torch.float32) + it
        y = torch.full((n,), -1.0, device="cuda")
        ar(x, y, width=width)
        torch.cuda.synchronize()
        assert torch.equal(y, x), (it, n, width)
        y.fill_(-1)
        eng.exeOp("ar", x, y, width=width, check=True)          # the interpreter on the same signal range and lane
        assert torch.equal(y, x)
        g = torch.zeros(n, device="cuda")
        ag(x, g)
        torch.cuda.synchronize()
        assert torch.equal(g, x)
    assert ar.compiled == 3 and eng.check_status(0)[0] == 0      # (4096, 1) was compiled once
    xb = torch.randn(8192, device="cuda").bfloat16()
    yb = torch.zeros_like(xb)
    ar(xb, yb, width=2)
    torch.cuda.synchronize()
    assert torch.equal(xb, yb)
    del ar, ag, eng
