"""The GPT model on this package's kernels against the same network written with stock PyTorch ops
in fp32, and the sharded data-parallel step with a world of one."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _reference_loss(model, ids, targets):
    """Same weights, fp32 math, stock ops."""
    cfg = model.cfg
    f = lambda t: t.detach().float().requires_grad_(True)  # noqa: E731
    P = {n: f(p) for n, p in model.named_parameters()}
    B, T = ids.shape
    x = P["wte.weight"][ids] + P["wpe.weight"][torch.arange(T, device=ids.device)][None]
    for i in range(cfg.n_layer):
        g = lambda n: P[f"blocks.{i}.{n}"]  # noqa: E731
        h = F.layer_norm(x, (cfg.d_model,), g("ln1.weight"), g("ln1.bias"))
        qkv = F.linear(h, g("qkv.weight"), g("qkv.bias")).view(B, T, 3, cfg.n_head, -1)
        q, k, v = (qkv[:, :, j].transpose(1, 2) for j in range(3))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, -1)
        x = x + F.linear(a, g("proj.weight"), g("proj.bias"))
        h = F.layer_norm(x, (cfg.d_model,), g("ln2.weight"), g("ln2.bias"))
        x = x + F.linear(F.gelu(F.linear(h, g("fc1.weight"), g("fc1.bias")), approximate="tanh"), g("fc2.weight"), g("fc2.bias"))
    x = F.layer_norm(x, (cfg.d_model,), P["ln_f.weight"], P["ln_f.bias"])
    loss = F.cross_entropy(F.linear(x, P["wte.weight"]).view(B * T, -1), targets.reshape(-1))
    loss.backward()
    return loss.item(), {n: p.grad for n, p in P.items()}


def test_gpt_forward_backward_matches_fp32_reference():
    from pccl_b200.models import GPT, GPTConfig
    from pccl_b200.ops import check_status
    torch.manual_seed(0)
    cfg = GPTConfig.tiny()
    model = GPT(cfg, device="cuda")
    ids = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len), device="cuda")
    tgt = ids.roll(-1, 1)
    loss = model(ids, tgt)
    loss.backward()
    check_status("gpt")
    ref_loss, ref_grads = _reference_loss(model, ids, tgt)
    assert abs(loss.item() - ref_loss) < 0.02 * ref_loss
    for name in ("blocks.0.qkv.weight", "blocks.1.fc1.weight", "blocks.1.fc2.weight", "blocks.0.proj.bias", "wte.weight",
                 "wpe.weight", "blocks.1.ln2.weight", "blocks.0.fc1.bias", "blocks.1.fc2.bias", "blocks.0.fc2.bias", "blocks.1.qkv.bias",
                 "blocks.0.ln1.weight", "ln_f.bias"):
        got = dict(model.named_parameters())[name].grad.float()
        ref = ref_grads[name]
        denom = ref.abs().max().item() + 1e-8
        assert (got - ref).abs().max().item() / denom < 0.08, name


def test_fused_cross_entropy_matches_torch():
    from pccl_b200.nn import fused_cross_entropy
    torch.manual_seed(1)
    rows, vocab, ld = 300, 50257, 50264
    store = (torch.randn(rows, ld, device="cuda") * 3).bfloat16()
    logits = store[:, :vocab]
    tgt = torch.randint(0, vocab, (rows,), device="cuda")
    ref_in = logits.float().clone().requires_grad_(True)
    ref = F.cross_entropy(ref_in, tgt)
    ref.backward()
    x = logits.clone().as_strided(logits.shape, logits.stride()) if False else store.clone()[:, :vocab]
    x.requires_grad_(True)
    loss = fused_cross_entropy(x, tgt)
    loss.backward()
    assert abs(loss.item() - ref.item()) < 1e-3
    assert (x.grad.float() - ref_in.grad).abs().max().item() < 2e-5 + 0.01 * ref_in.grad.abs().max().item()


def test_cross_entropy_reports_a_target_outside_the_vocabulary_instead_of_indexing_with_it():
    """An out-of-range target is never used as an index: its row gets loss 0 and a zero gradient, the first such
    row is written to the device status words, and ``ignore_index`` itself stays silent."""
    from pccl_b200.ops import check_status
    from pccl_b200.ops.elementwise import cross_entropy_
    import pytest as _pt
    torch.manual_seed(5)
    rows, vocab = 32, 512
    x = (torch.randn(rows, vocab, device="cuda") * 2).bfloat16()
    tgt = torch.randint(0, vocab, (rows,), device="cuda")
    tgt[5] = -100
    check_status("before")
    quiet = cross_entropy_(x.clone(), tgt, grad_scale=1.0, ignore_index=-100)
    check_status("ignore_index is not an error")
    assert quiet[5].item() == 0.0
    tgt[9] = vocab + 3
    y = x.clone()
    loss = cross_entropy_(y, tgt, grad_scale=1.0, ignore_index=-100)
    assert loss[9].item() == 0.0 and int(y[9].abs().sum()) == 0 and loss[8].item() > 0.0
    with _pt.raises(RuntimeError, match="device status"):
        check_status("cross entropy with a bad target")
    check_status("cleared")


def test_adamw_kernel_matches_torch():
    from pccl_b200.ops.elementwise import adamw_step
    torch.manual_seed(2)
    n = 100003
    p = torch.randn(n, device="cuda"); g = torch.randn(n, device="cuda") * 0.1
    ref_p = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v, out = torch.zeros_like(p), torch.zeros_like(p), torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in (1, 2, 3):
        ref_p.grad = g.clone() * step
        opt.step()
        adamw_step(p, m, v, g * step, out, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, step=step)
    assert (p - ref_p.detach()).abs().max().item() < 1e-5
    assert torch.equal(out, p.bfloat16())


def test_sharded_dp_world_of_one_trains_and_matches_plain_adamw():
    from pccl_b200.models import GPT, GPTConfig
    from pccl_b200.models.gpt import smoke_step
    from pccl_b200.ops import check_status, launch_count
    before = launch_count()
    last = smoke_step()
    check_status("dp")
    assert math.isfinite(last) and launch_count() - before > 50


def test_fused_and_unfused_optimizer_paths_agree():
    """Reduce-scatter + AdamW in one kernel gives the parameters of the two-kernel path."""
    from pccl_b200.engine import Engine
    from pccl_b200.models import GPT, GPTConfig
    from pccl_b200.parallel import ShardedDataParallel
    cfg = GPTConfig.tiny()
    ids = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    flats = []
    for fused in (True, False):
        torch.manual_seed(0)
        model = GPT(cfg, device="cuda")
        eng = Engine(0, 1); eng.initEngine("cuda", heap_bytes=256 << 20)
        dp = ShardedDataParallel(model, eng, lr=1e-3, bucket_mb=0.5, fuse_optimizer=fused)
        for _ in range(2):
            dp.train_step(ids, ids.roll(-1, 1))
        torch.cuda.synchronize()
        flats.append(dp.flat_params.float().clone())
        del dp, model, eng
    assert (flats[0] - flats[1]).abs().max().item() <= 2e-2 * flats[1].abs().max().item()
    assert (flats[0] == flats[1]).float().mean().item() > 0.9       # identical except where atomics order / bf16 rounding of a gradient differs


def test_timed_step_reports_every_bucket_and_trains_like_train_step():
    """The opt-in per-bucket timing takes the same step as train_step and returns ordered, non-negative spans."""
    from pccl_b200.engine import Engine
    from pccl_b200.models import GPT, GPTConfig
    from pccl_b200.parallel import ShardedDataParallel
    cfg = GPTConfig.tiny()
    ids = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    flats = []
    for timed in (False, True):
        torch.manual_seed(0)
        model = GPT(cfg, device="cuda")
        eng = Engine(0, 1); eng.initEngine("cuda", heap_bytes=256 << 20)
        dp = ShardedDataParallel(model, eng, lr=1e-3, bucket_mb=0.5)
        dp.train_step(ids, ids.roll(-1, 1))
        if timed:
            rep = dp.timed_step(ids, ids.roll(-1, 1))
            assert len(rep["buckets"]) == len(dp.buckets) and math.isfinite(rep["loss"])
            assert 0 < rep["forward_end"] < rep["backward_end"] <= rep["step_end"]
            for row in rep["buckets"]:
                assert row["ready"] <= row["start"] + 1e-3 and row["start"] <= row["reduced"] <= row["done"] <= rep["step_end"] + 1e-3
            assert rep["exposed_ms"] >= 0 and rep["comm_busy_ms"] > 0
        else:
            dp.train_step(ids, ids.roll(-1, 1))
        torch.cuda.synchronize()
        flats.append(dp.flat_params.float().clone())
        del dp, model, eng
    assert (flats[0] - flats[1]).abs().max().item() <= 2e-2 * flats[1].abs().max().item()


def test_dp_checkpoint_resume_matches_uninterrupted_training(tmp_path):
    """torch.save of the sharded optimizer state and flat parameters after two steps, loaded into a differently
    initialised trainer, continues like the run that was never interrupted."""
    from pccl_b200.engine import Engine
    from pccl_b200.models import GPT, GPTConfig
    from pccl_b200.parallel import ShardedDataParallel
    cfg = GPTConfig.tiny()
    ids = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))

    def make(seed):
        torch.manual_seed(seed)
        model = GPT(cfg, device="cuda")
        eng = Engine(0, 1); eng.initEngine("cuda", heap_bytes=256 << 20)
        return model, eng, ShardedDataParallel(model, eng, lr=1e-3, bucket_mb=0.5)

    model, eng, dp = make(0)
    for _ in range(2):
        dp.train_step(ids, ids.roll(-1, 1))
    torch.cuda.synchronize()
    torch.save(dp.gather_full_state(), tmp_path / "ckpt.pt")
    for _ in range(2):
        last = float(dp.train_step(ids, ids.roll(-1, 1)))
    torch.cuda.synchronize()
    want = dp.flat_params.float().clone()
    del dp, model, eng
    model, eng, dp = make(1)            # other initial weights: everything has to come from the checkpoint
    dp.load_full_state(torch.load(tmp_path / "ckpt.pt"))
    assert dp.step_count == 2
    for _ in range(2):
        resumed = float(dp.train_step(ids, ids.roll(-1, 1)))
    torch.cuda.synchronize()
    got = dp.flat_params.float()
    assert abs(resumed - last) <= 2e-2 * abs(last), (resumed, last)
    assert (got - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    assert (got == want).float().mean().item() > 0.9


@pytest.mark.parametrize("rows,D", [(37, 256), (4096, 2048), (600, 4096), (130, 8192)])
def test_layernorm_kernels_match_fp32_reference(rows, D):
    from pccl_b200.nn import LayerNorm
    torch.manual_seed(5)
    ln = LayerNorm(D, device="cuda")
    with torch.no_grad():
        ln.weight.copy_((torch.randn(D, device="cuda") * 0.5 + 1).bfloat16())
        ln.bias.copy_((torch.randn(D, device="cuda") * 0.1).bfloat16())
    x = (torch.randn(rows, D, device="cuda") * 2 + 0.5).bfloat16().requires_grad_(True)
    g = torch.randn(rows, D, device="cuda").bfloat16()
    y = ln(x)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = ln.weight.detach().float().requires_grad_(True)
    br = ln.bias.detach().float().requires_grad_(True)
    yr = F.layer_norm(xr, (D,), wr, br, 1e-5)
    yr.backward(g.float())
    assert ((y.float() - yr).abs() <= 0.01 + 0.008 * yr.abs()).all()       # one bf16 rounding of the output
    assert (x.grad.float() - xr.grad).abs().max().item() < 0.03 * max(1.0, xr.grad.abs().max().item())
    assert (ln.weight.grad.float() - wr.grad).abs().max().item() < 0.02 * max(1.0, wr.grad.abs().max().item())
    assert (ln.bias.grad.float() - br.grad).abs().max().item() < 0.02 * max(1.0, br.grad.abs().max().item())


@pytest.mark.parametrize("rows,D", [(512, 2048), (300, 256), (64, 4096)])
def test_fused_residual_add_layernorm_matches_fp32_reference(rows, D):
    """(x, delta) -> (x + delta, LN(x + delta)) forward, and backward with the gradient on the residual stream added in
    and the producing layer's bias gradient (column sums of d delta) as a by-product."""
    from pccl_b200.nn import LayerNorm
    torch.manual_seed(7)
    ln = LayerNorm(D, device="cuda")
    with torch.no_grad():
        ln.weight.copy_((1 + 0.1 * torch.randn(D, device="cuda")).bfloat16())
        ln.bias.copy_((0.1 * torch.randn(D, device="cuda")).bfloat16())
    x = torch.randn(rows, D, device="cuda").bfloat16().requires_grad_(True)
    delta = torch.randn(rows, D, device="cuda").bfloat16().requires_grad_(True)
    prev_bias = torch.zeros(D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    s, y = ln.add_norm(x, delta, prev_bias)
    gs, gy = torch.randn(rows, D, device="cuda").bfloat16(), torch.randn(rows, D, device="cuda").bfloat16()
    torch.autograd.backward([s, y], [gs, gy])
    xr, dr = x.detach().float().requires_grad_(True), delta.detach().float().requires_grad_(True)
    wr, br = ln.weight.detach().float().requires_grad_(True), ln.bias.detach().float().requires_grad_(True)
    # the norm sees the stored (bf16-rounded) sum; gradients pass straight through the rounding
    sr = (xr + dr) + ((xr + dr).detach().bfloat16().float() - (xr + dr).detach())
    yr = F.layer_norm(sr, (D,), wr, br, ln.eps)
    torch.autograd.backward([sr, yr], [gs.float(), gy.float()])
    assert (s.float() - sr).abs().max().item() <= 1e-6
    assert (y.float() - yr).abs().max().item() <= 3e-2
    tol = 3e-2 * max(1.0, xr.grad.abs().max().item())
    assert (x.grad.float() - xr.grad).abs().max().item() <= tol
    assert x.grad.data_ptr() == delta.grad.data_ptr() or torch.equal(x.grad, delta.grad)
    for got, ref in ((ln.weight.grad, wr.grad), (ln.bias.grad, br.grad), (prev_bias.grad, dr.grad.sum(0))):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())


def test_fused_mlp_backward_matches_fp32_reference():
    """fc2(gelu(fc1(x))) as one autograd node (GELU derivative and first bias gradient inside the GEMM epilogue)."""
    from pccl_b200.nn import Linear, mlp
    torch.manual_seed(8)
    rows, d, h = 512, 256, 1024
    fc1, fc2 = Linear(d, h, device="cuda"), Linear(h, d, device="cuda")
    with torch.no_grad():
        fc1.bias.copy_((0.1 * torch.randn(h, device="cuda")).bfloat16())
        fc2.bias.copy_((0.1 * torch.randn(d, device="cuda")).bfloat16())
    x = torch.randn(rows, d, device="cuda").bfloat16().requires_grad_(True)
    g = torch.randn(rows, d, device="cuda").bfloat16()
    mlp(x, fc1, fc2).backward(g)
    xr = x.detach().float().requires_grad_(True)
    P = {n: p.detach().float().requires_grad_(True) for n, p in (("w1", fc1.weight), ("b1", fc1.bias), ("w2", fc2.weight), ("b2", fc2.bias))}
    out = F.linear(F.gelu(F.linear(xr, P["w1"], P["b1"]), approximate="tanh"), P["w2"], P["b2"])
    out.backward(g.float())
    for got, ref, name in ((x.grad, xr.grad, "dx"), (fc1.weight.grad, P["w1"].grad, "dw1"), (fc1.bias.grad, P["b1"].grad, "db1"),
                           (fc2.weight.grad, P["w2"].grad, "dw2"), (fc2.bias.grad, P["b2"].grad, "db2")):
        assert (got.float() - ref).abs().max().item() <= 5e-2 * max(1e-3, ref.abs().max().item()), name
    # the second bias gradient can be left to the consumer of the output
    fc2.bias.grad = None
    mlp(x, fc1, fc2, defer_fc2_bias_grad=True).backward(g)
    assert fc2.bias.grad is None
