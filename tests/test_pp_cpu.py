"""Pipeline schedules on CPU ranks over gloo: the one-forward-one-backward training step gives every stage the
gradients that the whole model gets on one process."""
import pytest
import torch

from _ranks import run_ranks


def _stages(world, width):
    torch.manual_seed(11)
    return [torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.Tanh()) for _ in range(world)]


def _pp_rank(rank, world, port, n_micro):
    import torch
    import torch.distributed as dist
    from pccl_b200.parallel.pp import PipelineP2P
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        width, rows = 16, 5
        stage = _stages(world, width)[rank]
        g = torch.Generator().manual_seed(3)
        xs = [torch.randn(rows, width, generator=g) for _ in range(n_micro)]
        ts = [torch.randn(rows, width, generator=g) for _ in range(n_micro)]
        pp = PipelineP2P()
        losses = pp.run_1f1b(stage, n_micro, inputs=xs if rank == 0 else None, in_shape=(rows, width), out_shape=(rows, width),
                             loss_fn=(lambda y, i: ((y - ts[i]) ** 2).mean() / n_micro) if rank == world - 1 else None,
                             dtype=torch.float32)
        outs = pp.run_gpipe(lambda x: stage(x).detach(), xs, (rows, width), torch.float32)      # forward-only schedule
        return ([p.grad.tolist() for p in stage.parameters()], [float(v) for v in losses], outs[-1].tolist())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_micro", [(3, 5), (2, 1), (4, 2)])
def test_1f1b_matches_the_whole_model_on_one_process(world, n_micro):
    res = run_ranks(_pp_rank, world, args=(n_micro,), timeout=180)
    width, rows = 16, 5
    stages = _stages(world, width)
    g = torch.Generator().manual_seed(3)
    xs = [torch.randn(rows, width, generator=g) for _ in range(n_micro)]
    ts = [torch.randn(rows, width, generator=g) for _ in range(n_micro)]
    want_losses = []
    for x, t in zip(xs, ts):
        y = x
        for st in stages:
            y = st(y)
        loss = ((y - t) ** 2).mean() / n_micro
        loss.backward()
        want_losses.append(float(loss.detach()))
    for r in range(world):
        grads, losses, last_out = res[r]
        for got, p in zip(grads, stages[r].parameters()):
            assert torch.allclose(torch.tensor(got), p.grad, atol=1e-6), r
        assert losses == (pytest.approx(want_losses, abs=1e-7) if r == world - 1 else [])
    y = xs[-1]
    for st in stages:
        y = st(y)
    assert torch.allclose(torch.tensor(res[world - 1][2]), y.detach(), atol=1e-6)
