#!/usr/bin/env python
"""Tensor/sequence-parallel MLP halves with the collective fused into the GEMM kernel: all-gather -> GEMM(W1) and
GEMM(W2) -> reduce-scatter, in bf16 and in fp8 with hardware block scaling.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/parallel/tp_mlp.py
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from pccl_b200.engine import Engine  # noqa: E402
from pccl_b200.ops import check_status  # noqa: E402
from pccl_b200.ops.fused_tp import AllGatherGemm, AllGatherGemmFp8, GemmReduceScatter  # noqa: E402
from pccl_b200.ops.gemm import quant_blocks_mx  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    tokens, d_model, d_ff = 1024 * world, 4096, 2048 * world          # tokens are sharded by rows, d_ff by columns
    eng = Engine(rank, world)
    eng.initEngine("cuda", heap_bytes=8 * tokens * d_model + (1 << 30))
    eng.connect()
    g = torch.Generator(device="cuda").manual_seed(rank)
    x_local = torch.randn(tokens // world, d_model, device="cuda", generator=g).bfloat16()
    w1 = (torch.randn(d_ff // world, d_model, device="cuda", generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(d_model, d_ff // world, device="cuda", generator=g) * 0.02).bfloat16()

    # bf16: Y = all_gather(X) @ W1^T, H = gelu(Y), Z_r = reduce_scatter(H @ W2^T)
    ag = AllGatherGemm(eng, tokens, d_model, n_copy=16)
    rs = GemmReduceScatter(eng, tokens, d_model)
    ag.x_local.copy_(x_local)                       # this rank's rows of the symmetric gathered buffer
    h = torch.nn.functional.gelu(ag(w1), approximate="tanh")
    z = rs(h, w2)

    # fp8, scales applied by the tensor core: rows and their power-of-two scale bytes are gathered, bf16 output
    agx = AllGatherGemmFp8(eng, tokens, d_model, n_copy=8, mx=True)
    w1q, w1s = quant_blocks_mx(w1)
    agx.quantize_local(x_local)
    y8 = agx(w1q, w1s)
    torch.cuda.synchronize()
    check_status("tp mlp")
    rel = (y8.float() - ag(w1).float()).abs().max().item() / ag(w1).float().abs().max().item()
    if rank == 0:
        print(f"z shard {tuple(z.shape)}; fp8 vs bf16 first GEMM: max relative difference {rel:.3f}")
    dist.barrier()
    del ag, rs, agx, eng
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
