"""Run-time specialisation of registered programs: the generator and NVRTC need no GPU, so the whole path up to the
cubin is checked here for every family of library program; launching is checked by the GPU tests."""
import pytest
import torch

from pccl_b200.engine import Engine
from pccl_b200.lang import DeviceType, build


def _engine(world, rank=1):
    e = Engine(rank, world)
    e.initEngine("cpu")
    return e


@pytest.mark.parametrize("algo,world,kw", [("ring_allreduce", 4, {}), ("direct_allreduce", 8, {}), ("direct_reduce_scatter", 8, {}),
                                           ("direct_allgather", 4, {}), ("alltoall", 4, {}), ("tree_allreduce", 8, {}),
                                           ("broadcast", 4, {"root": 2}), ("nvls_allreduce", 8, {}), ("nvls_reduce_scatter", 4, {}),
                                           ("hierarchical_allreduce", 8, {"per_host": 4})])
def test_generated_kernels_compile_for_sm_100a(algo, world, kw):
    from pccl_b200.jit import compile_cubin, source_for
    e = _engine(world)
    e.regOp("op", build(algo, world, channels=2, **kw))
    nbytes = 4 * world * 2 * 1024
    for dtype in ("f32", "bf16"):
        src = source_for(e, "op", nbytes, dtype, width=2)
        assert "case 0:" in src and "fetch" not in src            # straight-line code per stream, no instruction fetch
        cubin = compile_cubin(src)
        assert len(cubin) > 1000 and cubin[:4] == b"\x7fELF"


def test_generator_folds_waits_and_reduces_into_one_pass():
    """direct reduce-scatter at 8 ranks: seven "wait, reduce into the output" pairs become seven waits and ONE n-ary reduce."""
    from pccl_b200.jit import source_for
    e = _engine(8, rank=3)
    e.regOp("rs", build("direct_reduce_scatter", 8, channels=1))
    src = source_for(e, "rs", 8 * 64 * 1024, "bf16", width=1)
    assert src.count("reduce_n_range_f<DT_BF16, RED_SUM>") == 1 and "reduce_range_f<DT_BF16, RED_SUM>(d, srcs[0]" not in src
    e2 = _engine(4, rank=0)
    e2.regOp("ar", build("nvls_allreduce", 4, channels=1))
    assert "mm_reduce_bcast_range<DT_F32, RED_SUM>" in source_for(e2, "ar", 4 * 4096, "f32")
    with pytest.raises(Exception, match="no generated form"):
        source_for(e2, "ar", 4 * 4096, "i32")
