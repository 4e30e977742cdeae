"""Multi-GPU tests: one process per GPU under torch.distributed.run, NCCL only for the rendezvous."""
import json
import os
import subprocess
import sys

import pytest
import torch

from _ranks import free_port

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(case, nproc, tmp_path, env=None, timeout=600):
    out = tmp_path / f"{case}.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(HERE, "mp_worker.py"), case, str(out)]
    e = dict(os.environ)
    e.update(env or {})
    for attempt in range(3):
        r = subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=timeout)
        if out.exists() or "EADDRINUSE" not in r.stderr:
            break
        cmd[cmd.index("--master-port") + 1] = str(free_port())      # the port was taken between the probe and the launch
    results = json.loads(out.read_text()) if out.exists() else None
    assert results is not None, f"workers left no result file\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    for rank, res in enumerate(results):
        assert res["ok"], f"rank {rank}: {res.get('error')}\n{res.get('trace', '')}"
    return results


def _world():
    return min(torch.cuda.device_count(), 8)


@pytest.mark.parametrize("case", ["heap", "coll_p2p", "coll_nvls", "coll_fp8", "interp", "rooted", "overlap", "mixed_hosts", "resident", "jit", "dp", "dp_milp_ring", "fused_tp",
                                  "fused_tp_fp8", "tp_mlp", "moe"])
def test_case(case, tmp_path):
    _run(case, _world(), tmp_path)


def test_cases_share_one_launch(tmp_path):
    """The heap is handed back between cases, so a list of cases runs in one set of processes."""
    _run("heap,coll_p2p", _world(), tmp_path)


def test_collectives_without_nvls(tmp_path):
    _run("coll_p2p", _world(), tmp_path, env={"PCCL_TEST_NVLS": "0", "NCCL_NVLS_ENABLE": "0"})


def test_device_side_trace_of_the_interpreter_kernel(tmp_path):
    """PCCL_TRACE=1: the interpreter kernel stamps %globaltimer around every instruction; the stamps come back as
    Chrome-trace events per rank."""
    res = _run("trace", _world(), tmp_path, env={"PCCL_TRACE": "1"})
    assert all(r["info"]["trace"]["events"] > 0 for r in res)


def test_pipeline_parallel_1f1b_on_nccl(tmp_path):
    """The one-forward-one-backward pipeline schedule with NCCL point-to-point hand-offs on real GPUs (the schedule
    itself is checked against a single-process model on gloo ranks in test_pp_cpu.py)."""
    if _world() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(os.path.dirname(HERE), "examples", "parallel", "pipeline_1f1b.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
