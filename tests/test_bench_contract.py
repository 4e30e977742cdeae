"""Contract of the repository-level entry points that do not need a GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_why_it_is_unavailable():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    doc = json.loads(r.stdout.strip().splitlines()[-1])
    assert doc["impl"] == "reference" and isinstance(doc["unavailable"], str) and len(doc["unavailable"]) > 20


def test_build_entry_point_compiles_and_imports():
    r = subprocess.run([sys.executable, "-c", "import __graft_entry__ as g; g.build(); print('ok')"], capture_output=True, text=True,
                       timeout=1500, cwd=ROOT)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), (r.stdout + r.stderr)[-3000:]


def test_every_kernel_source_targets_sm_100a_only():
    """One architecture, no fall-back code paths: the build passes exactly one -gencode and no source asks for another."""
    sys.path.insert(0, ROOT)
    from pccl_b200 import _build
    assert _build.ARCH_FLAGS == ["-gencode", "arch=compute_100a,code=sm_100a"]
    _, cu = _build.sources()
    assert len(cu) >= 10
    for src in cu:
        text = open(src).read()
        assert "wgmma" not in text and "__CUDA_ARCH__ <" not in text, src


def test_collective_algorithm_choice_follows_the_measured_crossovers():
    """`auto` picks the in-switch (NVLS) or the peer-to-peer kernel from measured cross-overs; no GPU is needed to check the rule."""
    from pccl_b200.ops import collectives as C

    class FakeEngine:
        def __init__(self, world, nvls):
            self.world, self.has_nvls = world, nvls

    e8, e4, e2, plain = FakeEngine(8, True), FakeEngine(4, True), FakeEngine(2, True), FakeEngine(8, False)
    assert C._algo(e8, "auto", "bf16", "sum", 1 << 20) == "nvls"
    assert C._algo(plain, "auto", "bf16", "sum", 1 << 20) == "p2p"               # no multicast object: peer loads
    assert C._algo(e8, "auto", "bf16", "sum", (1 << 20) + 8) == "p2p"            # multimem needs 16-byte vectors
    assert C._algo(e2, "auto", "f32", "sum", 4 << 20) == "nvls" and C._algo(e2, "auto", "f32", "sum", 16 << 20) == "p2p"
    assert C._algo(e4, "auto", "bf16", "sum", 32 << 20, "reduce_scatter") == "p2p"      # 128 MiB in total on four GPUs
    assert C._algo(e8, "auto", "bf16", "sum", 32 << 20, "reduce_scatter") == "nvls"
    assert C._algo(e8, "p2p", "bf16", "sum", 1 << 20) == "p2p"
    import pytest
    with pytest.raises(RuntimeError):
        C._algo(plain, "nvls", "bf16", "sum", 1 << 20)
    assert C._blocks(1 << 10, None) == 1 and C._blocks(64 << 20, None) == 128 and C._blocks(1 << 20, 7) == 7


def test_clock_sampler_reads_a_stand_in_for_nvidia_smi(tmp_path, monkeypatch):
    """The sampler only READS clocks and throttle reasons; here it reads a script that prints what the tool would."""
    import stat
    import time
    fake = tmp_path / "nvidia-smi"
    lines = ["#!/bin/sh", "for i in 1 2 3 4 5 6; do",
             "  echo '1410, 1965, 950.12, Not Active, Not Active, Not Active, Active'",
             "  echo '1395, 1965, 990.00, Not Active, Not Active, Not Active, Not Active'",
             "  sleep 0.05", "done", "sleep 5", ""]
    fake.write_text(chr(10).join(lines))
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    from pccl_b200.utils import ClockSampler
    s = ClockSampler(0, period_ms=50).start()
    time.sleep(0.6)
    out = s.stop()
    assert out["samples"] >= 4 and out["sm_max_mhz"] == 1965.0 and 1395.0 <= out["sm_mhz"] <= 1410.0
    assert out["reasons"] == ["sw_power_cap"]
    # without the tool the sampler stays silent instead of failing the benchmark
    monkeypatch.setenv("PATH", str(tmp_path / "nowhere"))
    assert ClockSampler(0).start().stop()["sm_mhz"] is None


def test_copy_cta_default_of_the_fused_all_gather_follows_the_world_size():
    """Measured choice: 8 copy CTAs on up to four GPUs, 16 on eight (an even number either way: CTA pairs copy as a cluster)."""
    from pccl_b200.ops.fused_tp import default_copy_ctas
    assert [default_copy_ctas(w) for w in (2, 4, 8)] == [8, 8, 16]
    assert all(default_copy_ctas(w) % 2 == 0 for w in range(2, 17))
