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
