"""The host side of the native extension (engine, cluster daemon, TCP transport, CPU executor, bindings) under
AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer: further builds of the extension with
instrumented host objects run part of the CPU suite in a child process.  compute-sanitizer is not available for the
device side; the kernels have their own bounds-checked mode and differential tests instead."""
import os
import shutil
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _runtime(name):
    r = subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True)
    path = r.stdout.strip()
    return path if r.returncode == 0 and os.path.isabs(path) and os.path.exists(path) else None


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_host_code_is_clean_under_asan_and_ubsan():
    asan, stdcxx = _runtime("libasan.so"), _runtime("libstdc++.so")
    if not asan or not stdcxx:
        pytest.skip("the sanitizer runtime of this gcc is not installed")
    sys.path.insert(0, ROOT)
    from pccl_b200 import _build
    lib = _build.build(verbose=False, sanitize=True)
    env = dict(os.environ)
    # libstdc++ is preloaded next to the sanitizer runtime: python itself does not link it, and the runtime's
    # interceptor of __cxa_throw must find the real one when it initialises
    env.update({"LD_PRELOAD": f"{asan} {stdcxx}", "PCCL_NATIVE_LIB": str(lib),
                "ASAN_OPTIONS": "detect_leaks=0:halt_on_error=1", "UBSAN_OPTIONS": "print_stacktrace=1:halt_on_error=1"})
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider",
           os.path.join(HERE, "test_native_common.py"),
           os.path.join(HERE, "test_engine_cpu.py") + "::test_one_op_may_run_at_a_different_width_on_every_launch",
           os.path.join(HERE, "test_engine_cpu.py") + "::test_two_ops_overlap_on_two_lanes_from_two_threads",
           os.path.join(HERE, "test_engine_cpu.py") + "::test_regop_accepts_file_and_rejects_garbage",
           os.path.join(HERE, "test_engine_cpu.py") + "::test_instruction_trace_is_chrome_trace_json",
           os.path.join(HERE, "test_engine_cpu.py") + "::test_device_stamps_become_trace_events",
           os.path.join(HERE, "test_engine_cpu.py") + "::test_a_rank_that_only_sends_cannot_overrun_the_receivers_workspace",
           os.path.join(HERE, "test_elastic_cpu.py") + "::test_survivors_run_in_the_resized_world",
           os.path.join(HERE, "test_elastic_cpu.py") + "::test_wait_on_a_rank_that_never_launches_times_out"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500, cwd=ROOT)
    text = r.stdout + r.stderr
    assert "AddressSanitizer" not in text and "runtime error:" not in text, text[-6000:]
    assert r.returncode == 0, text[-6000:]
    assert " passed" in text


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_host_threads_are_race_free_under_tsan(tmp_path):
    """The daemon's io/worker/heartbeat threads, two lanes driven from two Python threads and the CPU executor's
    stream threads, with every report written to a log file per process: none may appear."""
    tsan, stdcxx = _runtime("libtsan.so"), _runtime("libstdc++.so")
    if not tsan or not stdcxx:
        pytest.skip("the sanitizer runtime of this gcc is not installed")
    sys.path.insert(0, ROOT)
    from pccl_b200 import _build
    lib = _build.build(verbose=False, sanitize="thread")
    logs = tmp_path / "tsan"
    env = dict(os.environ)
    # OpenMP workers of torch synchronise through futexes that the sanitizer cannot see: one thread there, and
    # the suppression file covers what is left; torch's own exit-time mutex handling is not ours to report
    env.update({"LD_PRELOAD": f"{tsan} {stdcxx}", "PCCL_NATIVE_LIB": str(lib), "OMP_NUM_THREADS": "1",
                "TSAN_OPTIONS": f"halt_on_error=0:report_mutex_bugs=0:log_path={logs}:"
                                f"suppressions={os.path.join(HERE, 'tsan.supp')}"})
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider",
           os.path.join(HERE, "test_native_common.py"),
           os.path.join(HERE, "test_engine_cpu.py") + "::test_two_ops_overlap_on_two_lanes_from_two_threads",
           os.path.join(HERE, "test_engine_cpu.py") + "::test_one_op_may_run_at_a_different_width_on_every_launch",
           os.path.join(HERE, "test_engine_cpu.py") + "::test_instruction_trace_is_chrome_trace_json",
           os.path.join(HERE, "test_elastic_cpu.py") + "::test_wait_on_a_rank_that_never_launches_times_out"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500, cwd=ROOT)
    text = r.stdout + r.stderr
    if "unexpected memory mapping" in text:
        pytest.skip("this kernel's address-space layout is not one the sanitizer runtime supports")
    reports = sorted(tmp_path.glob("tsan.*"))
    assert not reports, reports[0].read_text()[:6000]
    assert r.returncode == 0, text[-6000:]
    assert " passed" in text
