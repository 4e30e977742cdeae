"""The InfiniBand / RoCE transport against a stand-in libibverbs, on a machine without an adapter.

``tests/fake_libibverbs.cc`` implements the verbs entry points in-process: it enforces the queue-pair state machine
(RESET -> INIT -> RTR -> RTS with the attribute masks the real library demands), checks keys and ranges of every
RDMA WRITE and fetch-and-add, and performs them on the process's own memory.  Two CPU engines (ranks 0 and 1) of ONE
process, driven from two threads, therefore run a whole collective "over verbs".  Each case is a child process because
the transport and the library are chosen from the environment when the package is imported.
"""
import json
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def fake_verbs(tmp_path_factory):
    out = tmp_path_factory.mktemp("fakeverbs") / "libfakeibverbs.so"
    subprocess.run(["g++", "-std=c++17", "-shared", "-fPIC", "-O1", "-o", str(out), os.path.join(ROOT, "tests", "fake_libibverbs.cc")],
                   check=True)
    return str(out)


def _run(fake_verbs, body, extra_env=None, timeout=180):
    code = textwrap.dedent("""
        import ctypes, json, os, sys, threading
        sys.path.insert(0, %r)
        import torch
        from pccl_b200.engine import Engine
        from pccl_b200.lang import DeviceType, build
        fake = ctypes.CDLL(os.environ["PCCL_IBVERBS_LIB"]) if os.path.exists(os.environ["PCCL_IBVERBS_LIB"]) else None
        if fake is not None:
            fake.fake_ibv_log.restype = ctypes.c_char_p
    """ % ROOT) + textwrap.dedent(body)
    env = dict(os.environ, PCCL_IBVERBS_LIB=fake_verbs, PCCL_TRANSPORT="verbs", PCCL_WORKSPACE_MB="8")
    env.update(extra_env or {})
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_ring_allreduce_between_two_engines_over_the_verbs_transport(fake_verbs):
    out = _run(fake_verbs, """
        engines = [Engine(r, 2) for r in range(2)]
        for e in engines:
            e.initEngine("cpu")
        docs = [e.exportEndpoint() for e in engines]
        for e in engines:
            e._e.importEndpoints(docs)
        for e in engines:
            e.regOp("ar", build("ring_allreduce", 2, channels=2, device_type=DeviceType.CPU))
            e.regOp("ag", build("direct_allgather", 2, channels=1, device_type=DeviceType.CPU))
        xs = [torch.arange(64 * 1024, dtype=torch.float32) * (r + 1) for r in range(2)]
        res = {"err": [], "status": []}

        def rank(r):
            for it in range(3):
                y = torch.zeros_like(xs[r])
                st = engines[r].exeOp("ar", xs[r] + it, y, width=2)
                res["status"].append(st)
                res["err"].append((y - (xs[0] + xs[1] + 2 * it)).abs().max().item())
            g = torch.zeros(2 * 4096)
            st = engines[r].exeOp("ag", xs[r][:4096].contiguous(), g)
            res["status"].append(st)
            res["err"].append((g - torch.cat([xs[0][:4096], xs[1][:4096]])).abs().max().item())

        ts = [threading.Thread(target=rank, args=(r,)) for r in range(2)]
        [t.start() for t in ts]; [t.join(120) for t in ts]
        stats = [e.stats() for e in engines]
        log = fake.fake_ibv_log().decode()
        print(json.dumps({"err": max(res["err"]), "status": res["status"], "n": len(res["err"]),
                          "qp": [stats[0].get("verbs_qp_state.1"), stats[1].get("verbs_qp_state.0")],
                          "sent": [s.get("verbs_bytes_sent", 0) for s in stats], "tcp": [s.get("tcp_bytes_sent", 0) for s in stats],
                          "log": log, "note": json.loads(docs[0])["endpoint_configs"].get("remote.verbs.note") if "endpoint_configs" in json.loads(docs[0]) else ""}))
    """)
    assert out["n"] == 8 and out["err"] < 1e-5 and all(s == 0 for s in out["status"]), out
    assert out["qp"] == ["RTS", "RTS"]
    assert min(out["sent"]) > 64 * 1024 * 4 and out["tcp"] == [0, 0]        # the payload went through verbs, none through TCP
    log = out["log"].split(";")
    # every queue pair went INIT -> RTR -> RTS in that order, nothing was posted early, nothing was refused
    for qp in {e.split(":")[0] for e in log if e.startswith("qp")}:
        states = [e.split(":")[1] for e in log if e.startswith(qp + ":")]
        assert states[:3] == ["INIT", "RTR", "RTS"], (qp, states)
    assert not any(e.startswith("error") or "bad-" in e or "before-RTS" in e for e in log), log
    assert sum(e.startswith("write:") for e in log) > 0 and log.count("faa") > 0


def test_asking_for_verbs_without_a_device_is_an_error_not_a_silent_fallback(fake_verbs):
    out = _run(fake_verbs, """
        fake.fake_ibv_set_devices(0)
        e = Engine(0, 2)
        try:
            e.initEngine("cpu")
            print(json.dumps({"raised": False}))
        except Exception as ex:
            print(json.dumps({"raised": True, "msg": str(ex)}))
    """)
    assert out["raised"] and "no verbs device" in out["msg"]


def test_without_the_library_the_engine_reports_verbs_as_unavailable_and_uses_tcp(fake_verbs):
    out = _run(fake_verbs, """
        e = Engine(0, 1)
        e.initEngine("cpu")
        doc = json.loads(e.exportEndpoint())
        cfg = doc.get("endpoint_configs", doc.get("configs", doc))
        print(json.dumps({"avail": cfg.get("remote.verbs.available"), "note": cfg.get("remote.verbs.note"), "tcp": "remote.tcp.endpoint" in cfg}))
    """, extra_env={"PCCL_IBVERBS_LIB": "/nonexistent/libibverbs.so", "PCCL_TRANSPORT": ""})
    assert out["avail"] == "0" and "not installed" in out["note"] and out["tcp"]
