"""The CUDA device plugin against a stand-in driver library, on a machine without a GPU.

``tests/fake_libcuda.c`` backs "device" allocations with memfd pages, so the real code paths run: allocation and
export, the handle server (SCM_RIGHTS over an abstract unix socket, guarded by SO_PEERCRED and a random token),
import and mapping in another process, and the multicast book-keeping.  Each case runs in a child process because
the driver library is chosen once per process (PCCL_CUDA_DRIVER_LIB).
"""
import ctypes
import json
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def fake_driver(tmp_path_factory):
    out = tmp_path_factory.mktemp("fakecuda") / "libfakecuda.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(out), os.path.join(ROOT, "tests", "fake_libcuda.c")], check=True)
    return str(out)


def _run(fake_driver, body, timeout=120, extra_env=None):
    code = textwrap.dedent("""
        import ctypes, json, os, sys
        sys.path.insert(0, %r)
        from pccl_b200._native import C
        U = C.utils
        fake = ctypes.CDLL(os.environ["PCCL_CUDA_DRIVER_LIB"])
        fake.fake_cuda_handle_alive.argtypes = [ctypes.c_ulonglong]
        fake.fake_cuda_handle_bound.argtypes = [ctypes.c_ulonglong]
    """ % ROOT) + textwrap.dedent(body)
    env = dict(os.environ, PCCL_CUDA_DRIVER_LIB=fake_driver, **(extra_env or {}))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_releasing_one_owners_multicast_object_leaves_the_other_owners_alone(fake_driver):
    """Two owners (two engines of one process) bind two heaps to two multicast objects through the one process-wide
    device.  Releasing the first must not unmap, unbind or release the second."""
    out = _run(fake_driver, """
        assert U.cuda_device_available()
        size = 4 << 20
        a, _ = U.cuda_device_alloc(size)
        b, _ = U.cuda_device_alloc(size)
        x, y = U.cuda_mc_new(), U.cuda_mc_new()
        hx = U.cuda_mc_create(x, size, 1); U.cuda_mc_join(x, hx); vx = U.cuda_mc_bind(x, a)
        hy = U.cuda_mc_create(y, size, 1); U.cuda_mc_join(y, hy); vy = U.cuda_mc_bind(y, b)
        handle_x, handle_y = U.cuda_mc_state(x)[0], U.cuda_mc_state(y)[0]
        assert handle_x != handle_y and vx != vy
        ctypes.memset(vy, 0x5a, 4096)
        U.cuda_mc_release(x)
        res = {"x_alive": fake.fake_cuda_handle_alive(handle_x), "y_alive": fake.fake_cuda_handle_alive(handle_y),
               "y_bound": fake.fake_cuda_handle_bound(handle_y), "y_state": list(U.cuda_mc_state(y)),
               "y_byte": ctypes.string_at(vy, 1)[0], "x_state": list(U.cuda_mc_state(x))}
        U.cuda_mc_release(x)            # a second release is a no-op
        U.cuda_device_free(a)           # freeing the first heap does not touch the second owner's object either
        res["y_alive_after_free"] = fake.fake_cuda_handle_alive(handle_y)
        U.cuda_mc_release(y)
        res["y_alive_end"] = fake.fake_cuda_handle_alive(handle_y)
        U.cuda_device_free(b)
        res["live_end"] = fake.fake_cuda_live_handles()
        res["maps_end"] = fake.fake_cuda_mappings()
        print(json.dumps(res))
    """)
    assert out["x_alive"] == 0 and out["x_state"] == [0, 0, False]
    assert out["y_alive"] == 1 and out["y_bound"] == 1 and out["y_state"][1] != 0 and out["y_state"][2] is True
    assert out["y_byte"] == 0x5a and out["y_alive_after_free"] == 1
    assert out["y_alive_end"] == 0 and out["live_end"] == 0 and out["maps_end"] == 0


def test_memory_handle_reaches_another_process_only_with_the_token_and_the_same_user(fake_driver):
    """The owner serves its allocation's descriptor over an abstract unix socket.  A peer that presents the token from
    the handle document maps the memory and sees the owner's bytes; a wrong token, or (when the test runs as root
    and can change user) another user id, gets no descriptor."""
    out = _run(fake_driver, """
        import multiprocessing as mp
        size = 2 << 20
        ptr, handle = U.cuda_device_alloc(size)
        ctypes.memmove(ptr, b"pccl-heap", 9)
        doc = json.loads(handle)
        res = {"token_len": len(doc["token"]), "sock": doc["sock"]}
        res["good"] = U.cuda_fd_probe(doc["sock"], doc["id"], doc["token"])
        res["wrong_token"] = U.cuda_fd_probe(doc["sock"], doc["id"], "0" * 32)
        res["short_token"] = U.cuda_fd_probe(doc["sock"], doc["id"], "abc")
        res["unknown_id"] = U.cuda_fd_probe(doc["sock"], doc["id"] + 77, doc["token"])

        def peer(handle, q, uid):
            try:
                if uid is not None:
                    os.setgid(uid); os.setuid(uid)
                from pccl_b200._native import C as C2
                p = C2.utils.cuda_device_map(handle)
                q.put(ctypes.string_at(p, 9).decode())
            except Exception as e:
                q.put("refused: " + str(e)[:80])

        ctx = mp.get_context("fork")
        q = ctx.Queue()
        p = ctx.Process(target=peer, args=(handle, q, None)); p.start(); res["peer_read"] = q.get(timeout=60); p.join()
        if os.geteuid() == 0:
            p = ctx.Process(target=peer, args=(handle, q, 65534)); p.start(); res["other_user"] = q.get(timeout=60); p.join()
        res["refused"] = U.cuda_fd_refused()
        U.cuda_device_free(ptr)
        print(json.dumps(res))
    """)
    assert out["token_len"] == 32 and out["good"] is True
    assert out["wrong_token"] is False and out["short_token"] is False and out["unknown_id"] is False
    assert out["peer_read"] == "pccl-heap"
    if "other_user" in out:
        assert out["other_user"].startswith("refused"), out
        assert out["refused"] >= 3
    else:
        assert out["refused"] >= 2


_FABRIC_BODY = """
    import multiprocessing as mp
    size = 2 << 20
    ptr, handle = U.cuda_device_alloc(size)
    ctypes.memmove(ptr, b"pccl-heap", 9)
    doc = json.loads(handle)

    def peer(handle, q):
        try:
            from pccl_b200._native import C as C2
            f2 = ctypes.CDLL(os.environ["PCCL_CUDA_DRIVER_LIB"])
            p = C2.utils.cuda_device_map(handle)
            q.put([ctypes.string_at(p, 9).decode(), f2.fake_cuda_fabric_imports()])
        except Exception as e:
            q.put(["failed: " + str(e)[:120], -1])

    ctx = mp.get_context("fork")
    q = ctx.Queue()
    p = ctx.Process(target=peer, args=(handle, q)); p.start(); got = q.get(timeout=60); p.join()
    U.cuda_device_free(ptr)
    print(json.dumps({"has_fabric": "fabric" in doc, "fabric_len": len(doc.get("fabric", "")), "exports": fake.fake_cuda_fabric_exports(),
                      "peer_read": got[0], "peer_fabric_imports": got[1], "has_sock": bool(doc.get("sock"))}))
"""


def test_fabric_handle_travels_in_the_handle_document_when_asked_for(fake_driver):
    """PCCL_HANDLE_TYPE=fabric: the allocation is exported as 64 opaque bytes inside the handle document and a peer maps
    it from those, without asking the owner's descriptor server; the POSIX descriptor stays available next to it."""
    out = _run(fake_driver, _FABRIC_BODY, extra_env={"PCCL_HANDLE_TYPE": "fabric"})
    assert out["has_fabric"] and out["fabric_len"] == 128 and out["exports"] == 1 and out["has_sock"]
    assert out["peer_read"] == "pccl-heap" and out["peer_fabric_imports"] == 1


def test_fabric_request_falls_back_to_descriptors_where_the_driver_refuses(fake_driver):
    """A driver without an IMEX channel refuses allocations that ask for fabric handles: the plugin allocates again
    without them and peers map through the descriptor server, as they do by default."""
    out = _run(fake_driver, _FABRIC_BODY, extra_env={"PCCL_HANDLE_TYPE": "fabric", "FAKE_CUDA_NO_FABRIC": "1"})
    assert not out["has_fabric"] and out["exports"] == 0
    assert out["peer_read"] == "pccl-heap" and out["peer_fabric_imports"] == 0
    out = _run(fake_driver, _FABRIC_BODY)                      # not asked for: nothing changes
    assert not out["has_fabric"] and out["peer_read"] == "pccl-heap"
