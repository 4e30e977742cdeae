"""In-tree build of the native extension ``pccl_b200/_C.so`` for sm_100a.

Host sources (``csrc/**/*.cc``) go through g++, device sources (``csrc/kernels/*.cu``) through
``nvcc -gencode arch=compute_100a,code=sm_100a`` (cross-compiles without a GPU).  Objects are
cached under ``build/obj`` by source mtime and flags; the link output stays in the package so a
snapshot of the tree carries it.  Replaces the reference's setup.py (setup.py:42-113), which
globbed csrc/ into a ``CppExtension`` with no GPU architecture at all.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build" / "obj"
TARGET = Path(__file__).resolve().parent / "_C.so"
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _flags():
    import pybind11
    inc = [f"-I{CSRC}", f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
           f"-I{CUDA_HOME}/include"]
    cxx = ["g++", "-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function"] + inc
    nv = [NVCC, "-std=c++17", "-O3", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
          "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"] + ARCH_FLAGS + inc
    for d in filter(None, os.environ.get("PCCL_NVCC_DEFINES", "").split(",")):       # e.g. PCCL_NVCC_DEFINES=NAME=1,OTHER
        nv.append(f"-D{d}")
    if os.environ.get("PCCL_DEBUG", "0") not in ("", "0"):       # the reference's debug build (setup.py:78-81): PCCL_DLOG_* become real
        cxx.append("-DPCCL_DEBUG")
        nv.append("-DPCCL_DEBUG")
    return cxx, nv


def sources():
    cc = sorted(p for p in CSRC.rglob("*.cc"))
    cu = sorted(p for p in CSRC.rglob("*.cu"))
    return cc, cu


def _newest_header() -> float:
    return max((p.stat().st_mtime for ext in ("*.h", "*.cuh") for p in CSRC.rglob(ext)), default=0.0)


def _compile(cmd, src: Path, hdr_mtime: float, verbose: bool, extra=()):
    key = hashlib.sha1((" ".join(cmd) + str(src)).encode()).hexdigest()[:10]
    obj = OBJ / f"{src.stem}.{key}.o"
    if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr_mtime):
        return obj, False
    full = list(cmd) + list(extra) + ["-c", str(src), "-o", str(obj)]
    if verbose:
        print("[pccl build]", " ".join(full[:1] + [src.name]), flush=True)
    r = subprocess.run(full, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{r.stdout}\n{r.stderr}")
    return obj, True


_lock = threading.Lock()


SANITIZED_TARGET = ROOT / "build" / "sanitize" / "_C.so"
THREAD_SANITIZED_TARGET = ROOT / "build" / "sanitize-thread" / "_C.so"
_SANITIZERS = {"address": ("address,undefined", SANITIZED_TARGET), "thread": ("thread", THREAD_SANITIZED_TARGET)}


def build(verbose: bool = True, force: bool = False, ptxas_info: bool = False, sanitize=False) -> Path:
    """Compile whatever changed and link ``_C.so``.  Safe to call repeatedly.

    ``sanitize=True`` (or ``"address"``) builds a second copy, ``build/sanitize/_C.so``, whose HOST objects are
    compiled with ``-fsanitize=address,undefined``; ``sanitize="thread"`` builds ``build/sanitize-thread/_C.so`` with
    ``-fsanitize=thread``.  The device objects are shared with the normal build.  Load such a copy with
    ``PCCL_NATIVE_LIB=<that path>`` and ``LD_PRELOAD=$(gcc -print-file-name=libasan.so)`` (``libtsan.so`` for the
    thread build); it is what the CPU test suite uses to run the engine, daemon, transport and executor under the
    sanitizers."""
    with _lock:
        OBJ.mkdir(parents=True, exist_ok=True)
        cxx, nv = _flags()
        target = TARGET
        if sanitize:
            fsan, target = _SANITIZERS["address" if sanitize is True else sanitize]
            cxx = [c for c in cxx if c != "-O2"] + ["-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={fsan}"]
            target.parent.mkdir(parents=True, exist_ok=True)
        cc, cu = sources()
        hdr = _newest_header()
        if force:
            for o in OBJ.glob("*.o"):
                o.unlink()
        jobs = []
        with ThreadPoolExecutor(max_workers=max(2, (os.cpu_count() or 4))) as ex:
            for s in cc:
                jobs.append(ex.submit(_compile, cxx, s, hdr, verbose))
            extra = ["-Xptxas", "-v"] if ptxas_info else []
            for s in cu:
                jobs.append(ex.submit(_compile, nv, s, hdr, verbose, extra))
            results = [j.result() for j in jobs]
        objs = [str(o) for o, _ in results]
        changed = any(c for _, c in results)
        if changed or not target.exists():
            link = ["g++", "-shared", "-o", str(target)] + objs + [
                f"-L{CUDA_HOME}/lib64", "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
            if sanitize:
                link += [f"-fsanitize={fsan}"]
            if verbose:
                print("[pccl build] link", target, flush=True)
            r = subprocess.run(link, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        return target


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas-info" in sys.argv, sanitize="thread" if "--sanitize-thread" in sys.argv else "--sanitize" in sys.argv))
