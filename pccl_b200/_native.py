"""Loader of the native extension.  Importing it never silently falls back: if ``_C.so`` is
missing it is built in-tree, and if that fails the import error says why."""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys
from pathlib import Path

_HERE = Path(__file__).resolve().parent


def load():
    override = os.environ.get("PCCL_NATIVE_LIB")
    if override:
        # an alternative build of the same extension (the sanitizer build of the host code, for one)
        spec = importlib.util.spec_from_file_location("pccl_b200._C", override)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules["pccl_b200._C"] = mod
        return mod
    so = _HERE / "_C.so"
    if not so.exists() or os.environ.get("PCCL_REBUILD") == "1":
        from . import _build
        _build.build(verbose=os.environ.get("PCCL_BUILD_VERBOSE", "0") == "1")
    try:
        return importlib.import_module("pccl_b200._C")
    except ImportError as e:  # stale object from another toolchain: rebuild once, then fail loudly
        from . import _build
        _build.build(verbose=True, force=True)
        try:
            return importlib.import_module("pccl_b200._C")
        except ImportError:
            raise ImportError(f"pccl_b200: native extension cannot be loaded ({e}); "
                              f"run `python -m pccl_b200._build` to see the compiler output") from e


C = load()
