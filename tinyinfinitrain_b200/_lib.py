"""Loader for the in-tree native libraries.

``C`` is the pybind module ``_C`` (op bindings + C++ core).  If the shared
objects are missing they are built once, in-tree, with ``_build.build()``.
A CUDA tensor reaching an op while the library is absent is an error: there is
no eager fallback for the GPU path.
"""
from __future__ import annotations

import importlib
import os
import threading

import torch  # noqa: F401  (libtorch must be loaded before _C)

_lock = threading.Lock()
_C = None
_err = None


def load():
    global _C, _err
    if _C is not None:
        return _C
    with _lock:
        if _C is not None:
            return _C
        from . import _build

        try:
            if not _build.is_built():
                if os.environ.get("TITB200_NO_AUTOBUILD"):
                    raise ImportError("native libraries not built; run `python -m tinyinfinitrain_b200._build`")
                _build.build()
            _C = importlib.import_module("tinyinfinitrain_b200._C")
        except Exception as e:  # noqa: BLE001
            _err = e
            raise
    return _C


def available() -> bool:
    try:
        load()
        return True
    except Exception:  # noqa: BLE001
        return False


class _Lazy:
    def __getattr__(self, name):
        return getattr(load(), name)


C = _Lazy()
