"""Loader of the native library ``_C`` (built in-tree by :mod:`parameter_server_b200._build`).

The shared object is never built implicitly on a machine with a GPU: there it must already be in
the tree (it travels with the source snapshot), and a missing library is an error rather than a
silent fallback to PyTorch ops.
"""
from __future__ import annotations

import importlib
import os


def _import_native():
    # RTLD_GLOBAL: operator plug-ins opened later (load_operator_library) bind to the registry accessor that the
    # module exports (its only symbol with default visibility besides the Python init and the C entry points)
    import sys

    flags = sys.getdlopenflags()
    sys.setdlopenflags(flags | os.RTLD_GLOBAL)
    try:
        return importlib.import_module("parameter_server_b200._C")
    finally:
        sys.setdlopenflags(flags)


def _load():
    try:
        return _import_native()
    except ImportError as first:
        import torch

        if torch.cuda.is_available() and not os.environ.get("PSB200_ALLOW_BUILD"):
            raise ImportError(
                "parameter_server_b200._C is missing on a GPU machine; build it with "
                "`python -m parameter_server_b200._build` (nvcc, sm_100a) before running"
            ) from first
        from . import _build

        _build.build()
        importlib.invalidate_caches()
        return _import_native()


C = _load()
