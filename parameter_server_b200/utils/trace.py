"""Opt-in NVTX ranges around the public operations (set ``PSB_NVTX=1``): the counterpart of the scoped
phase timers that bracket every client / server phase in the reference (VTIMER sites such as
pico-ps/operator/SparsePullOperator.h:84,116,160 and pico-ps/operator/SparsePushOperator.h:112,160,202).
Phase times INSIDE the fused kernels come from ``SparseEngine.phase_stamps`` (globaltimer stamps)."""
from __future__ import annotations

import contextlib
import os

import torch

ENABLED = os.environ.get("PSB_NVTX", "0") not in ("", "0")


@contextlib.contextmanager
def _range(name: str):
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


_NULL = contextlib.nullcontext()


def nvtx(name: str):
    """Context manager: an NVTX range when tracing is on, nothing otherwise."""
    return _range(name) if ENABLED else _NULL
