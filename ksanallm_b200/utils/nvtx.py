"""NVTX ranges around the engine's phases and the fused operators, for timelines taken with an external profiler.

Off unless ``KSANA_NVTX=1`` (a push/pop pair costs about a microsecond of host time per range, which matters at a few
hundred launches per decode step). ``annotate`` is a context manager; nested ranges are fine.
"""
from __future__ import annotations

import os
from contextlib import contextmanager

ENABLED = os.environ.get("KSANA_NVTX", "0") == "1"
_nvtx = None


def _backend():
    global _nvtx
    if _nvtx is None:
        import torch
        _nvtx = torch.cuda.nvtx if torch.cuda.is_available() else False
    return _nvtx


@contextmanager
def annotate(name: str):
    be = _backend() if ENABLED else False
    if be:
        be.range_push(name)
        try:
            yield
        finally:
            be.range_pop()
    else:
        yield


def mark(name: str) -> None:
    be = _backend() if ENABLED else False
    if be:
        be.mark(name)
