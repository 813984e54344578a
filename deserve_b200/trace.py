"""Named phases of a step for profilers and for the host-time breakdown.

`with phase("descriptors"):` opens an NVTX range when DESERVE_NVTX=1 (so a
timeline shows alloc / descriptors / append+attention / swap / send / recv per
slot) and, when host timing is switched on with enable_host_timing(), adds the
host time spent inside to a per-phase total. Both are off by default and then
cost one dictionary lookup. The reference has no such ranges; its only timing is
the 5-second log of deserve_worker/engine/pipeline/processor.py:113-140.
"""
from __future__ import annotations

import os
import time
from contextlib import contextmanager

_NVTX = os.environ.get("DESERVE_NVTX", "0") == "1"
_HOST = {"on": False}
_TOTALS: dict[str, list] = {}


def enable_host_timing(on: bool = True) -> None:
    _HOST["on"] = on
    if on:
        _TOTALS.clear()


def host_totals() -> dict:
    """{phase: {"calls": n, "ms": total host milliseconds}} since enable_host_timing()."""
    return {k: {"calls": v[0], "ms": v[1] * 1e3} for k, v in _TOTALS.items()}


@contextmanager
def phase(name: str):
    if not _NVTX and not _HOST["on"]:
        yield
        return
    if _NVTX:
        import torch

        torch.cuda.nvtx.range_push(name)
    t0 = time.perf_counter()
    try:
        yield
    finally:
        if _HOST["on"]:
            rec = _TOTALS.setdefault(name, [0, 0.0])
            rec[0] += 1
            rec[1] += time.perf_counter() - t0
        if _NVTX:
            import torch

            torch.cuda.nvtx.range_pop()
