"""Reusable pinned host buffers for the small per-step uploads (descriptors,
attention plans, page-id lists).

The step path uploads a few KB to a few hundred KB of int32 metadata per
microbatch step. Asking the pinned allocator for a fresh buffer each time costs
host time on the critical path; a ring of a few buffers that are reused once the
copy that read them has finished does not. The reference builds the same arrays
with torch.tensor(..., device="cuda") from pageable memory, one blocking copy
each (deserve_worker/model/context/flash.py:50-64).
"""
from __future__ import annotations

import threading

import torch


class PinnedRing:
    """`slots` pinned int32 buffers handed out round-robin.

    take(n) returns (buffer[:n], slot). After queuing the host->device copy that
    reads the buffer, call done(slot) on the stream of the copy; the slot is then
    reused only after that copy has finished. Host-side readers of a buffer (a C
    call that reads a plan header during the step) stay valid for slots - 1
    further take() calls."""

    def __init__(self, slots: int = 8, capacity: int = 1 << 14, pin: bool | None = None):
        self._pin = torch.cuda.is_available() if pin is None else pin
        self._bufs = [torch.empty(capacity, dtype=torch.int32, pin_memory=self._pin) for _ in range(slots)]
        self._events: list = [None] * slots
        self._next = 0
        self._lock = threading.Lock()  # rings are process-wide: the engine thread and a transfer thread may share one

    def take(self, n: int) -> tuple[torch.Tensor, int]:
        with self._lock:
            slot = self._next
            self._next = (slot + 1) % len(self._bufs)
        ev = self._events[slot]
        if ev is not None:
            ev.synchronize()  # the copy queued slots steps ago: long done in steady state
            self._events[slot] = None
        if self._bufs[slot].numel() < n:
            self._bufs[slot] = torch.empty(max(n, 2 * self._bufs[slot].numel()), dtype=torch.int32, pin_memory=self._pin)
        return self._bufs[slot][:n], slot

    def done(self, slot: int, stream=None) -> None:
        if not self._pin:
            return
        ev = self._events[slot]
        if ev is None:
            ev = self._events[slot] = torch.cuda.Event()
        ev.record(stream if stream is not None else torch.cuda.current_stream())


_RINGS: dict = {}

# bytes of step metadata queued for upload since the last reset (descriptors, plans, page-id lists):
# what a benchmark reports as the host->device traffic the API itself causes
COUNTERS = {"h2d_bytes": 0}


def ring(name: str, slots: int = 8, capacity: int = 1 << 14) -> PinnedRing:
    """Process-wide ring by name (one per kind of upload)."""
    r = _RINGS.get(name)
    if r is None:
        r = _RINGS[name] = PinnedRing(slots, capacity)
    return r


def bind_host_to_gpu(device_index: int) -> dict:
    """Restrict this process to the CPUs NVML reports as local to the GPU, so that the pinned buffers it
    allocates afterwards (swap images, descriptor rings) and the threads that feed the GPU sit on the GPU's
    NUMA node. On a two-socket host with eight GPUs every rank otherwise allocates wherever it happens to
    run, and the region DMA of all ranks shares one socket's memory and the link between the sockets.
    Changes nothing outside this process (its own CPU affinity mask); returns what it did for the record.
    A host without NVML, or a mask that leaves no CPU of the current one, is left alone."""
    import os

    info = {"bound": False}
    try:
        import pynvml

        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        index = int(visible.split(",")[device_index]) if visible else device_index
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (max(os.cpu_count() or 1, 1) + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        local = {64 * w + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        cpus = local & allowed
        info.update(local_cpus=len(local), allowed_cpus=len(allowed))
        if cpus and cpus != allowed:
            os.sched_setaffinity(0, cpus)
            info.update(bound=True, cpus=len(cpus))
        elif cpus:
            info.update(cpus=len(cpus), note="already local")
    except Exception as exc:  # no NVML, no permission, a single-node host: nothing to do
        info["note"] = repr(exc)[:120]
    return info

