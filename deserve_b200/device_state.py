"""Allocator, page tables and descriptor build resident on the device.

`DevicePageState` is the device-side alternative to PagePool's host bitmap +
PageTableAllocator + context.build_step for a plain (non-virtual) pool: the free
bitmap, the prefetch buffer, the page tables and the per-row page counts are
device arrays advanced by the kernels of csrc/device_step.cu, which run the same
allocation function as the host builder, so the page ids are the ones the
reference hands out (deserve_worker/kvcache/paged/page_pool.py:38-55,
page_table.py:29-60, kvcache.py:21-33, model/context/flash.py:29-64).

The host keeps only COUNTS, which it can advance without looking at the device
because every allocation and free is its own call: free pages (`num_avails`, what
a scheduler reads every step) and pages per table row. They let it raise the
reference's errors ("Not enough pages", "No available slots") before anything is
launched. Per step it uploads six int32 per request; the page-id lists (one int32
per page of every request, 150 KB for 256 sequences of ~2300 tokens) are written
by the device from its own tables. The split-KV plan needs page COUNTS only, which
follow from the token counts, so planning stays on the host without a copy back.

Swap regions, per-task offload and the reference's attribute surface stay with the
host classes (kvcache.py); this class covers the decode / prefill step itself.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib
from .pinned import COUNTERS, ring as _pinned_ring

_NAMES = ("indptr", "kv_page_indptr", "kv_last_page_lens", "offsets", "seqlens", "kv_page_indices")


class DevicePageState:
    def __init__(self, num_pages: int, page_size: int, max_requests: int, max_context_len: int, device,
                 fetch_size: int = 64):
        self.device = torch.device(device)
        _lib.require_cuda(torch.empty(0, device=self.device))
        self.num_pages, self.page_size, self.fetch_size = num_pages, page_size, fetch_size
        self.max_requests = max_requests
        self.table_cols = max_context_len // page_size
        self.bitmap = torch.ones(num_pages, dtype=torch.uint8, device=self.device)
        self.buffer = torch.zeros(num_pages, dtype=torch.int32, device=self.device)
        self.state = torch.zeros(2, dtype=torch.int64, device=self.device)
        self.state[0] = num_pages
        self.tables = torch.zeros(max_requests, self.table_cols, dtype=torch.int32, device=self.device)
        self.occupied = torch.zeros(max_requests, dtype=torch.int32, device=self.device)
        # host-side counts
        self.num_avails = num_pages
        self._occupied = np.zeros(max_requests, dtype=np.int32)
        self.slots = list(range(max_requests))  # LIFO, the last row first, like PageTableAllocator

    # ---- table rows ---------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        if not self.slots:
            raise ValueError("No available slots")
        return self.slots.pop()

    def free_slots(self, slots) -> None:
        """The requests in these table rows are over: their pages go back to the bitmap (not to the
        prefetch buffer), the rows to the stack."""
        slots = [int(s) for s in slots]
        if not slots:
            return
        host, ring_slot = _pinned_ring("device_state").take(len(slots))
        host.numpy()[:] = slots
        dev = host.to(self.device, non_blocking=True)
        _pinned_ring("device_state").done(ring_slot)
        _lib.check(_lib.lib.dsv_device_free_rows(
            self.bitmap.data_ptr(), self.num_pages, self.state.data_ptr(), self.tables.data_ptr(), self.table_cols,
            self.occupied.data_ptr(), dev.data_ptr(), len(slots), _lib.current_stream_ptr(self.device)))
        _lib.LAUNCHES[0] += 1
        for s in slots:
            self.num_avails += int(self._occupied[s])
            self._occupied[s] = 0
            self.slots.append(s)

    # ---- one step -----------------------------------------------------------------------------
    def build_step(self, slots, start_pos, seqlen, initial_seqlen):
        """Grow the requests (in this order) to max(start_pos + seqlen, initial_seqlen) tokens and build the
        step's descriptors. Returns (device tensors by name, host arrays of everything except the page ids).
        Raises ValueError("Not enough pages ...") at the first request the pool cannot serve; the requests
        before it stay grown, as in the reference."""
        slots = np.asarray(slots, dtype=np.int32)
        start = np.asarray(start_pos, dtype=np.int32)
        new = np.asarray(seqlen, dtype=np.int32)
        initial = np.asarray(initial_seqlen, dtype=np.int32)
        bsz, ps = len(slots), self.page_size
        cur = start + new
        want_pages = (np.maximum(cur, initial) + ps - 1) // ps
        have = self._occupied[slots]
        grow_by = np.where(np.maximum(cur, initial) > have * ps, want_pages - have, 0)
        if (want_pages > self.table_cols).any():
            i = int(np.flatnonzero(want_pages > self.table_cols)[0])
            raise ValueError(f"request {i} needs {int(want_pages[i])} pages, a table row holds {self.table_cols}")
        # the first request whose pages are not there: everything before it is grown, then the error is raised
        left = self.num_avails - np.cumsum(grow_by)
        fail = int(np.flatnonzero(left < 0)[0]) if (left < 0).any() else bsz
        n_grow = fail
        n_pages = (cur + ps - 1) // ps
        host = {
            "indptr": np.concatenate([[0], np.cumsum(new)]).astype(np.int32),
            "kv_page_indptr": np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32),
            "kv_last_page_lens": (((cur - 1) % ps + ps) % ps + 1).astype(np.int32),
            "offsets": start.copy(), "seqlens": new.copy(),
        }
        req = np.stack([slots, start, new, initial, host["indptr"][:-1], host["kv_page_indptr"][:-1]], axis=1)
        sizes = (bsz + 1, bsz + 1, bsz, bsz, bsz, int(n_pages.sum()))
        offs = np.zeros(7, dtype=np.int64)
        offs[1:] = np.cumsum([(s + 3) & ~3 for s in sizes])
        st = _lib.current_stream_ptr(self.device)
        out = torch.empty(int(offs[6]), dtype=torch.int32, device=self.device)

        def launch(count: int, grow: bool, describe_from: np.ndarray, describe_offs: np.ndarray):
            pinned, ring_slot = _pinned_ring("device_state").take(describe_from.size)
            pinned.numpy()[:] = describe_from.reshape(-1)
            dev = pinned.to(self.device, non_blocking=True)
            _pinned_ring("device_state").done(ring_slot)
            COUNTERS["h2d_bytes"] += describe_from.size * 4
            _lib.check(_lib.lib.dsv_device_build_step(
                self.bitmap.data_ptr(), self.num_pages, self.buffer.data_ptr(), self.state.data_ptr(), self.fetch_size,
                ps, self.tables.data_ptr(), self.table_cols, self.occupied.data_ptr(), self.max_requests,
                dev.data_ptr(), count, 1 if grow else 0, out.data_ptr(), describe_offs.ctypes.data, st))
            _lib.LAUNCHES[0] += 2 if grow else 1

        if fail < bsz:  # grow what can be grown (the error below leaves them grown), describe nothing
            if n_grow:
                launch(n_grow, True, req[:n_grow], offs)
            self._commit(slots[:n_grow], grow_by[:n_grow])
            raise ValueError(f"Not enough pages {int(grow_by[fail])} > {self.num_avails}")
        launch(bsz, True, req, offs)
        self._commit(slots, grow_by)
        dev = {n: out[int(offs[k]) : int(offs[k]) + sizes[k]] for k, n in enumerate(_NAMES)}
        return dev, host

    def _commit(self, slots: np.ndarray, grow_by: np.ndarray) -> None:
        for s, g in zip(slots.tolist(), grow_by.tolist()):
            self._occupied[s] += g
            self.num_avails -= g

    # ---- checks ---------------------------------------------------------------------------------
    def snapshot(self) -> dict:
        """Device state copied to the host (tests): bitmap, prefetch window, tables, counts."""
        torch.cuda.synchronize(self.device)
        state = self.state.cpu()
        win = state[1:2].view(torch.int32).tolist()
        buf = self.buffer.cpu().numpy()
        return {"bitmap": self.bitmap.cpu().numpy().astype(bool), "buffer": buf[win[0] : win[0] + win[1]].copy(),
                "num_avails": int(state[0]), "tables": self.tables.cpu().numpy(), "occupied": self.occupied.cpu().numpy()}
