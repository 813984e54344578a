"""KV-cache classes with the reference's names, constructor signatures and
attributes (deserve_worker/kvcache/**), re-designed for a B200 host:

* all allocator state (free bitmap, prefetch buffer, page tables, isswap flags,
  region bookkeeping) lives on the HOST as numpy arrays, so that alloc / extend /
  switch never launch a kernel nor wait for the device (the reference keeps the
  bitmap on the device and synchronises in torch.nonzero and .item());
* page ids are handed out in exactly the reference's order (prefetch buffer of
  64, lowest free index first, freed pages return through the bitmap), so page
  CONTENTS can be compared at identical page ids;
* data movement (region swap, per-task offload / reload) goes through the C ABI
  of libdeserve_kv.so on side streams with explicit event edges.

Shapes are parameters: n_kv_heads and head_dim default to the reference's
hard-coded 8 and 128 (page_pool.py:26).
"""
from __future__ import annotations

import bisect
import ctypes
import math
import threading
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from .pinned import ring as _pinned_ring


def _as_ids(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy().astype(np.int64, copy=False)
    return np.asarray(x, dtype=np.int64)


def _is_cuda(device: torch.device) -> bool:
    return torch.device(device).type == "cuda"


# --------------------------------------------------------------------------
# page pool
# --------------------------------------------------------------------------
class PagePool:
    """KV storage + free-page allocator (reference: paged/page_pool.py:7-82)."""

    def __init__(
        self,
        num_layers: int,
        num_pages: int,
        page_size: int,
        main_device: torch.device,
        main_dtype: torch.dtype,
        n_kv_heads: int = 8,
        head_dim: int = 128,
    ):
        self.num_layers = num_layers
        self.num_pages = num_pages
        self.page_size = page_size
        self.main_device = torch.device(main_device)
        self.main_dtype = main_dtype
        self.n_kv_heads = n_kv_heads
        self.head_dim = head_dim
        self.fetch_size = 64
        self.mutex = threading.Lock()
        self.pages = torch.empty(
            (num_layers, num_pages, 2, page_size, n_kv_heads, head_dim), device=self.main_device, dtype=main_dtype
        )
        self._bitmap = np.ones(num_pages, dtype=bool)  # True = free
        # ids already taken out of the bitmap: a window (start, length) of a fixed array, so that the
        # native step builder can work on the same state
        self._buf_store = np.zeros(max(num_pages, 1), dtype=np.int32)
        self._buf_win = np.zeros(2, dtype=np.int32)
        self._avails = np.array([num_pages], dtype=np.int64)

    @property
    def num_avails(self) -> int:
        return int(self._avails[0])

    @num_avails.setter
    def num_avails(self, value: int) -> None:
        self._avails[0] = value

    @property
    def _buffer(self) -> np.ndarray:
        return self._buf_store[self._buf_win[0] : self._buf_win[0] + self._buf_win[1]]

    @_buffer.setter
    def _buffer(self, ids: np.ndarray) -> None:
        n = len(ids)
        self._buf_store[:n] = ids
        self._buf_win[0], self._buf_win[1] = 0, n

    # attributes the reference exposes as tensors
    @property
    def page_bitmap(self) -> torch.Tensor:
        return torch.from_numpy(self._bitmap)

    @property
    def page_buffer(self) -> torch.Tensor:
        return torch.from_numpy(self._buffer.copy())

    @property
    def page_elems(self) -> int:
        return 2 * self.page_size * self.n_kv_heads * self.head_dim

    @property
    def page_bytes(self) -> int:
        return self.page_elems * self.pages.element_size()

    @property
    def layer_stride_bytes(self) -> int:
        return self.pages.stride(0) * self.pages.element_size()

    def calc_num_pages(self, size: int) -> int:
        return (size + self.page_size - 1) // self.page_size

    def _alloc_np(self, size: int) -> np.ndarray:
        with self.mutex:
            if size > self.num_avails:
                raise ValueError(f"Not enough pages {size} > {self.num_avails}")
            self.num_avails -= size
            short = size - len(self._buffer)
            if short > 0:
                want = max(self.fetch_size, short)
                got = np.flatnonzero(self._bitmap)[:want].astype(np.int32)
                self._bitmap[got] = False
                self._buffer = np.concatenate([self._buffer, got])
            out = self._buffer[:size].copy()
            self._buf_win[0] += size
            self._buf_win[1] -= size
            return out

    def alloc(self, size: int) -> Optional[torch.Tensor]:
        """`size` page ids as an int32 tensor (host memory). Raises ValueError
        when the pool cannot satisfy the request."""
        return torch.from_numpy(self._alloc_np(size))

    def reserve(self, ids) -> None:
        """Take the given page ids out of the free set (they must all be free and not
        in the prefetch buffer): for callers that place a cache on pages of their own
        choosing, e.g. a seeded random permutation of the pool, and hand the ids to
        PageTableHandle.extend themselves. free() returns them as usual."""
        ids = _as_ids(ids)
        with self.mutex:
            if len(ids) == 0:
                return
            if ids.min() < 0 or ids.max() >= self.num_pages:
                raise ValueError("reserve: page id outside the pool")
            if len(np.unique(ids)) != len(ids) or not self._bitmap[ids].all():
                raise ValueError("reserve: a page is not free (or is listed twice)")
            self._bitmap[ids] = False
            self.num_avails -= len(ids)

    def alloc_consecutive(self, size: int) -> Optional[torch.Tensor]:
        """First run of `size` consecutive free pages, or None."""
        with self.mutex:
            if size > self.num_avails or size <= 0:
                return None
            free = np.concatenate([[0], self._bitmap.astype(np.int8), [0]])
            edges = np.diff(free)
            starts, ends = np.flatnonzero(edges == 1), np.flatnonzero(edges == -1)
            fits = np.flatnonzero(ends - starts >= size)
            if len(fits) == 0:
                return None
            self.num_avails -= size
            s = int(starts[fits[0]])
            # the reference returns the whole run it found and leaves the bitmap to the caller
            return torch.arange(s, int(ends[fits[0]]), dtype=torch.int64)

    def free(self, blocks) -> None:
        ids = _as_ids(blocks)
        with self.mutex:
            self.num_avails += len(ids)
            self._bitmap[ids] = True
            rows = getattr(self, "rows_used", None)
            if rows is not None and len(ids):  # whoever gets a swap-region page next holds whole pages until told otherwise
                reg = ids[ids >= self.num_pages_main] - self.num_pages_main
                rows[reg] = self.page_size

    def retrieve(self, indices) -> torch.Tensor:
        idx = torch.as_tensor(_as_ids(indices), device=self.pages.device)
        return self.pages[:, idx]

    def get_layered_pages(self, layer: int) -> torch.Tensor:
        return self.pages[layer]


class GpuPagePool(PagePool):
    pass


class CpuPagePool(PagePool):
    def __init__(self, num_layers: int, num_pages: int, page_size: int, main_dtype: torch.dtype,
                 n_kv_heads: int = 8, head_dim: int = 128):
        super().__init__(num_layers, num_pages, page_size, torch.device("cpu"), main_dtype, n_kv_heads, head_dim)


# --------------------------------------------------------------------------
# page tables
# --------------------------------------------------------------------------
@dataclass
class PageTableHandle:
    """One row of the table: `offset` = row, `occupied` = pages in use
    (reference: paged/page_table.py:8-26)."""

    offset: int
    occupied: int
    allocator: "PageTableAllocator"

    def retrieve(self) -> torch.Tensor:
        return self.allocator.tables[self.offset, : self.occupied]

    def retrieve_all(self) -> torch.Tensor:
        return self.allocator.tables[self.offset, :]

    def retrieve_np(self) -> np.ndarray:
        return self.allocator._tables_np[self.offset, : self.occupied]

    def extend(self, fill) -> None:
        ids = _as_ids(fill)
        self.allocator._tables_np[self.offset, self.occupied : self.occupied + len(ids)] = ids
        self.occupied += len(ids)

    def free(self) -> None:
        self.allocator.free(self)


class PageTableAllocator:
    """(max_requests, max_context_len // page_size) int32 table + a LIFO stack of
    free rows; the first row handed out is the last one (reference:
    paged/page_table.py:29-60). The table lives in host memory."""

    def __init__(self, max_requests_num: int, max_context_len: int, page_size: int, main_device: torch.device) -> None:
        self.max_requests_num = max_requests_num
        self.max_context_len = max_context_len
        self.page_size = page_size
        self.main_device = torch.device(main_device)
        self.mutex = threading.Lock()
        self._tables_np = np.zeros((max_requests_num, max_context_len // page_size), dtype=np.int32)
        self.tables = torch.from_numpy(self._tables_np)
        self._isswap_np = np.zeros(self._tables_np.shape, dtype=bool)  # per entry: page sits in a swap region
        self.slots = list(range(max_requests_num))

    def alloc(self) -> PageTableHandle:
        with self.mutex:
            if len(self.slots) == 0:
                raise ValueError("No available slots")
            num = self.slots.pop()
        return PageTableHandle(num, 0, self)

    def free(self, handle: PageTableHandle) -> None:
        with self.mutex:
            self.slots.append(handle.offset)


class PagedKVCache:
    """Per-sequence handle: a page-table row that grows on demand (reference:
    paged/kvcache.py:12-33)."""

    def __init__(self, page_table: PageTableHandle, pool: PagePool) -> None:
        self.page_table = page_table
        self.pool = pool

    def __class_getitem__(cls, item):
        # the reference declares the class generic in its pool type and its callers write
        # PagedKVCache[GpuPagePool] in casts that are evaluated at run time (exec.py, processor.py)
        return cls

    @staticmethod
    def empty(allocator: PageTableAllocator, pool: PagePool) -> "PagedKVCache":
        return PagedKVCache(allocator.alloc(), pool)

    def extend(self, num_tokens: int) -> bool:
        if num_tokens > self.page_table.occupied * self.pool.page_size:
            delta = self.pool.calc_num_pages(num_tokens) - self.page_table.occupied
            self.page_table.extend(self.pool._alloc_np(delta))
        return True

    def free(self) -> None:
        self.pool.free(self.page_table.retrieve_np())
        self.page_table.free()


GpuPagedKVCache = PagedKVCache
CpuPagedKVCache = PagedKVCache


# --------------------------------------------------------------------------
# pinned host memory
# --------------------------------------------------------------------------
class PinnedMemory:
    """1-D pinned host buffer (reference: pinned/pinned_memory.py:4-9, where the
    element type is always fp16; here it follows `dtype`)."""

    def __init__(self, size: int, dtype: torch.dtype = torch.float16) -> None:
        self.size = 0
        self.memory = torch.empty((size,), dtype=dtype, pin_memory=torch.cuda.is_available())


class PinnedKVCache:
    """A range of a PinnedMemory (reference: pinned/kvcache.py:4-8; nothing on the path uses it)."""

    def __init__(self, memory: PinnedMemory, ptr: int, size: int):
        self.memory, self.ptr, self.size = memory, ptr, size


class CopiedPinnedMemory(PinnedMemory):
    """Host image of one swap region plus the free bitmap / count that travel
    with it (reference: virtual.py:12-16)."""

    def __init__(self, size: int, num_pages_swap: int, device: torch.device, dtype: torch.dtype = torch.float16) -> None:
        super().__init__(size, dtype)
        self.bitmap = np.ones(num_pages_swap, dtype=bool)
        self.count = num_pages_swap
        # token rows in use per page of the image (None = unknown: whole pages travel); written by swap2
        self.rows = None


# --------------------------------------------------------------------------
# virtual pool: main pages + two swap regions
# --------------------------------------------------------------------------
class VirtualPagePool(GpuPagePool):
    """Pages [0, main) are shared by all microbatches; [main, main+swap) and
    [main+swap, main+2*swap) are the two swap regions. Region `on` belongs to the
    microbatch computing now, the other one is in flight to / from pinned host
    memory (reference: virtual.py:19-116)."""

    def __init__(
        self,
        num_layers: int,
        num_pages_main: int,
        num_pages_swap: int,
        page_size: int,
        main_device: torch.device,
        main_dtype: torch.dtype,
        n_kv_heads: int = 8,
        head_dim: int = 128,
    ):
        super().__init__(num_layers, num_pages_main + 2 * num_pages_swap, page_size, main_device, main_dtype,
                         n_kv_heads, head_dim)
        m, s = num_pages_main, num_pages_swap
        self.slices = [(m, m + s), (m + s, m + 2 * s)]
        self._bitmap[self.slices[1][0] : self.slices[1][1]] = False
        self._swap_bitmap = np.ones(s, dtype=bool)
        self.swap_count = s
        self.num_avails = m + s
        self.num_pages_main = m
        self.num_pages_swap = s
        self.on = 0
        self.live_only = True            # swap2 moves only the head of a region that is in use
        self.last_swap_pages = (0, 0)    # pages per layer the last swap2 moved (out, in)
        self.last_swap_rows = (page_size, page_size)  # token rows of each half page it moved (out, in)
        # token rows that carry data, per page of the two regions (page_size = the whole page: the state of a
        # page nobody has described yet); the step builder lowers it for the pages it describes (note_rows)
        self.rows_used: np.ndarray | None = np.full(2 * s, page_size, dtype=np.int32) if s > 0 else None
        self.dma_events: list | None = None  # set to [] to collect (out start, out end, in start, in end) timing events
        if _is_cuda(self.main_device):
            self.stream = torch.cuda.Stream(device=self.main_device)   # outgoing DMA
            self.stream2 = torch.cuda.Stream(device=self.main_device)  # incoming DMA
            self._edge = torch.cuda.Event()
            self._edge.record(self.stream)  # forces creation of the underlying cudaEvent_t
        else:
            self.stream = self.stream2 = self._edge = None

    @property
    def swap_bitmap(self) -> torch.Tensor:
        return torch.from_numpy(self._swap_bitmap)

    def switch(self) -> None:
        """Flip the active region: hand the prefetch buffer back, publish the
        incoming region's saved bitmap, save and clear the outgoing one."""
        with self.mutex:
            self._bitmap[self._buffer.astype(np.int64)] = True
            self._buf_win[:] = 0
            on, off = self.on, 1 - self.on
            a, b = self.slices[on]
            c, d = self.slices[off]
            remained = int(self._bitmap[a:b].sum())
            self.num_avails -= remained
            self._bitmap[c:d] = self._swap_bitmap
            self.num_avails += self.swap_count
            self._swap_bitmap = self._bitmap[a:b].copy()
            self.swap_count = remained
            self._bitmap[a:b] = False
            self.on = off

    def _handoff(self, from_memory: CopiedPinnedMemory, to_memory: CopiedPinnedMemory) -> tuple[int, int]:
        to_memory.bitmap = self._swap_bitmap
        to_memory.count = self.swap_count
        self._swap_bitmap = np.asarray(from_memory.bitmap).astype(bool)
        self.swap_count = from_memory.count
        return self.slices[1 - self.on]

    def note_rows(self, page_ids: np.ndarray, tails: np.ndarray, tail_rows: np.ndarray) -> None:
        """Called by the step builder: the pages a step's requests hold (`page_ids`, full but for each
        request's last page `tails`, which holds `tail_rows` tokens). Keeps, per page of the swap regions,
        how many token rows carry data, so that swap2 moves only those rows of each half page."""
        if self.rows_used is None:
            return
        main = self.num_pages_main
        reg = page_ids[page_ids >= main]
        if reg.size:
            self.rows_used[reg - main] = self.page_size
        sel = tails >= main
        if sel.any():
            self.rows_used[tails[sel] - main] = tail_rows[sel]

    def _rows_of(self, lo: int, n_pages: int, free_bitmap) -> int:
        """Most token rows any page in use among the first n_pages of the region at page `lo` holds."""
        if n_pages == 0:
            return 0
        if self.rows_used is None:
            return self.page_size
        used = ~np.asarray(free_bitmap[:n_pages], dtype=bool)
        rows = self.rows_used[lo - self.num_pages_main : lo - self.num_pages_main + n_pages][used]
        return int(rows.max()) if rows.size else 0

    @staticmethod
    def _live_pages(free_bitmap) -> int:
        """Pages of a region that have to travel: everything up to the highest page in
        use (the allocator hands out the lowest free page first, so the pages in use sit
        at the head of the region and the tail is free)."""
        used = np.flatnonzero(~np.asarray(free_bitmap, dtype=bool))
        return int(used[-1]) + 1 if len(used) else 0

    def swap2(self, from_memory: CopiedPinnedMemory, to_memory: CopiedPinnedMemory) -> None:
        """Region `off` -> to_memory, from_memory -> region `off`, asynchronously
        on the two side streams. The outgoing copy first waits for everything
        already queued on the current stream (the region's last kernels). Only the
        head of each region up to its highest page in use travels (`live_only`; the
        reference moves the whole region whether or not a page of it is in use): the
        contents of free pages are never read, so leaving them behind changes no
        result. Set `live_only = False` for the reference's exact byte movement."""
        lo, hi = self._handoff(from_memory, to_memory)
        rows_out = rows_in = self.page_size
        if self.live_only:
            n_out, n_in = self._live_pages(to_memory.bitmap), self._live_pages(self._swap_bitmap)
            if self.rows_used is not None:
                # of the pages that travel, only the token rows that hold data: the outgoing image remembers
                # its pages' rows, the incoming one brings its own back into this region's slots
                rel = lo - self.num_pages_main
                rows_out = self._rows_of(lo, n_out, to_memory.bitmap)
                to_memory.rows = self.rows_used[rel : rel + (hi - lo)].copy()
                if from_memory.rows is not None:
                    self.rows_used[rel : rel + (hi - lo)] = from_memory.rows
                    rows_in = self._rows_of(lo, n_in, self._swap_bitmap)
                else:
                    self.rows_used[rel : rel + (hi - lo)] = self.page_size
        else:
            n_out = n_in = hi - lo
        self.last_swap_pages = (n_out, n_in)
        self.last_swap_rows = (rows_out, rows_in)
        self._region_dma(lo, hi, to_memory.memory, from_memory.memory, n_out, n_in, rows_out, rows_in)

    def swap(self, from_memory: CopiedPinnedMemory, to_memory: CopiedPinnedMemory) -> None:
        """Same data movement as swap2; the reference's torch statement of it
        copies the bitmap instead of aliasing it (virtual.py:100-103)."""
        off = 1 - self.on
        to_memory.bitmap = self._swap_bitmap.copy()
        self._swap_bitmap = np.asarray(from_memory.bitmap).astype(bool)
        lo, hi = self.slices[off]
        self._region_dma(lo, hi, to_memory.memory, from_memory.memory)

    def _region_dma(self, lo: int, hi: int, host_out: torch.Tensor, host_in: torch.Tensor,
                    n_out: int | None = None, n_in: int | None = None, rows_out: int | None = None,
                    rows_in: int | None = None) -> None:
        _lib.require_cuda(self.pages)
        n_out = hi - lo if n_out is None else n_out
        n_in = hi - lo if n_in is None else n_in
        need = self.calc_swap_size()
        for name, t in (("to_memory", host_out), ("from_memory", host_in)):
            if t.numel() * t.element_size() < need * self.pages.element_size():
                raise ValueError(f"{name} holds {t.numel()} elements, the swap region needs {need}")
            if t.dtype != self.main_dtype:
                raise ValueError(f"{name} dtype {t.dtype} differs from the pool dtype {self.main_dtype}")
        self.stream.wait_stream(torch.cuda.current_stream(self.main_device))
        self.stream2.wait_stream(torch.cuda.current_stream(self.main_device))
        timing = None
        if self.dma_events is not None and (n_out or n_in):
            timing = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            timing[0].record(self.stream)
            timing[2].record(self.stream2)
        _lib.check(_lib.lib.dsv_region_swap(
            self.pages.data_ptr(), self.num_layers, self.layer_stride_bytes, lo * self.page_bytes,
            (hi - lo) * self.page_bytes, n_out * self.page_bytes, n_in * self.page_bytes, host_out.data_ptr(),
            host_in.data_ptr(), self.stream.cuda_stream, self.stream2.cuda_stream, self._edge.cuda_event,
            self.page_bytes, self.page_size, self.page_size if rows_out is None else rows_out,
            self.page_size if rows_in is None else rows_in))
        if timing is not None:
            timing[1].record(self.stream)
            timing[3].record(self.stream2)
            self.dma_events.append(timing)

    def wait_swap(self) -> None:
        """Make the current stream wait for the DMA queued so far (device-side
        edge; the host does not block)."""
        cur = torch.cuda.current_stream(self.main_device)
        cur.wait_stream(self.stream)
        cur.wait_stream(self.stream2)

    def calc_swap_size(self) -> int:
        return self.num_layers * self.num_pages_swap * self.page_elems


class VirtualPagedKVCache(PagedKVCache):
    """PagedKVCache over a VirtualPagePool; remembers which of its pages sit in a
    swap region so they can be shifted when the microbatch changes region
    (reference: virtual.py:119-161). The flags live beside the page table row."""

    def __init__(self, page_table: PageTableHandle, isswap, pool: VirtualPagePool) -> None:
        super().__init__(page_table, pool)
        row = page_table.allocator._isswap_np[page_table.offset]
        row[:] = False
        if isswap is not None:
            flags = np.asarray(isswap.cpu() if isinstance(isswap, torch.Tensor) else isswap).astype(bool)
            n = min(len(flags), len(row))
            row[:n] = flags[:n]

    @property
    def _isswap(self) -> np.ndarray:
        return self.page_table.allocator._isswap_np[self.page_table.offset]

    @property
    def isswap(self) -> torch.Tensor:
        return torch.from_numpy(self._isswap)

    @staticmethod
    def empty(allocator: PageTableAllocator, pool: VirtualPagePool) -> "VirtualPagedKVCache":
        return VirtualPagedKVCache(allocator.alloc(), None, pool)

    def extend(self, num_tokens: int) -> bool:
        occ = self.page_table.occupied
        if num_tokens > occ * self.pool.page_size:
            new_n = self.pool.calc_num_pages(num_tokens)
            ids = self.pool._alloc_np(new_n - occ)
            self._isswap[occ:new_n] = ids >= self.pool.num_pages_main
            self.page_table.extend(ids)
        return True

    def adjust(self, offset: int) -> None:
        row = self.page_table.retrieve_np()
        row[self._isswap[: self.page_table.occupied]] += offset

    def free(self) -> None:
        self._isswap[:] = False
        super().free()


# --------------------------------------------------------------------------
# pinned buddy pool of page chunks
# --------------------------------------------------------------------------
@dataclass
class ChunkHandle:
    id: int
    level: int
    initial_size: int
    pool: "ChunkPool"

    def free(self) -> None:
        self.pool.free(self.id, self.level)

    @property
    def row_begin(self) -> int:
        return self.id * (1 << self.level) * self.pool.num_layers

    def retrieve(self) -> torch.Tensor:
        n = (1 << self.level) * self.pool.num_layers
        return self.pool.chunks[self.row_begin : self.row_begin + n]


class ChunkPool:
    """Binary buddy allocator over 2**(height-1) page rows x num_layers of host
    memory; a chunk of level k holds 2**k pages of every layer, layer-major
    (reference: paged/chunk_pool.py:26-96, including its list discipline: split
    appends the children at the end, alloc pops the first id, free merges with
    buddy id^1 by bisection)."""

    def __init__(self, num_layers: int, height: int, page_size: int, main_device: torch.device,
                 main_dtype: torch.dtype, n_kv_heads: int = 8, head_dim: int = 128):
        self.num_layers = num_layers
        self.height = height
        self.page_size = page_size
        self.main_device = torch.device(main_device)
        self.main_dtype = main_dtype
        self.mutex = threading.Lock()
        self.per_token_shape = (2, page_size, n_kv_heads, head_dim)
        self.chunks = torch.empty(((1 << (height - 1)) * num_layers, *self.per_token_shape), device=self.main_device,
                                  dtype=main_dtype, pin_memory=torch.cuda.is_available())
        self.available_ids: list[list[int]] = [[] for _ in range(height)]
        self.available_ids[height - 1] = [0]

    def split(self, begin: int, end: int) -> None:
        for level in range(end, begin, -1):
            parent = self.available_ids[level].pop()
            self.available_ids[level - 1].extend([2 * parent, 2 * parent + 1])

    def alloc(self, size: int) -> ChunkHandle:
        if size <= 0:
            raise ValueError("chunk size must be positive")
        with self.mutex:
            level = math.ceil(math.log2(size))
            if level >= self.height:
                raise RuntimeError(f"Failed to allocate chunks for size {size} on level {level}")
            if not self.available_ids[level]:
                for i in range(level + 1, self.height):
                    if self.available_ids[i]:
                        self.split(level, i)
                        break
            if not self.available_ids[level]:
                raise RuntimeError(f"Failed to allocate chunks for size {size} on level {level}")
            return ChunkHandle(self.available_ids[level].pop(0), level, size, self)

    def free(self, id: int, level: int) -> None:
        with self.mutex:
            for lv in range(level, self.height):
                ids = self.available_ids[lv]
                pos = bisect.bisect_left(ids, id)
                if pos != 0 and (ids[pos - 1] ^ 1) == id:
                    ids.pop(pos - 1)
                elif pos != len(ids) and (ids[pos] ^ 1) == id:
                    ids.pop(pos)
                else:
                    ids.insert(pos, id)
                    break
                id //= 2


class CpuChunkPool(ChunkPool):
    def __init__(self, num_layers: int, height: int, page_size: int, main_dtype: torch.dtype,
                 n_kv_heads: int = 8, head_dim: int = 128):
        super().__init__(num_layers, height, page_size, torch.device("cpu"), main_dtype, n_kv_heads, head_dim)


# --------------------------------------------------------------------------
# per-task offload / reload
# --------------------------------------------------------------------------
class KVCacheManager:
    """Moves one task's (or many tasks') scattered pages between the device pool
    and pinned host chunks (reference: manager.py:12-89). The copies are queued
    on two side streams — pack / unpack kernels on `stream`, DMA on
    `dma_stream` — and ordered against the caller's stream with events, so the
    pages may be freed (offload) or read (reload after synchronize()) right
    after the call returns, as in the reference's blocking version."""

    DEFAULT_STAGING_BYTES = 256 << 20

    def __init__(self, virtual_page_pool: VirtualPagePool, cpu_chunk_pool: CpuChunkPool,
                 page_table_allocator: PageTableAllocator, staging_bytes: int | None = None):
        self.virtual_page_pool = virtual_page_pool
        self.cpu_chunk_pool = cpu_chunk_pool
        self.page_table_allocator = page_table_allocator
        self._staging_bytes = staging_bytes or self.DEFAULT_STAGING_BYTES
        self._staging: torch.Tensor | None = None
        dev = virtual_page_pool.main_device
        if _is_cuda(dev):
            self.stream = torch.cuda.Stream(device=dev)
            self.dma_stream = torch.cuda.Stream(device=dev)
            self._events = [torch.cuda.Event() for _ in range(4)]
            for e in self._events:
                e.record(self.stream)
            self._event_ptrs = (ctypes.c_void_p * 4)(*[e.cuda_event for e in self._events])
        else:
            self.stream = self.dma_stream = None

    # ---- helpers ---------------------------------------------------------------
    def _check_pools(self) -> None:
        pool, chunks = self.virtual_page_pool, self.cpu_chunk_pool
        if chunks.per_token_shape != tuple(pool.pages.shape[2:]) or chunks.main_dtype != pool.main_dtype:
            raise ValueError("chunk pool and page pool disagree on page shape or dtype")
        if chunks.num_layers != pool.num_layers:
            raise ValueError("chunk pool and page pool disagree on num_layers")

    def _ensure_staging(self, per_layer_bytes: int) -> torch.Tensor:
        need = max(self._staging_bytes, 2 * per_layer_bytes + 512)
        if self._staging is None or self._staging.numel() < need:
            if self._staging is not None:
                # earlier calls may still be packing into / copying out of the old buffer on the side
                # streams; it goes back to the allocator only once they are done (growth is rare)
                self.stream.synchronize()
                self.dma_stream.synchronize()
            self._staging = torch.empty(need, dtype=torch.uint8, device=self.virtual_page_pool.main_device)
        return self._staging

    def _upload(self, ids: np.ndarray, indptr: np.ndarray) -> tuple[torch.Tensor, torch.Tensor]:
        host, slot = _pinned_ring("swap_ids").take(len(ids) + len(indptr))
        host_np = host.numpy()
        host_np[: len(ids)] = ids
        host_np[len(ids) :] = indptr
        dev = host.to(self.virtual_page_pool.main_device, non_blocking=True)
        _pinned_ring("swap_ids").done(slot)
        return dev[: len(ids)], dev[len(ids) :]

    def _move(self, out: bool, id_lists: Sequence[np.ndarray], handles: Sequence[ChunkHandle]) -> None:
        pool = self.virtual_page_pool
        _lib.require_cuda(pool.pages)
        self._check_pools()
        indptr = np.zeros(len(id_lists) + 1, dtype=np.int32)
        indptr[1:] = np.cumsum([len(x) for x in id_lists])
        if indptr[-1] == 0:
            return
        ids = np.concatenate(id_lists).astype(np.int32)
        rows = np.array([h.row_begin for h in handles], dtype=np.int64)
        cur = torch.cuda.current_stream(pool.main_device)
        self.stream.wait_stream(cur)  # pages written by earlier kernels / ids freed later
        staging = self._ensure_staging(int(indptr[-1]) * pool.page_bytes)
        with torch.cuda.stream(self.stream):
            ids_dev, indptr_dev = self._upload(ids, indptr)
            fn = _lib.lib.dsv_swap_out_pages if out else _lib.lib.dsv_swap_in_pages
            common = (pool.layer_stride_bytes, pool.page_bytes, pool.num_pages, pool.num_layers, ids_dev.data_ptr(),
                      indptr_dev.data_ptr(), indptr.ctypes.data, rows.ctypes.data, len(id_lists),
                      staging.data_ptr(), staging.numel())
            if out:
                rc = fn(pool.pages.data_ptr(), *common, self.cpu_chunk_pool.chunks.data_ptr(),
                        self.stream.cuda_stream, self.dma_stream.cuda_stream, self._event_ptrs)
            else:
                rc = fn(self.cpu_chunk_pool.chunks.data_ptr(), pool.pages.data_ptr(), *common,
                        self.stream.cuda_stream, self.dma_stream.cuda_stream, self._event_ptrs)
            _lib.check(rc)
        # the caller may free (offload) or must not read (reload) the pages until
        # the pack / unpack kernels are done: a device-side edge, no host wait
        cur.wait_stream(self.stream)

    # ---- reference API ------------------------------------------------------------
    def copy_gpu_to_cpu(self, paged_kvcache: PagedKVCache, task_id: str) -> ChunkHandle:
        """Only does the copy; the caller manages the KV cache's life cycle."""
        return self.offload_many([paged_kvcache])[0]

    def copy_cpu_to_gpu(self, chunk_handle: ChunkHandle, task_id: str) -> VirtualPagedKVCache:
        """Only does the copy; the caller frees the chunk."""
        return self.reload_many([chunk_handle])[0]

    def offload_many(self, kvcaches: Sequence[PagedKVCache]) -> list[ChunkHandle]:
        handles = []
        for kv in kvcaches:
            h = self.cpu_chunk_pool.alloc(kv.page_table.occupied)
            if h is None:
                raise RuntimeError("Failed to allocate chunks")
            handles.append(h)
        self._move(True, [kv.page_table.retrieve_np().copy() for kv in kvcaches], handles)
        return handles

    def reload_many(self, handles: Sequence[ChunkHandle]) -> list[VirtualPagedKVCache]:
        pool = self.virtual_page_pool
        caches, id_lists = [], []
        for h in handles:
            ids = pool._alloc_np(h.initial_size)
            table = self.page_table_allocator.alloc()
            table.extend(ids)
            caches.append(VirtualPagedKVCache(table, ids >= pool.num_pages_main, pool))
            id_lists.append(ids.copy())
        self._move(False, id_lists, handles)
        return caches

    def synchronize(self) -> None:
        """Order the current stream after every queued pack / unpack kernel and
        wait on the host for the DMA (host chunks reusable, pages readable)."""
        if self.stream is None:
            return
        torch.cuda.current_stream(self.virtual_page_pool.main_device).wait_stream(self.stream)
        self.dma_stream.synchronize()


# --------------------------------------------------------------------------
# one-object configuration, and the page-ownership check
# --------------------------------------------------------------------------
@dataclass
class KVConfig:
    """Everything that sizes a stage's KV cache in one place. The reference spreads
    these over its worker's command line (deserve_worker/worker_api.py:131-147:
    num-main-pages, num-swap-pages, buddy-height, batch-size, num-rounds) and over
    constants inside the constructors (8 kv heads x 128, page_pool.py:26; context
    4096, engine/pipeline/processor.py:74). build() calls the same constructors a
    maintainer would call by hand."""

    num_layers: int
    n_q_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    page_size: int = 16
    dtype: torch.dtype = torch.bfloat16
    num_pages_main: int = 1024
    num_pages_swap: int = 0
    max_requests: int = 256
    max_context_len: int = 4096
    buddy_height: int = 8

    def pool_bytes(self) -> int:
        elem = torch.empty(0, dtype=self.dtype).element_size()
        return (self.num_layers * (self.num_pages_main + 2 * self.num_pages_swap) * 2 * self.page_size
                * self.n_kv_heads * self.head_dim * elem)

    def build(self, device) -> tuple:
        """(pool, page table allocator, chunk pool, manager) on `device`."""
        pool = VirtualPagePool(self.num_layers, self.num_pages_main, self.num_pages_swap, self.page_size,
                               torch.device(device), self.dtype, n_kv_heads=self.n_kv_heads, head_dim=self.head_dim)
        tables = PageTableAllocator(self.max_requests, self.max_context_len, self.page_size, torch.device(device))
        chunks = CpuChunkPool(self.num_layers, self.buddy_height, self.page_size, self.dtype,
                              n_kv_heads=self.n_kv_heads, head_dim=self.head_dim)
        return pool, tables, chunks, KVCacheManager(pool, chunks, tables)


def check_page_ownership(pool: PagePool, caches: Sequence[PagedKVCache], in_flight: Optional[tuple] = None) -> None:
    """Debug check of the allocator's invariants over the caches that are live right
    now (the reference has no such check): no page id appears in two page tables
    or twice in one; every id lies inside the pool; no owned page is marked free
    in the bitmap or waits in the prefetch buffer; and, for a virtual pool, no
    table of these caches points into `in_flight` = (lo, hi), the region that is
    travelling to or from the host (pass pool.slices[1 - pool.on] for the caches
    of the microbatch that is about to compute). Raises AssertionError naming the
    first offending page. Host arithmetic only."""
    seen: dict = {}
    buffered = set(pool._buffer.tolist())
    for c, kv in enumerate(caches):
        ids = kv.page_table.retrieve_np()
        for j, pid in enumerate(ids.tolist()):
            if not 0 <= pid < pool.num_pages:
                raise AssertionError(f"cache {c} entry {j}: page id {pid} outside the pool of {pool.num_pages}")
            if pid in seen:
                raise AssertionError(f"page {pid} is owned twice: cache {seen[pid][0]} entry {seen[pid][1]} and "
                                     f"cache {c} entry {j}")
            seen[pid] = (c, j)
            if pool._bitmap[pid]:
                raise AssertionError(f"cache {c} entry {j}: page {pid} is marked free in the bitmap")
            if pid in buffered:
                raise AssertionError(f"cache {c} entry {j}: page {pid} also waits in the prefetch buffer")
            if in_flight is not None and in_flight[0] <= pid < in_flight[1]:
                raise AssertionError(f"cache {c} entry {j}: page {pid} lies in the region [{in_flight[0]}, "
                                     f"{in_flight[1]}) that is in flight")
