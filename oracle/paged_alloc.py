"""Allocator state machines of the reference, restated on host integers.

Every class keeps plain Python / numpy state and returns numpy int32 arrays so
that a test can compare, op by op, against the product's host classes and
against traces recorded from the reference's torch classes.
"""
from __future__ import annotations

import bisect
import math

import numpy as np


class OraclePagePool:
    """deserve_worker/kvcache/paged/page_pool.py:7-82.

    State: bitmap (True = free), a prefetch buffer of page ids already removed
    from the bitmap, and num_avails. alloc() takes from the buffer first and
    refills it with max(64, shortfall) lowest-index free pages
    (page_pool.py:38-55); free() only sets bitmap bits (page_pool.py:73-76).
    """

    FETCH = 64  # page_pool.py:21

    def __init__(self, num_pages: int, page_size: int):
        self.num_pages = num_pages
        self.page_size = page_size
        self.num_avails = num_pages
        self.bitmap = np.ones(num_pages, dtype=bool)
        self.buffer = np.zeros(0, dtype=np.int32)

    def calc_num_pages(self, size: int) -> int:  # page_pool.py:35-36
        return (size + self.page_size - 1) // self.page_size

    def alloc(self, size: int) -> np.ndarray:
        if size > self.num_avails:  # page_pool.py:40-41
            raise ValueError(f"Not enough pages {size} > {self.num_avails}")
        self.num_avails -= size
        if size > len(self.buffer):  # page_pool.py:44-53
            want = max(self.FETCH, size - len(self.buffer))
            got = np.flatnonzero(self.bitmap)[:want].astype(np.int32)
            self.bitmap[got] = False
            self.buffer = np.concatenate([self.buffer, got])
        out, self.buffer = self.buffer[:size], self.buffer[size:]
        return out.copy()

    def free(self, ids: np.ndarray) -> None:
        self.num_avails += len(ids)
        self.bitmap[np.asarray(ids, dtype=np.int64)] = True


class OraclePageTables:
    """deserve_worker/kvcache/paged/page_table.py:29-60: slot stack (pop from
    the end, append on free) over an int32 table of max_context_len // page_size
    columns."""

    def __init__(self, max_requests: int, max_context_len: int, page_size: int):
        self.tables = np.zeros((max_requests, max_context_len // page_size), dtype=np.int32)
        self.slots = list(range(max_requests))
        self.max_context_len = max_context_len

    def alloc(self) -> int:
        if not self.slots:
            raise ValueError("No available slots")  # page_table.py:52-53
        return self.slots.pop()

    def free(self, slot: int) -> None:
        self.slots.append(slot)


class OracleKVCache:
    """deserve_worker/kvcache/paged/kvcache.py:12-33 (+ the isswap flags of
    deserve_worker/kvcache/virtual.py:119-161 when the pool is virtual)."""

    def __init__(self, tables: OraclePageTables, pool: OraclePagePool):
        self.tables, self.pool = tables, pool
        self.slot = tables.alloc()
        self.occupied = 0
        self.isswap = np.zeros(tables.max_context_len, dtype=bool)

    def page_ids(self) -> np.ndarray:
        return self.tables.tables[self.slot, : self.occupied]

    def extend(self, num_tokens: int) -> None:
        if num_tokens > self.occupied * self.pool.page_size:  # kvcache.py:22
            new_n = self.pool.calc_num_pages(num_tokens)
            ids = self.pool.alloc(new_n - self.occupied)
            main = getattr(self.pool, "num_pages_main", None)
            if main is not None:  # virtual.py:145-147
                self.isswap[self.occupied : new_n] = ids >= main
            self.tables.tables[self.slot, self.occupied : new_n] = ids  # page_table.py:19-23
            self.occupied = new_n

    def adjust(self, offset: int) -> None:  # virtual.py:151-152
        row = self.tables.tables[self.slot, : self.occupied]
        row[self.isswap[: self.occupied]] += offset

    def free(self) -> None:  # kvcache.py:31-33
        self.pool.free(self.page_ids().copy())
        self.tables.free(self.slot)
        self.occupied = 0


class OracleVirtualPool(OraclePagePool):
    """deserve_worker/kvcache/virtual.py:19-95: pages [0, main) are shared,
    [main, main+swap) and [main+swap, main+2*swap) are the two swap regions.
    `on` is the region of the microbatch computing now; the saved bitmap of the
    other region travels with the pinned buffer that holds its data."""

    def __init__(self, num_pages_main: int, num_pages_swap: int, page_size: int):
        super().__init__(num_pages_main + 2 * num_pages_swap, page_size)
        m, s = num_pages_main, num_pages_swap
        self.num_pages_main, self.num_pages_swap = m, s
        self.slices = [(m, m + s), (m + s, m + 2 * s)]
        self.bitmap[self.slices[1][0] : self.slices[1][1]] = False  # virtual.py:42
        self.swap_bitmap = np.ones(s, dtype=bool)
        self.swap_count = s
        self.num_avails = m + s
        self.on = 0

    def switch(self) -> None:  # virtual.py:54-77
        self.bitmap[self.buffer.astype(np.int64)] = True
        self.buffer = np.zeros(0, dtype=np.int32)
        on, off = self.on, 1 - self.on
        a, b = self.slices[on]
        c, d = self.slices[off]
        remained = int(self.bitmap[a:b].sum())
        self.num_avails -= remained
        self.bitmap[c:d] = self.swap_bitmap
        self.num_avails += self.swap_count
        self.swap_bitmap = self.bitmap[a:b].copy()
        self.swap_count = remained
        self.bitmap[a:b] = False
        self.on = off

    def swap2_bookkeeping(self, from_mem: dict, to_mem: dict) -> None:
        """The hand-off half of swap2 (virtual.py:82-86): the outgoing region's
        bitmap/count go with `to_mem`, the incoming ones come from `from_mem`.
        A pinned buffer is represented by a dict {bitmap, count}."""
        to_mem["bitmap"], to_mem["count"] = self.swap_bitmap, self.swap_count
        self.swap_bitmap = np.asarray(from_mem["bitmap"]).astype(bool)
        self.swap_count = from_mem["count"]


class OracleChunkPool:
    """deserve_worker/kvcache/paged/chunk_pool.py:26-96: binary buddy allocator
    over 2**(height-1) page rows (times num_layers). alloc(size) takes level
    ceil(log2(size)), splitting the nearest non-empty higher level; children
    are appended unsorted (chunk_pool.py:52-59); the lowest-position id is
    popped (chunk_pool.py:73); free() merges with buddy id^1 upward using a
    bisect insert (chunk_pool.py:76-96)."""

    def __init__(self, height: int):
        self.height = height
        self.available = [[] for _ in range(height)]
        self.available[height - 1] = [0]

    def alloc(self, size: int) -> tuple[int, int]:
        level = math.ceil(math.log2(size))
        if not self.available[level]:
            for i in range(level + 1, self.height):
                if self.available[i]:
                    for lv in range(i, level, -1):
                        parent = self.available[lv].pop()
                        self.available[lv - 1].extend([2 * parent, 2 * parent + 1])
                    break
        if not self.available[level]:
            raise RuntimeError(f"Failed to allocate chunks for size {size} on level {level}")
        return self.available[level].pop(0), level

    def free(self, cid: int, level: int) -> None:
        for lv in range(level, self.height):
            ids = self.available[lv]
            pos = bisect.bisect_left(ids, cid)
            if pos != 0 and (ids[pos - 1] ^ 1) == cid:
                ids.pop(pos - 1)
                cid //= 2
            elif pos != len(ids) and (ids[pos] ^ 1) == cid:
                ids.pop(pos)
                cid //= 2
            else:
                ids.insert(pos, cid)
                break

    @staticmethod
    def row_range(cid: int, level: int, num_layers: int) -> tuple[int, int]:
        """Rows of the chunk in the pool tensor (chunk_pool.py:20-23)."""
        return cid * (2**level) * num_layers, (cid + 1) * (2**level) * num_layers
