"""Per-step ragged-batch descriptors (reference: deserve_worker/model/context/
forward.py:8-18 and flash.py:17-120).

The reference builds five small device tensors with a Python loop of device
slices, a torch.cat and five host->device copies. Here the loop only touches
host integers (page tables live in host memory); everything is packed into one
pinned int32 buffer and sent with a single asynchronous copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

from . import _lib
from .pinned import COUNTERS as _COUNTERS, ring as _pinned_ring
from .kvcache import PagedKVCache, PagePool
from .task import TaskData


@dataclass
class ForwardCtx:
    bsz: int
    seqlens: torch.Tensor
    layer_id: int


@dataclass
class PagedForwardCtx(ForwardCtx):
    page_pool: PagePool
    offsets: torch.Tensor


_NAMES = ("indptr", "kv_page_indptr", "kv_last_page_lens", "offsets", "seqlens", "kv_page_indices")


def build_step(task_datas: list[TaskData], kvcaches: list[PagedKVCache], buf: np.ndarray | None = None):
    """Grow every cache for this step and write the six descriptor arrays into one
    packed int32 buffer, in ONE native call (dsv_host_build_step). For a chunked
    prefill the cache is grown to the whole prompt on the first chunk while the
    descriptors cover only start_pos + seqlen tokens. Returns (buffer, views)."""
    bsz = len(task_datas)
    pool = kvcaches[0].pool
    alloc = kvcaches[0].page_table.allocator
    ps = pool.page_size
    start = np.fromiter((t.start_pos for t in task_datas), dtype=np.int32, count=bsz)
    seqlen = np.fromiter((t.seqlen for t in task_datas), dtype=np.int32, count=bsz)
    initial = np.fromiter((t.initial_seqlen for t in task_datas), dtype=np.int32, count=bsz)
    slot = np.fromiter((kv.page_table.offset for kv in kvcaches), dtype=np.int32, count=bsz)
    occupied = np.fromiter((kv.page_table.occupied for kv in kvcaches), dtype=np.int32, count=bsz)
    n_idx = int(((start + seqlen + ps - 1) // ps).sum())
    cap = 5 * (bsz + 4) + n_idx + 4
    if buf is None or buf.size < cap:
        buf = np.empty(cap, dtype=np.int32)
    offs = np.zeros(7, dtype=np.int64)
    failed = np.full(2, -1, dtype=np.int32)
    main = getattr(pool, "num_pages_main", -1)
    isswap = alloc._isswap_np if main >= 0 else None
    with pool.mutex:
        rc = _lib.lib.dsv_host_build_step(
            pool._bitmap.ctypes.data, pool.num_pages, pool._buf_store.ctypes.data, pool._buf_store.size,
            pool._buf_win[0:].ctypes.data, pool._buf_win[1:].ctypes.data, pool._avails.ctypes.data, pool.fetch_size, ps,
            main, alloc._tables_np.ctypes.data, None if isswap is None else isswap.ctypes.data,
            alloc._tables_np.shape[1], bsz, slot.ctypes.data, occupied.ctypes.data, start.ctypes.data,
            seqlen.ctypes.data, initial.ctypes.data, buf.ctypes.data, buf.size, offs.ctypes.data,
            failed[0:].ctypes.data, failed[1:].ctypes.data)
    for kv, occ in zip(kvcaches, occupied.tolist()):  # also after a failure: earlier requests stay grown
        kv.page_table.occupied = occ
    if rc == _lib.E_WORKSPACE and failed[0] >= 0:
        raise ValueError(f"Not enough pages {int(failed[1])} > {pool.num_avails}")
    _lib.check(rc)
    sizes = (bsz + 1, bsz + 1, bsz, bsz, bsz, n_idx)
    views = {n: buf[int(o) : int(o) + sz] for n, o, sz in zip(_NAMES, offs[:6], sizes)}
    if getattr(pool, "rows_used", None) is not None and n_idx:
        # the swap regions learn how many token rows of their pages this step's requests fill
        kvp, idx = views["kv_page_indptr"], views["kv_page_indices"]
        has = kvp[1:] > kvp[:-1]
        pool.note_rows(idx, idx[kvp[1:][has] - 1], views["kv_last_page_lens"][has])
    return buf, int(offs[6]), views


def pack_descriptors(task_datas: list[TaskData], kvcaches: list[PagedKVCache]) -> dict[str, np.ndarray]:
    """The descriptor arrays of a step on the host (caches are grown as a side effect)."""
    return build_step(task_datas, kvcaches)[2]


@dataclass
class FlashForwardCtx(PagedForwardCtx):
    indptr: torch.Tensor
    kv_page_indices: torch.Tensor
    kv_page_indptr: torch.Tensor
    kv_last_page_lens: torch.Tensor
    # host copies of the descriptor arrays: views of a pinned buffer that is reused once 15 later steps have
    # been prepared, i.e. valid for this step (planning, bookkeeping), not to be kept
    host: dict[str, np.ndarray] = field(default_factory=dict, repr=False)

    @staticmethod
    def init_paged_forward_ctx(task_datas: list[TaskData], kvcaches: list[PagedKVCache]) -> "FlashForwardCtx":
        pool = kvcaches[0].pool
        on_gpu = pool.main_device.type == "cuda"
        bsz = len(task_datas)
        ps = pool.page_size
        cap = 5 * (bsz + 4) + sum((t.start_pos + t.seqlen + ps - 1) // ps for t in task_datas) + 4
        if on_gpu:
            pinned, slot = _pinned_ring("descriptors", slots=16).take(cap)
        else:
            pinned = torch.empty(cap, dtype=torch.int32)
        _, used, host = build_step(task_datas, kvcaches, pinned.numpy())
        if on_gpu:
            dev = pinned[:used].to(pool.main_device, non_blocking=True)
            _pinned_ring("descriptors").done(slot)
            _COUNTERS["h2d_bytes"] += used * 4
        else:
            dev = pinned
        starts = {n: host[n].ctypes.data - pinned.data_ptr() for n in _NAMES}
        t = {n: dev[starts[n] // 4 : starts[n] // 4 + len(host[n])] for n in _NAMES}
        ctx = FlashForwardCtx(
            bsz=bsz, seqlens=t["seqlens"], layer_id=0, page_pool=pool, offsets=t["offsets"],
            indptr=t["indptr"], kv_page_indices=t["kv_page_indices"], kv_page_indptr=t["kv_page_indptr"],
            kv_last_page_lens=t["kv_last_page_lens"], host=host)
        ctx._pinned = pinned  # `host` are views of it
        return ctx


@dataclass
class FlashDecodeCtx(FlashForwardCtx):
    decode_wrapper: Any = None

    @staticmethod
    def init_paged_decode_ctx(task_datas, kvcaches, wrapper) -> "FlashDecodeCtx":
        c = FlashForwardCtx.init_paged_forward_ctx(task_datas, kvcaches)
        return FlashDecodeCtx(**{k: getattr(c, k) for k in c.__dataclass_fields__}, decode_wrapper=wrapper)


@dataclass
class FlashPrefillCtx(FlashForwardCtx):
    prefill_wrapper: Any = None

    @staticmethod
    def init_paged_prefill_ctx(task_datas, kvcaches, wrapper) -> "FlashPrefillCtx":
        c = FlashForwardCtx.init_paged_forward_ctx(task_datas, kvcaches)
        return FlashPrefillCtx(**{k: getattr(c, k) for k in c.__dataclass_fields__}, prefill_wrapper=wrapper)
