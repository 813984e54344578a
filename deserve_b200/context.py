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


def _ceil4(n: int) -> int:
    return (n + 3) & ~3


def pack_descriptors(task_datas: list[TaskData], kvcaches: list[PagedKVCache]) -> dict[str, np.ndarray]:
    """Grow every cache for this step and return the descriptor arrays on the
    host. For a chunked prefill the cache is grown to the whole prompt on the
    first chunk while the descriptors cover only start_pos + seqlen tokens."""
    bsz = len(task_datas)
    n_pages = np.empty(bsz, dtype=np.int32)
    last = np.empty(bsz, dtype=np.int32)
    seqlens = np.empty(bsz, dtype=np.int32)
    offsets = np.empty(bsz, dtype=np.int32)
    rows = []
    for i, (task, kv) in enumerate(zip(task_datas, kvcaches)):
        ps = kv.pool.page_size
        cur = task.start_pos + task.seqlen
        kv.extend(max(cur, task.initial_seqlen))
        n_pages[i] = (cur + ps - 1) // ps
        last[i] = (cur - 1) % ps + 1
        seqlens[i] = task.seqlen
        offsets[i] = task.start_pos
        rows.append(kv.page_table.allocator._tables_np[kv.page_table.offset, : n_pages[i]])
    indptr = np.zeros(bsz + 1, dtype=np.int32)
    np.cumsum(seqlens, out=indptr[1:])
    kv_page_indptr = np.zeros(bsz + 1, dtype=np.int32)
    np.cumsum(n_pages, out=kv_page_indptr[1:])
    kv_page_indices = np.concatenate(rows) if rows else np.zeros(0, dtype=np.int32)
    return {"indptr": indptr, "kv_page_indptr": kv_page_indptr, "kv_last_page_lens": last, "offsets": offsets,
            "seqlens": seqlens, "kv_page_indices": kv_page_indices}


@dataclass
class FlashForwardCtx(PagedForwardCtx):
    indptr: torch.Tensor
    kv_page_indices: torch.Tensor
    kv_page_indptr: torch.Tensor
    kv_last_page_lens: torch.Tensor
    host: dict[str, np.ndarray] = field(default_factory=dict, repr=False)

    @staticmethod
    def init_paged_forward_ctx(task_datas: list[TaskData], kvcaches: list[PagedKVCache]) -> "FlashForwardCtx":
        host = pack_descriptors(task_datas, kvcaches)
        pool = kvcaches[0].pool
        names = ["indptr", "kv_page_indptr", "kv_last_page_lens", "offsets", "seqlens", "kv_page_indices"]
        sizes = [len(host[n]) for n in names]
        starts = np.concatenate([[0], np.cumsum([_ceil4(s) for s in sizes])])
        on_gpu = pool.main_device.type == "cuda"
        buf = torch.empty(int(starts[-1]), dtype=torch.int32, pin_memory=on_gpu)
        buf_np = buf.numpy()
        for n, s, sz in zip(names, starts, sizes):
            buf_np[s : s + sz] = host[n]
        dev = buf.to(pool.main_device, non_blocking=True) if on_gpu else buf
        t = {n: dev[s : s + sz] for n, s, sz in zip(names, starts, sizes)}
        return FlashForwardCtx(
            bsz=len(task_datas), seqlens=t["seqlens"], layer_id=0, page_pool=pool, offsets=t["offsets"],
            indptr=t["indptr"], kv_page_indices=t["kv_page_indices"], kv_page_indptr=t["kv_page_indptr"],
            kv_last_page_lens=t["kv_last_page_lens"], host=host)


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
