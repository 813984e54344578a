"""KV swap data movement of the reference, restated with CPU tensors."""
from __future__ import annotations

import numpy as np
import torch


def region_swap(pages: torch.Tensor, lo: int, hi: int, host_out: torch.Tensor | None, host_in: torch.Tensor | None) -> None:
    """deserve_worker/kvcache/virtual.py:97-113 with the host buffer in the
    pool's own dtype: host_out viewed as (L, swap, 2, ps, Hkv, D) receives
    pages[:, lo:hi], then pages[:, lo:hi] is filled from host_in."""
    shape = (pages.shape[0], hi - lo, *pages.shape[2:])
    if host_out is not None:
        host_out.view(shape).copy_(pages[:, lo:hi])
    if host_in is not None:
        pages[:, lo:hi].copy_(host_in.view(shape))


def offload_rows(pages: torch.Tensor, page_ids: np.ndarray) -> torch.Tensor:
    """deserve_worker/kvcache/manager.py:38-44: rows of the host chunk for one
    task, layer-major (row l*n + p = pages[l, ids[p]]): [L*n, 2, ps, Hkv, D]."""
    ids = torch.as_tensor(np.asarray(page_ids, dtype=np.int64))
    sel = pages[:, ids]
    return sel.reshape(sel.shape[0] * sel.shape[1], *sel.shape[2:]).clone()


def reload_rows(pages: torch.Tensor, new_ids: np.ndarray, rows: torch.Tensor) -> None:
    """deserve_worker/kvcache/manager.py:63-73: scatter a chunk's rows into
    freshly allocated page ids: pages[:, new_ids] = rows.view(L, n, ...)."""
    ids = torch.as_tensor(np.asarray(new_ids, dtype=np.int64))
    n = len(ids)
    pages[:, ids] = rows[: pages.shape[0] * n].view(pages.shape[0], n, *pages.shape[2:])
