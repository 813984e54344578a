"""Task stepping and the per-step ragged-batch descriptors of the reference."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class OracleTask:
    """deserve_worker/task.py:26-65 (fields that drive the index arithmetic)."""

    start_pos: int = 0
    seqlen: int = 0
    initial_seqlen: int = 0
    round: int = 0

    def init(self, seqlen: int) -> None:  # task.py:48-49
        self.seqlen = seqlen

    def step(self) -> None:  # task.py:57-65
        assert self.seqlen > 0
        self.start_pos += self.seqlen
        self.seqlen = 1 if self.start_pos >= self.initial_seqlen else 0
        self.round += 1


def build_descriptors(tasks, caches, page_size: int) -> dict[str, np.ndarray]:
    """deserve_worker/model/context/flash.py:24-70.

    For each task: total = max(start+seqlen, initial) is what the cache is grown
    to (chunked prefill pre-allocates the whole prompt, flash.py:31-39); the
    descriptors cover only cur = start+seqlen tokens: ceil(cur/ps) pages and
    (cur-1) % ps + 1 tokens in the last one (flash.py:35-37)."""
    last, rows = [], []
    for task, cache in zip(tasks, caches):
        total = max(task.start_pos + task.seqlen, task.initial_seqlen)
        cur = task.start_pos + task.seqlen
        n_pages = (cur + page_size - 1) // page_size
        last.append((cur - 1) % page_size + 1)
        cache.extend(total)
        rows.append(np.array(cache.page_ids()[:n_pages], dtype=np.int32))
    seqlens = [t.seqlen for t in tasks]
    return {
        "indptr": np.cumsum([0] + seqlens).astype(np.int32),
        "kv_page_indices": np.concatenate(rows).astype(np.int32) if rows else np.zeros(0, np.int32),
        "kv_page_indptr": np.cumsum([0] + [len(r) for r in rows]).astype(np.int32),
        "kv_last_page_lens": np.array(last, dtype=np.int32),
        "offsets": np.array([t.start_pos for t in tasks], dtype=np.int32),
        "seqlens": np.array(seqlens, dtype=np.int32),
    }
