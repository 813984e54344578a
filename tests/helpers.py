"""Shared test scaffolding: golden fixtures and seeded paged-KV scenarios."""
from __future__ import annotations

import hashlib
import json
from functools import lru_cache
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


@lru_cache(maxsize=None)
def host_traces() -> dict:
    return json.loads((GOLDEN / "host_traces.json").read_text())


@lru_cache(maxsize=None)
def dense_attention() -> dict:
    return dict(np.load(GOLDEN / "dense_attention.npz"))


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def bits(s: str) -> np.ndarray:
    return np.array([c == "1" for c in s], dtype=bool)


def random_descriptors(seed: int, batch: int, len_lo: int, len_hi: int, page_size: int, pool_factor: float = 1.25,
                       new_tokens=None) -> tuple[dict, int]:
    """Descriptors of a batch whose pages are dealt from a seeded random
    permutation of a pool sized pool_factor x the pages in use. Returns
    (descriptors as numpy int32 arrays, number of pages in the pool)."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(len_lo, len_hi + 1, size=batch)
    n_pages = (lens + page_size - 1) // page_size
    total = int(n_pages.sum())
    pool_pages = int(np.ceil(total * pool_factor)) + 1
    perm = rng.permutation(pool_pages)[:total].astype(np.int32)
    if new_tokens is None:
        new_tokens = np.ones(batch, dtype=np.int64)
    new_tokens = np.minimum(np.asarray(new_tokens), lens)
    desc = {
        "indptr": np.concatenate([[0], np.cumsum(new_tokens)]).astype(np.int32),
        "kv_page_indices": perm,
        "kv_page_indptr": np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32),
        "kv_last_page_lens": ((lens - 1) % page_size + 1).astype(np.int32),
        "offsets": (lens - new_tokens).astype(np.int32),
        "seqlens": new_tokens.astype(np.int32),
    }
    return desc, pool_pages


def to_device(desc: dict, device) -> dict:
    return {k: torch.from_numpy(np.ascontiguousarray(v)).to(device) for k, v in desc.items()}
