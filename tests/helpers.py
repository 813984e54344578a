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


def lattice(seed: int, shape, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Seeded values k/64, k in [-128, 128]: exact in fp16 and bf16, and from a
    generator (numpy's legacy MT19937 stream) that does not change between
    library versions, so fixtures made elsewhere can be rebuilt here bit for bit."""
    vals = np.random.RandomState(seed).randint(-128, 129, size=tuple(shape)).astype(np.float32) / 64.0
    return torch.from_numpy(vals).to(dtype)


def table_descriptors(seed: int, lens, new_tokens, page_size: int) -> tuple[dict, int]:
    """Descriptors for requests of the given post-append lengths, the last
    new_tokens[i] of which are new; pages dealt from a seeded (legacy numpy
    stream) permutation of a pool 1.25 x the pages in use."""
    lens = np.asarray(lens, dtype=np.int64)
    new_tokens = np.asarray(new_tokens, dtype=np.int64)
    n_pages = (lens + page_size - 1) // page_size
    total = int(n_pages.sum())
    pool_pages = total + total // 4 + 1
    perm = np.random.RandomState(seed).permutation(pool_pages)[:total].astype(np.int32)
    desc = {
        "indptr": np.concatenate([[0], np.cumsum(new_tokens)]).astype(np.int32),
        "kv_page_indices": perm,
        "kv_page_indptr": np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32),
        "kv_last_page_lens": ((lens - 1) % page_size + 1).astype(np.int32),
        "offsets": (lens - new_tokens).astype(np.int32),
        "seqlens": new_tokens.astype(np.int32),
    }
    return desc, pool_pages


FLASHINFER_CASES = {
    # name: (n_q_heads, n_kv_heads, head_dim, page_size, dtype, post-append lengths, new tokens, seed)
    "decode_8b": (32, 8, 128, 16, "bfloat16", [2, 16, 17, 18, 100, 257, 512, 1025], [1] * 8, 11),
    "decode_small_f16": (8, 2, 64, 16, "float16", [3, 16, 33, 300], [1] * 4, 12),
    "decode_70b": (64, 8, 128, 16, "bfloat16", [48, 129, 700], [1] * 3, 13),
    "prefill_chunks": (8, 2, 128, 16, "bfloat16", [300, 17, 200, 100], [1, 17, 64, 100], 14),
    "prefill_8b": (32, 8, 128, 16, "bfloat16", [64, 133], [33, 5], 15),
}


def flashinfer_case_inputs(name: str):
    """Inputs of one recorded flashinfer case: descriptors of the prefix append
    (everything before the new tokens), descriptors of the step itself, the K/V
    rows of both appends and the step's queries."""
    hq, hkv, d, ps, dt, lens, new, seed = FLASHINFER_CASES[name]
    dtype = getattr(torch, dt)
    lens, new = np.asarray(lens), np.asarray(new)
    step, pool_pages = table_descriptors(seed, lens, new, ps)
    prefix_lens = lens - new
    # the prefix uses the same page lists, cut to the pages its tokens reach
    n_pre = (prefix_lens + ps - 1) // ps
    idx = [step["kv_page_indices"][step["kv_page_indptr"][i]: step["kv_page_indptr"][i] + n_pre[i]]
           for i in range(len(lens))]
    prefix = {
        "indptr": np.concatenate([[0], np.cumsum(prefix_lens)]).astype(np.int32),
        "kv_page_indices": np.concatenate(idx).astype(np.int32) if idx else np.zeros(0, np.int32),
        "kv_page_indptr": np.concatenate([[0], np.cumsum(n_pre)]).astype(np.int32),
        "kv_last_page_lens": np.where(prefix_lens > 0, (prefix_lens - 1) % ps + 1, 0).astype(np.int32),
        "offsets": np.zeros(len(lens), np.int32),
        "seqlens": prefix_lens.astype(np.int32),
    }
    n_prefix, n_new = int(prefix_lens.sum()), int(new.sum())
    return {
        "hq": hq, "hkv": hkv, "d": d, "ps": ps, "dtype": dtype, "pool_pages": pool_pages,
        "prefix": prefix, "step": step,
        "k_prefix": lattice(seed * 10 + 1, (n_prefix, hkv, d), dtype),
        "v_prefix": lattice(seed * 10 + 2, (n_prefix, hkv, d), dtype),
        "k_new": lattice(seed * 10 + 3, (n_new, hkv, d), dtype),
        "v_new": lattice(seed * 10 + 4, (n_new, hkv, d), dtype),
        "q": lattice(seed * 10 + 5, (n_new, hq, d), dtype),
    }


@lru_cache(maxsize=None)
def flashinfer_golden() -> tuple[dict, dict]:
    """(arrays, metadata) recorded from flashinfer on a B200 by
    tests/golden/make_flashinfer_golden.py."""
    meta = json.loads((GOLDEN / "flashinfer_golden.json").read_text())
    return dict(np.load(GOLDEN / "flashinfer_golden.npz")), meta
