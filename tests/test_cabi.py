"""The C ABI itself: every symbol of include/deserve_kv.h is exported, argument
validation answers with error codes before any launch, and the host-side decode
planner covers every page exactly once. No GPU needed."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

from deserve_b200 import _lib, ops

HEADER = Path(__file__).resolve().parent.parent / "include" / "deserve_kv.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return re.findall(r"\b(dsv_\w+)\s*\(", text)


def test_every_declared_symbol_is_exported():
    names = declared_symbols()
    assert len(names) >= 12 and len(set(names)) == len(names)
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} is declared in deserve_kv.h but not exported"
        assert n in _lib._SIGNATURES, f"{n} has no ctypes signature"
    assert _lib.lib.dsv_version() == 100


def test_invalid_arguments_return_codes_not_crashes():
    L = _lib.lib
    assert L.dsv_append_paged_kv(None, None, 0, 0, None, None, 0, 4, None, None, None, 1, 1, 8, 128, 16, 2, None) == -1
    assert "null pointer" in _lib.last_error()
    assert L.dsv_append_paged_kv(None, None, 0, 0, None, None, 0, 4, None, None, None, 1, 1, 8, 128, 16, 9, None) == -1
    assert "dtype" in _lib.last_error()
    # nothing to do is not an error
    assert L.dsv_append_paged_kv(None, None, 0, 0, None, None, 0, 4, None, None, None, 0, 0, 8, 128, 16, 2, None) == 0
    assert L.dsv_region_swap(None, 4, 1024, 512, 1024, 1024, 1024, None, None, None, None, None, 0, 0, 0, 0) == 0  # both directions skipped
    buf = (ctypes.c_char * 64)()
    assert L.dsv_region_swap(buf, 4, 1024, 512, 1024, 1024, 0, buf, None, None, None, None, 0, 0, 0, 0) == -1
    assert "outside a layer" in _lib.last_error()
    # rows beyond the page, or byte counts that are not whole pages, are refused before any copy
    assert L.dsv_region_swap(buf, 4, 4096, 512, 1024, 1024, 0, buf, None, None, None, None, 512, 16, 17, 0) == -1
    assert L.dsv_region_swap(buf, 4, 4096, 512, 1024, 768, 0, buf, None, None, None, None, 512, 16, 4, 0) == -1
    assert "whole pages" in _lib.last_error()
    assert L.dsv_region_swap(buf, 4, 4096, 512, 1024, 2048, 0, buf, None, None, None, None, 0, 0, 0, 0) == -1
    assert "out_bytes" in _lib.last_error()
    assert L.dsv_pack_pages(buf, 1024, 100, 4, buf, buf, 1, 1, 0, 1, buf, None) == -1
    assert "multiple of 16" in _lib.last_error()
    # a layer slab that cannot hold num_pages pages is refused before anything is launched
    assert L.dsv_pack_pages(buf, 1024, 256, 5, buf, buf, 1, 1, 0, 1, buf, None) == -1
    assert "cannot hold" in _lib.last_error()
    assert L.dsv_unpack_pages(buf, buf, 1024, 256, 0, buf, buf, 1, 1, 0, 1, None) == -1
    assert "num_pages" in _lib.last_error()
    with pytest.raises(ValueError):
        _lib.check(-1)
    with pytest.raises(_lib.DeserveKVError):
        _lib.check(-3)


def _plan(n_pages, hq=32, hkv=8, d=128, ps=16, sms=148):
    indptr = np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32)
    plan = np.zeros(ops.plan_capacity(len(n_pages), sms), dtype=np.int32)
    used, ws = ops.make_decode_plan(indptr, hq, hkv, d, ps, torch.bfloat16, sms, plan)
    return plan[:used], ws


@pytest.mark.parametrize("seed,batch,lo,hi", [(0, 256, 32, 256), (1, 4, 7, 19), (2, 1, 4000, 4000), (3, 700, 1, 3),
                                              (4, 5, 0, 2), (5, 128, 32, 48), (6, 64, 32, 256), (7, 16, 256, 256),
                                              (8, 130, 20, 90), (9, 300, 5, 9)])
def test_decode_plan_covers_every_page_once(seed, batch, lo, hi):
    rng = np.random.default_rng(seed)
    n_pages = rng.integers(lo, hi + 1, size=batch)
    plan, ws = _plan(n_pages)
    n_items, slots, chunk, b = plan[1], plan[2], plan[3], plan[4]
    assert b == batch and plan[5] == 8 and plan[6] == 8 + 4 * n_items
    items = plan[8 : 8 + 4 * n_items].reshape(-1, 4)
    merge = plan[plan[6] : plan[6] + 2 * batch].reshape(-1, 2)
    cover = [np.zeros(n, dtype=int) for n in n_pages]
    for req, pb, pe, slot in items:
        assert 0 <= pb <= pe <= n_pages[req] and pe - pb <= chunk
        cover[req][pb:pe] += 1
        if merge[req][1] > 1:
            assert merge[req][0] <= slot < merge[req][0] + merge[req][1]
        else:
            assert slot == -1
    assert all((c == 1).all() for c in cover)
    assert np.bincount(items[:, 0], minlength=batch).tolist() == merge[:, 1].tolist()
    used_slots = sorted(s for s in items[:, 3] if s >= 0)
    assert used_slots == list(range(slots))
    assert ws == slots * 32 * (128 + 2) * 4
    sizes = items[:, 2] - items[:, 1]
    assert (np.diff(sizes) <= 0).all()  # longest first


def test_decode_plan_keeps_a_small_microbatch_unsplit():
    """128 sequences with 512-768 tokens (the 70B pipeline's microbatch) stream 0.3 GB per launch: one item
    per request on 128 of the 148 SMs and no merge launch beats three short items per request."""
    n_pages = (np.random.default_rng(0).integers(512, 769, size=128) + 15) // 16
    plan, ws = _plan(n_pages, hq=64)
    assert plan[1] == 128 and plan[2] == 0 and ws == 0 and plan[3] == n_pages.max()
    # a single long request still spreads over the machine
    plan, _ = _plan(np.array([2048]))
    assert plan[1] >= 100


def test_decode_plan_balances_the_llama8b_batch():
    rng = np.random.default_rng(0)
    n_pages = (rng.integers(512, 4097, size=256) + 15) // 16
    plan, _ = _plan(n_pages)
    assert 256 <= plan[1] <= 4 * 148 + 256
    sizes = plan[8 : 8 + 4 * plan[1]].reshape(-1, 4)
    sizes = sizes[:, 2] - sizes[:, 1]
    assert sizes.max() <= plan[3] and sizes.min() >= min(n_pages.min(), plan[3] // 2)


def test_decode_plan_rejects_bad_input():
    with pytest.raises(ValueError):
        _plan([3, 4], hq=30, hkv=8)
    with pytest.raises(ValueError):
        _plan([3, 4], d=96)
    plan = np.zeros(4, dtype=np.int32)
    with pytest.raises(_lib.DeserveKVError, match="plan needs"):
        ops.make_decode_plan(np.array([0, 5], dtype=np.int32), 8, 2, 64, 16, torch.float32, 148, plan)


@pytest.mark.parametrize("causal", [True, False])
def test_prefill_plan_tiles_every_new_token_once(causal, monkeypatch):
    monkeypatch.setenv("DESERVE_PREFILL_PAIRS", "1")
    qo = np.array([0, 100, 101, 613, 613, 650], dtype=np.int32)
    kv_len = np.array([100, 900, 1024, 7, 37], dtype=np.int32)
    plan = np.zeros(ops.prefill_plan_capacity(650, 5, 4), dtype=np.int32)
    used = ops.make_prefill_plan(qo, kv_len, 32, 8, 128, 16, torch.bfloat16, causal, plan)
    n_items, tq, n_pairs = plan[1], plan[2], plan[8]
    assert tq == 32 and used == 12 + 4 * (n_items + n_pairs) and plan[3] == int(causal)
    assert plan[5] == 12 and plan[9] == 12 + 4 * n_items
    singles = plan[12 : 12 + 4 * n_items].reshape(-1, 4)
    pairs = plan[plan[9] : used].reshape(-1, 4)
    cover = [np.zeros(n, dtype=int) for n in np.diff(qo)]
    # head_dim 128: a pair item is two q tiles (one per CTA of a cluster), a single-CTA item a lone last tile
    for lo, hi_, items in ((0, tq, singles), (tq, 2 * tq, pairs)):
        for req, q0, nq, hi in items:
            assert lo < nq <= hi_ and q0 % (2 * tq) == 0
            cover[req][q0 : q0 + nq] += 1
            n = qo[req + 1] - qo[req]
            assert hi == (kv_len[req] - n + q0 + nq if causal else kv_len[req])
        # most work first, a request's items together (they read the same K/V): requests by their longest
        # item over both lists, inside a request the longest item first
        reqs = items[:, 0].tolist()
        order = [r for k, r in enumerate(reqs) if k == 0 or reqs[k - 1] != r]
        assert len(order) == len(set(order))
        every = np.concatenate([singles, pairs])
        longest = {int(r): int(every[every[:, 0] == r][:, 3].max()) for r in set(every[:, 0].tolist())}
        assert all(longest[x] >= longest[y] for x, y in zip(order, order[1:]))
        for r in order:
            assert (np.diff(items[items[:, 0] == r][:, 3]) <= 0).all()
    assert all((c == 1).all() for c in cover)
    assert n_pairs == 11 and n_items == 1  # 100 -> 64 + 36; 1 -> a single; 512 -> 8 x 64; 37 -> one pair


def test_prefill_plan_head_dim_64_has_no_pair_items():
    qo = np.array([0, 300], dtype=np.int32)
    plan = np.zeros(ops.prefill_plan_capacity(300, 1, 4), dtype=np.int32)
    ops.make_prefill_plan(qo, np.array([300], dtype=np.int32), 8, 2, 64, 16, torch.float16, True, plan)
    assert plan[8] == 0 and plan[1] == 5  # 300 tokens in items of 64


def test_prefill_plan_rejects_inconsistent_lengths():
    plan = np.zeros(64, dtype=np.int32)
    with pytest.raises(ValueError, match="new tokens"):
        ops.make_prefill_plan(np.array([0, 50], dtype=np.int32), np.array([20], dtype=np.int32), 8, 2, 64, 16,
                              torch.float16, True, plan)
