"""Ragged causal paged prefill attention (tcgen05 kernel) against the fp32 oracle:
whole prompts, chunked prefill on top of an existing context, mixed prefill +
decode batches, lengths around tile and page boundaries."""
import numpy as np
import pytest
import torch

import deserve_b200 as dk
from deserve_b200 import _lib, ops
from helpers import random_descriptors, to_device
from oracle import kv_math

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.fixture(autouse=True, params=["single", "pairs"])
def _device_status_clean(request, monkeypatch):
    # every case runs twice: single-CTA items only, and with the two-CTA pair kernel taking the items of
    # more than one q tile (head_dim 128)
    monkeypatch.setenv("DESERVE_PREFILL_PAIRS", "1" if request.param == "pairs" else "0")
    yield
    assert _lib.read_device_status() == 0, "a kernel self-check fired"


def _run(seed, kv_lens, new_tokens, hq, hkv, d, ps, dtype, causal=True, poison=False):
    batch = len(kv_lens)
    rng = np.random.default_rng(seed)
    kv_lens, new_tokens = np.asarray(kv_lens), np.asarray(new_tokens)
    n_pages = (kv_lens + ps - 1) // ps
    total = int(n_pages.sum())
    pool_pages = int(total * 1.25) + 2
    desc = {
        "indptr": np.concatenate([[0], np.cumsum(new_tokens)]).astype(np.int32),
        "kv_page_indices": rng.permutation(pool_pages)[:total].astype(np.int32),
        "kv_page_indptr": np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32),
        "kv_last_page_lens": ((kv_lens - 1) % ps + 1).astype(np.int32),
    }
    g = torch.Generator().manual_seed(seed)
    pages = (torch.randn(pool_pages, 2, ps, hkv, d, generator=g) * 0.5).to(dtype)
    if poison:  # slots past the end of each request's last page must never leak
        for i in range(batch):
            last_page = desc["kv_page_indices"][desc["kv_page_indptr"][i + 1] - 1]
            pages[last_page, :, desc["kv_last_page_lens"][i]:] = float("nan")
    nnz = int(desc["indptr"][-1])
    q = torch.randn(nnz, hq, d, generator=g).to(dtype)
    want = kv_math.paged_attention(q, pages, desc, ps, causal=causal)
    ws = torch.empty(32 << 20, dtype=torch.uint8, device=DEV)
    wrapper = dk.BatchPrefillWithPagedKVCacheWrapper(ws)
    dd = to_device(desc, DEV)
    wrapper.begin_forward(dd["indptr"], dd["kv_page_indptr"], dd["kv_page_indices"], dd["kv_last_page_lens"], hq, hkv, d,
                          ps, data_type=dtype, causal=causal, qo_indptr_host=desc["indptr"],
                          kv_indptr_host=desc["kv_page_indptr"], last_page_len_host=desc["kv_last_page_lens"])
    got = wrapper.forward(q.to(DEV), pages.to(DEV), causal=causal)
    wrapper.end_forward()
    torch.cuda.synchronize()
    assert got.shape == (nnz, hq, d) and got.dtype == dtype
    err = (got.float().cpu() - want).abs()
    return err.max().item(), err


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_whole_prompt_prefill(dtype):
    err, _ = _run(1, [100, 37, 16, 513, 128], [100, 37, 16, 513, 128], 32, 8, 128, 16, dtype)
    assert err <= 2e-2, f"max-abs error {err}"


@pytest.mark.parametrize("hq,hkv,d,ps", [(32, 8, 128, 16), (64, 8, 128, 16), (8, 2, 64, 16), (8, 8, 128, 8),
                                         (16, 1, 64, 32), (4, 4, 64, 4)])
def test_chunked_prefill_on_existing_context(hq, hkv, d, ps):
    # chunk of new tokens appended after an older context; q rows align to the END of the kv sequence
    err, _ = _run(2, [700, 300, 1029, 64], [512, 44, 5, 64], hq, hkv, d, ps, torch.bfloat16, poison=True)
    assert err <= 2e-2, f"max-abs error {err}"


def test_mixed_prefill_and_decode_rows():
    # rows with one new token and a long context go to the decode kernel, the chunks to the prefill kernel
    err, _ = _run(3, [2000, 17, 900, 1, 333, 4000], [1, 17, 1, 1, 200, 1], 32, 8, 128, 16, torch.bfloat16, poison=True)
    assert err <= 2e-2, f"max-abs error {err}"


def test_all_rows_are_decode_rows_through_the_prefill_wrapper():
    err, _ = _run(8, [300, 64, 1500], [1, 1, 1], 32, 8, 128, 16, torch.bfloat16, poison=True)
    assert err <= 2e-2, f"max-abs error {err}"


def test_small_workspace_keeps_decode_rows_in_the_prefill_kernel():
    import deserve_b200.ops as o
    saved = o.BatchPrefillWithPagedKVCacheWrapper.SPLIT_MIN_KV
    o.BatchPrefillWithPagedKVCacheWrapper.SPLIT_MIN_KV = 1 << 30  # never split: the tensor-core kernel handles n = 1 rows too
    try:
        err, _ = _run(3, [2000, 17, 900, 1, 333], [1, 17, 1, 1, 200], 32, 8, 128, 16, torch.bfloat16, poison=True)
    finally:
        o.BatchPrefillWithPagedKVCacheWrapper.SPLIT_MIN_KV = saved
    assert err <= 2e-2, f"max-abs error {err}"


def test_tile_and_page_boundaries():
    lens = [127, 128, 129, 255, 256, 257, 15, 16, 17, 1]
    err, _ = _run(4, lens, lens, 8, 2, 64, 16, torch.float16, poison=True)
    assert err <= 2e-2, f"max-abs error {err}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_pair_items_around_block_and_tile_boundaries(dtype):
    # head_dim 128, GQA 4: every 64 new tokens (two q tiles) are worked by a cluster of two CTAs, the
    # two softmax groups of a CTA taking alternate 128-token K/V blocks. Lengths around the tile and
    # block sizes, one to many blocks, ragged last blocks (not a multiple of 16: the poisoned tail of
    # the last page must not leak), items whose second tile is partly or wholly empty, a context of 0.
    new = [65, 96, 97, 128, 129, 191, 192, 193, 70, 300]
    ctx = [0, 31, 0, 64, 1000, 63, 7, 515, 2041, 1]
    lens = [c + n for c, n in zip(ctx, new)]
    err, _ = _run(11, lens, new, 32, 8, 128, 16, dtype, poison=True)
    assert err <= 2e-2, f"max-abs error {err}"


def test_pair_items_non_causal_and_wide_group():
    err, _ = _run(12, [700, 333, 129], [130, 333, 129], 64, 8, 128, 16, torch.bfloat16, causal=False, poison=True)
    assert err <= 2e-2, f"max-abs error {err}"
    err, _ = _run(13, [1100, 600], [1030, 270], 4, 4, 128, 32, torch.bfloat16, poison=True)  # no grouping: 128-token tiles
    assert err <= 2e-2, f"max-abs error {err}"


def test_non_causal():
    err, _ = _run(5, [300, 90], [40, 90], 32, 8, 128, 16, torch.bfloat16, causal=False)
    assert err <= 2e-2, f"max-abs error {err}"


def test_long_context_chunk():
    err, _ = _run(6, [8192 + 128], [512], 32, 8, 128, 16, torch.bfloat16)
    assert err <= 2e-2, f"max-abs error {err}"


def test_fp32_is_refused_not_faked():
    desc, pool_pages = random_descriptors(7, 2, 10, 40, 16, new_tokens=[4, 4])
    pages = torch.zeros(pool_pages, 2, 16, 2, 64, device=DEV)
    q = torch.zeros(8, 8, 64, device=DEV)
    plan = np.zeros(64, dtype=np.int32)
    kv_len = (np.diff(desc["kv_page_indptr"]) - 1) * 16 + desc["kv_last_page_lens"]
    used = ops.make_prefill_plan(desc["indptr"], kv_len, 8, 2, 64, 16, torch.float32, True, plan)
    dd = to_device(desc, DEV)
    with pytest.raises(_lib.DeserveKVError, match="fp32"):
        ops.paged_prefill(q, dd["indptr"], pages, dd["kv_page_indices"], dd["kv_page_indptr"], dd["kv_last_page_lens"],
                          plan, torch.from_numpy(plan[:used]).to(DEV))
