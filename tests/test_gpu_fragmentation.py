"""Mixed prefill / decode under page churn (the fragmentation configuration at test scale): lognormal
prompt lengths prefilled in chunks through the tensor-core prefill kernel, decode
steps through the decode kernel, sequences finishing at seeded random times, their
pages freed and handed to new arrivals. The product's host classes and the oracle's
run in lockstep (same page ids), so every attention output and the final page
contents can be compared."""
import numpy as np
import pytest
import torch

import deserve_b200 as dk
from deserve_b200 import _lib
from oracle import kv_math
from oracle.descriptors import OracleTask, build_descriptors
from oracle.paged_alloc import OracleKVCache, OraclePagePool, OraclePageTables

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def test_fragmented_pool_mixed_batches_match_oracle():
    hq, hkv, d, ps, chunk = 8, 2, 64, 16, 96
    pool_pages, max_live, dtype = 160, 10, torch.bfloat16
    rng = np.random.default_rng(5)
    g = torch.Generator().manual_seed(5)
    pool = dk.GpuPagePool(1, pool_pages, ps, DEV, dtype, n_kv_heads=hkv, head_dim=d)
    init = (torch.randn(pool.pages.shape, generator=g) * 0.5).to(dtype)
    pool.pages.copy_(init)
    o_pages = init[0].clone()
    pta = dk.PageTableAllocator(max_live, 2048, ps, DEV)
    o_pool, o_tab = OraclePagePool(pool_pages, ps), OraclePageTables(max_live, 2048, ps)
    ws = torch.empty(8 << 20, dtype=torch.uint8, device=DEV)
    dec, pre = dk.BatchDecodeWithPagedKVCacheWrapper(ws), dk.BatchPrefillWithPagedKVCacheWrapper(ws.clone())
    live = {}  # id -> (TaskData, PagedKVCache, OracleTask, OracleKVCache, steps_left)
    next_id, worst, n_prefill_batches, n_decode_batches, reused = 0, 0.0, 0, 0, set()
    ever_used, prev_used = set(), set()
    for step in range(200):
        # arrivals: fill up to max_live
        while len(live) < max_live and next_id < 40:
            n = int(np.clip(rng.lognormal(4.6, 0.8), 8, 600))
            t, ot = dk.TaskData.empty(f"t{next_id}", n), OracleTask(initial_seqlen=n)
            live[next_id] = [t, dk.PagedKVCache.empty(pta, pool), ot, OracleKVCache(o_tab, o_pool), int(rng.integers(2, 14))]
            next_id += 1
        if not live:
            break
        ids = sorted(live)
        for i in ids:
            t, _, ot, _, _ = live[i]
            n = min(chunk, t.initial_seqlen - t.start_pos) if t.start_pos < t.initial_seqlen else 1
            t.init(n)
            ot.init(n)
        tasks, caches = [live[i][0] for i in ids], [live[i][1] for i in ids]
        o_desc = build_descriptors([live[i][2] for i in ids], [live[i][3] for i in ids], ps)
        all_decode = all(t.seqlen == 1 for t in tasks)
        if all_decode:
            ctx = dk.FlashDecodeCtx.init_paged_decode_ctx(tasks, caches, dec)
        else:
            ctx = dk.FlashPrefillCtx.init_paged_prefill_ctx(tasks, caches, pre)
        for key in ("indptr", "kv_page_indices", "kv_page_indptr", "kv_last_page_lens"):
            assert getattr(ctx, key).cpu().numpy().tolist() == o_desc[key].tolist(), key
        used_now = set(o_desc["kv_page_indices"].tolist())
        reused |= {p for p in used_now if p in ever_used and p not in prev_used}  # came back after being freed
        prev_used = used_now
        ever_used |= used_now
        nnz = int(o_desc["indptr"][-1])
        q = torch.randn(nnz, hq, d, generator=g).to(dtype)
        k = (torch.randn(nnz, hkv, d, generator=g) * 0.5).to(dtype)
        v = (torch.randn(nnz, hkv, d, generator=g) * 0.5).to(dtype)
        dk.append_paged_kv_cache(k.to(DEV), v.to(DEV), ctx.indptr, pool.pages[0], ctx.kv_page_indices, ctx.kv_page_indptr,
                                 ctx.kv_last_page_lens)
        kv_math.append_paged(o_pages, k, v, o_desc, ps)
        if all_decode:
            dec.begin_forward(ctx.kv_page_indptr, ctx.kv_page_indices, ctx.kv_last_page_lens, hq, hkv, d, ps,
                              data_type=dtype, indptr_host=ctx.host["kv_page_indptr"])
            got = dec.forward(q.to(DEV), pool.pages[0])
            dec.end_forward()
            n_decode_batches += 1
        else:
            pre.begin_forward(ctx.indptr, ctx.kv_page_indptr, ctx.kv_page_indices, ctx.kv_last_page_lens, hq, hkv, d, ps,
                              data_type=dtype, causal=True, qo_indptr_host=ctx.host["indptr"],
                              kv_indptr_host=ctx.host["kv_page_indptr"], last_page_len_host=ctx.host["kv_last_page_lens"])
            got = pre.forward(q.to(DEV), pool.pages[0], causal=True)
            pre.end_forward()
            n_prefill_batches += 1
        want = kv_math.paged_attention(q, o_pages, o_desc, ps, causal=True)
        worst = max(worst, (got.float().cpu() - want).abs().max().item())
        for i in ids:
            t, kv, ot, okv, left = live[i]
            t.step()
            ot.step()
            if t.start_pos >= t.initial_seqlen:
                live[i][4] = left - 1
                if live[i][4] <= 0:  # finished: pages and table row go back
                    kv.free()
                    okv.free()
                    del live[i]
    assert n_prefill_batches >= 10 and n_decode_batches >= 3 and next_id == 40
    assert len(reused) > 20, "the workload must recycle pages"
    assert worst <= 2e-2, f"max-abs attention error {worst}"
    assert torch.equal(pool.pages[0].cpu().view(torch.uint8), o_pages.view(torch.uint8)), "pages differ from the oracle"
    assert pool.num_avails == o_pool.num_avails and _lib.read_device_status() == 0
