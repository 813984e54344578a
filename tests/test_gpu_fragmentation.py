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


def test_fragmentation_full_size_one_layer_pool_hash():
    """The mixed prefill / decode configuration at its full size on one layer of the 8B head shape: 512
    arrivals with prompts ~ LogNormal(6.5, 0.8) clipped to [16, 8192], prefilled in 512-token chunks
    through the tensor-core kernel (mixed with the decode rows of the others), 16-128 decode tokens
    each, departures free the pages for later arrivals. The product's host classes and the oracle's
    run in lockstep; descriptors are compared at every step, the attention output on a sample of the
    steps, and at the end the SHA-256 of the whole page pool and the allocator state."""
    import hashlib

    hq, hkv, d, ps, chunk = 32, 8, 128, 16, 512
    pool_pages, max_live, n_arrivals, dtype = 12000, 64, 512, torch.bfloat16
    rng = np.random.default_rng(0)
    lens = np.clip(rng.lognormal(6.5, 0.8, size=n_arrivals), 16, 8192).astype(np.int64)
    new = rng.integers(16, 129, size=n_arrivals)
    g = torch.Generator().manual_seed(9)
    g_dev = torch.Generator(device=DEV).manual_seed(9)
    pool = dk.GpuPagePool(1, pool_pages, ps, DEV, dtype, n_kv_heads=hkv, head_dim=d)
    pool.pages.zero_()
    o_pages = torch.zeros(pool_pages, 2, ps, hkv, d, dtype=dtype)
    pta = dk.PageTableAllocator(max_live, 8192 + 256, ps, DEV)
    o_pool, o_tab = OraclePagePool(pool_pages, ps), OraclePageTables(max_live, 8192 + 256, ps)
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=DEV)
    dec, pre = dk.BatchDecodeWithPagedKVCacheWrapper(ws), dk.BatchPrefillWithPagedKVCacheWrapper(
        torch.empty(64 << 20, dtype=torch.uint8, device=DEV))
    live, next_id, step, worst, checked, reserved = {}, 0, 0, 0.0, 0, 0
    ever_used, prev_used, reused = np.zeros(pool_pages, bool), np.zeros(pool_pages, bool), 0
    prompt_rows = decode_rows = 0
    while live or next_id < n_arrivals:
        while next_id < n_arrivals and len(live) < max_live:
            need = -(-(int(lens[next_id]) + int(new[next_id])) // ps)
            if reserved + need > pool_pages - 64:
                break                                   # waits for departures
            n = int(lens[next_id])
            live[next_id] = [dk.TaskData.empty(f"t{next_id}", n), dk.PagedKVCache.empty(pta, pool),
                             OracleTask(initial_seqlen=n), OracleKVCache(o_tab, o_pool), int(new[next_id]), need]
            reserved += need
            next_id += 1
        ids = sorted(live)
        for i in ids:
            t, _, ot = live[i][:3]
            n = min(chunk, t.initial_seqlen - t.start_pos) if t.start_pos < t.initial_seqlen else 1
            t.init(n)
            ot.init(n)
        tasks, caches = [live[i][0] for i in ids], [live[i][1] for i in ids]
        o_desc = build_descriptors([live[i][2] for i in ids], [live[i][3] for i in ids], ps)
        all_decode = all(t.seqlen == 1 for t in tasks)
        ctx = (dk.FlashDecodeCtx.init_paged_decode_ctx(tasks, caches, dec) if all_decode
               else dk.FlashPrefillCtx.init_paged_prefill_ctx(tasks, caches, pre))
        for key in ("indptr", "kv_page_indices", "kv_page_indptr", "kv_last_page_lens"):
            assert np.array_equal(ctx.host[key], o_desc[key]), (step, key)
        used = np.zeros(pool_pages, bool)
        used[o_desc["kv_page_indices"]] = True
        reused += int((used & ever_used & ~prev_used).sum())
        prev_used, ever_used = used, ever_used | used
        nnz = int(o_desc["indptr"][-1])
        prompt_rows += sum(t.seqlen for t in tasks if t.start_pos < t.initial_seqlen)   # a last chunk may be one row
        decode_rows += sum(1 for t in tasks if t.start_pos >= t.initial_seqlen)
        q = torch.randn(nnz, hq, d, generator=g_dev, device=DEV).to(dtype)  # copied to the host only when checked
        k = (torch.randn(nnz, hkv, d, generator=g) * 0.5).to(dtype)
        v = (torch.randn(nnz, hkv, d, generator=g) * 0.5).to(dtype)
        dk.append_paged_kv_cache(k.to(DEV), v.to(DEV), ctx.indptr, pool.pages[0], ctx.kv_page_indices, ctx.kv_page_indptr,
                                 ctx.kv_last_page_lens)
        kv_math.append_paged(o_pages, k, v, o_desc, ps)
        if all_decode:
            dec.begin_forward(ctx.kv_page_indptr, ctx.kv_page_indices, ctx.kv_last_page_lens, hq, hkv, d, ps,
                              data_type=dtype, indptr_host=ctx.host["kv_page_indptr"])
            got = dec.forward(q, pool.pages[0])
            dec.end_forward()
        else:
            pre.begin_forward(ctx.indptr, ctx.kv_page_indptr, ctx.kv_page_indices, ctx.kv_last_page_lens, hq, hkv, d, ps,
                              data_type=dtype, causal=True, qo_indptr_host=ctx.host["indptr"],
                              kv_indptr_host=ctx.host["kv_page_indptr"], last_page_len_host=ctx.host["kv_last_page_lens"],
                              kv_indices_host=ctx.host["kv_page_indices"])
            got = pre.forward(q, pool.pages[0], causal=True)
            pre.end_forward()
        if step % 25 == 0:  # the oracle's attention on a few requests of this step (short contexts keep it quick)
            got_cpu, q_cpu = got.float().cpu(), q.cpu()
            kv_len = kv_math.kv_lengths(o_desc, ps)
            for j in [j for j in range(len(ids)) if kv_len[j] <= 1536][:4]:
                a, b = int(o_desc["indptr"][j]), int(o_desc["indptr"][j + 1])
                kk, vv = kv_math.gather_kv(o_pages, o_desc, j, ps)
                want = kv_math.dense_attention(q_cpu[a:b], kk, vv, True)
                worst = max(worst, (got_cpu[a:b] - want).abs().max().item())
                checked += 1
        for i in ids:
            t, kv, ot, okv, left, need = live[i]
            t.step()
            ot.step()
            if t.start_pos >= t.initial_seqlen:
                live[i][4] = left - 1
                if live[i][4] <= 0:
                    kv.free()
                    okv.free()
                    reserved -= need
                    del live[i]
        step += 1
        assert step < 5000
    assert next_id == n_arrivals and not live
    # the step that finishes a prompt yields the first token, so a request runs new - 1 decode rows
    assert prompt_rows == int(lens.sum()) and decode_rows == int(new.sum()) - n_arrivals
    assert reused > 5000, "the workload must recycle pages"
    assert checked >= 40 and worst <= 2e-2, (checked, worst)
    sha = lambda t: hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()
    assert sha(pool.pages[0].cpu()) == sha(o_pages), "page pool differs from the oracle's"
    assert pool.num_avails == o_pool.num_avails == pool_pages and _lib.read_device_status() == 0
