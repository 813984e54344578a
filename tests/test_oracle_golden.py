"""The oracle against fixtures recorded from the reference's own classes
(tests/golden/make_golden.py). These pin the CPU restatement before it is
trusted as the checker of the CUDA path."""
import numpy as np
import pytest
import torch

from helpers import bits, dense_attention, host_traces, sha
from oracle import descriptors as odesc
from oracle import kv_math, swap_ops
from oracle.paged_alloc import (OracleChunkPool, OracleKVCache, OraclePagePool, OraclePageTables,
                                OracleVirtualPool)


@pytest.mark.parametrize("idx", [0, 1, 2])
def test_allocator_trace(idx):
    tr = host_traces()["alloc_traces"][idx]
    pool = OraclePagePool(tr["num_pages"], tr["page_size"])
    tables = OraclePageTables(tr["max_req"], 4096, tr["page_size"])
    live = {}
    for op in tr["ops"]:
        if op["op"] == "new":
            live[op["id"]] = OracleKVCache(tables, pool)
            assert live[op["id"]].slot == op["slot"]
        elif op["op"] == "extend":
            c = live[op["id"]]
            if "error" in op:
                with pytest.raises(ValueError):
                    c.extend(op["tokens"])
            else:
                c.extend(op["tokens"])
                assert c.page_ids().tolist() == op["table"]
            assert pool.num_avails == op["num_avails"]
            assert pool.buffer.tolist() == op["buffer"]
        else:
            live.pop(op["id"]).free()
            assert pool.num_avails == op["num_avails"]
            assert int(pool.bitmap.sum()) == op["bitmap_free"]


@pytest.mark.parametrize("idx", [0, 1, 2])
def test_descriptor_trace(idx):
    tr = host_traces()["desc_traces"][idx]
    ps = tr["page_size"]
    pool = OraclePagePool(tr["num_pages"], ps)
    tables = OraclePageTables(len(tr["prompts"]), 4096, ps)
    tasks = [odesc.OracleTask(initial_seqlen=p) for p in tr["prompts"]]
    caches = [OracleKVCache(tables, pool) for _ in tr["prompts"]]
    for step in tr["steps"]:
        sel_t = [tasks[i] for i in step["tasks"]]
        sel_c = [caches[i] for i in step["tasks"]]
        for t, n in zip(sel_t, step["seqlens"]):
            t.init(n)
        d = odesc.build_descriptors(sel_t, sel_c, ps)
        for key, want in step["desc"].items():
            assert d[key].tolist() == want, key
        assert [c.occupied for c in sel_c] == step["occupied"]
        for t in sel_t:
            t.step()


def test_descriptor_known_answers():
    """Hand-checkable values: prompts 100/37/16 at page size 16, then one decode
    step in which the third request crosses a page boundary."""
    pool, tables = OraclePagePool(200, 16), OraclePageTables(8, 4096, 16)
    tasks = [odesc.OracleTask(initial_seqlen=n) for n in (100, 37, 16)]
    caches = [OracleKVCache(tables, pool) for _ in tasks]
    for t in tasks:
        t.init(t.initial_seqlen)
    d = odesc.build_descriptors(tasks, caches, 16)
    assert d["indptr"].tolist() == [0, 100, 137, 153]
    assert d["kv_page_indptr"].tolist() == [0, 7, 10, 11]
    assert d["kv_last_page_lens"].tolist() == [4, 5, 16]
    assert d["kv_page_indices"].tolist() == list(range(11))
    for t in tasks:
        t.step()
    d = odesc.build_descriptors(tasks, caches, 16)
    assert d["kv_page_indptr"].tolist() == [0, 7, 10, 12]
    assert d["kv_last_page_lens"].tolist() == [5, 6, 1]
    assert d["offsets"].tolist() == [100, 37, 16]
    assert d["kv_page_indices"].tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11]


def _check_vstate(pool, st):
    assert pool.on == st["on"]
    assert pool.num_avails == st["num_avails"]
    assert (pool.bitmap == bits(st["bitmap"])).all()
    assert (pool.swap_bitmap == bits(st["swap_bitmap"])).all()
    assert pool.swap_count == st["swap_count"]
    assert pool.buffer.tolist() == st["buffer"]


@pytest.mark.parametrize("idx", [0, 1, 2])
def test_virtual_pool_trace(idx):
    tr = host_traces()["virtual_traces"][idx]
    pool = OracleVirtualPool(tr["main"], tr["swap"], tr["page_size"])
    tables = OraclePageTables(64, 4096, tr["page_size"])
    rounds = tr["rounds"]
    pinned = [{"bitmap": np.ones(tr["swap"], dtype=bool), "count": tr["swap"]} for _ in range(rounds)]
    live = {}
    for op in tr["ops"]:
        kind = op["op"]
        if kind == "init":
            _check_vstate(pool, op["state"])
        elif kind == "switch":
            pool.switch()
            _check_vstate(pool, op["state"])
        elif kind == "adjust":
            for cid, table in op["tables"].items():
                live[int(cid)].adjust(op["offset"])
                assert live[int(cid)].page_ids().tolist() == table
        elif kind == "free":
            live.pop(op["id"]).free()
            _check_vstate(pool, op["state"])
        elif kind == "new":
            live[op["id"]] = OracleKVCache(tables, pool)
            assert live[op["id"]].slot == op["slot"]
        elif kind == "extend":
            c = live[op["id"]]
            if "error" in op:
                with pytest.raises(ValueError):
                    c.extend(op["tokens"])
            else:
                c.extend(op["tokens"])
                assert c.page_ids().tolist() == op["table"]
                assert c.isswap[: c.occupied].tolist() == op["isswap"]
            _check_vstate(pool, op["state"])
        elif kind == "swap2":
            mb = op["mb"]
            to = pinned[(mb - 1 + rounds) % rounds]
            pool.swap2_bookkeeping(pinned[(mb + 1) % rounds], to)
            _check_vstate(pool, op["state"])
            assert to["count"] == op["to_count"]
            assert (np.asarray(to["bitmap"]).astype(bool) == bits(op["to_bitmap"])).all()


def test_virtual_pool_scenario():
    ops = host_traces()["virtual_a2"]
    pool = OracleVirtualPool(6, 4, 16)
    tables = OraclePageTables(8, 4096, 16)
    _check_vstate(pool, ops[0]["state"])
    mb0 = OracleKVCache(tables, pool)
    mb0.extend(8 * 16)
    _check_vstate(pool, ops[1]["state"])
    assert mb0.page_ids().tolist() == ops[1]["table"] and mb0.isswap[:8].tolist() == ops[1]["isswap"]
    pool.switch()
    _check_vstate(pool, ops[2]["state"])
    mb1 = OracleKVCache(tables, pool)
    mb1.extend(3 * 16)
    _check_vstate(pool, ops[3]["state"])
    assert mb1.page_ids().tolist() == ops[3]["table"] and mb1.isswap[:3].tolist() == ops[3]["isswap"]
    pool.switch()
    _check_vstate(pool, ops[4]["state"])
    mb0.extend(9 * 16)
    _check_vstate(pool, ops[5]["state"])
    assert mb0.page_ids().tolist() == ops[5]["table"]
    mb0.adjust(4)
    assert mb0.page_ids().tolist() == ops[6]["table"] == [0, 1, 2, 3, 4, 5, 10, 11, 12]


@pytest.mark.parametrize("idx", [0, 1])
def test_chunk_pool_trace(idx):
    tr = host_traces()["chunk_traces"][idx]
    cp = OracleChunkPool(tr["height"])
    for op in tr["ops"]:
        if op["op"] == "alloc":
            if "error" in op:
                with pytest.raises(RuntimeError):
                    cp.alloc(op["size"])
            else:
                assert cp.alloc(op["size"]) == (op["id"], op["level"])
        else:
            cp.free(op["id"], op["level"])
        assert cp.available == op["available"]


def test_offload_reload_layout():
    o = host_traces()["offload"]
    g = torch.Generator().manual_seed(o["seed"])
    L, ps = o["L"], o["ps"]
    pool = OracleVirtualPool(o["main"], o["swap"], ps)
    pages = torch.empty(L, pool.num_pages, 2, ps, 8, 128, dtype=torch.float16)
    pages.copy_(torch.randn(pages.shape, generator=g).to(torch.float16))
    assert sha(pages) == o["pages_before_sha"]
    tables = OraclePageTables(8, 4096, ps)
    chunks = OracleChunkPool(o["height"])
    c0 = OracleKVCache(tables, pool)
    c0.extend(2 * ps)
    c1 = OracleKVCache(tables, pool)
    c1.extend(5 * ps)
    assert c1.page_ids().tolist() == o["ids"]
    cid, level = chunks.alloc(c1.occupied)
    assert (cid, level) == (o["chunk_id"], o["chunk_level"])
    rows = swap_ops.offload_rows(pages, c1.page_ids())
    assert sha(rows) == o["rows_sha"]
    c1.free()
    c2 = OracleKVCache(tables, pool)
    c2.extend(3 * ps)
    assert c2.page_ids().tolist() == o["c2_ids"]
    new_ids = pool.alloc(5)
    slot = tables.alloc()
    assert new_ids.tolist() == o["new_ids"] and slot == o["new_slot"]
    assert (new_ids >= pool.num_pages_main).tolist() == o["isswap"]
    swap_ops.reload_rows(pages, new_ids, rows)
    assert sha(pages) == o["pages_after_sha"]


@pytest.mark.parametrize("case", ["a", "b", "c", "d"])
def test_dense_attention_and_rope(case):
    """Rotary embedding and dense causal attention against tensors traced from
    the reference's Attention.traced_forward (fp32, positions from 0)."""
    d = dense_attention()
    hq, hkv, dim, n, theta = d[f"{case}_meta"]
    n = int(n)
    xq, xk, xv = (torch.from_numpy(d[f"{case}_{k}"]) for k in ("xq", "xk", "xv"))
    pos = torch.arange(n)
    q_rot = kv_math.apply_rope(xq, pos, float(theta))
    k_rot = kv_math.apply_rope(xk, pos, float(theta))
    assert torch.equal(q_rot, torch.from_numpy(d[f"{case}_xq_rotary"]))
    assert torch.equal(k_rot, torch.from_numpy(d[f"{case}_xk_rotary"]))
    out = kv_math.dense_attention(q_rot, k_rot, xv, causal_tail=True)
    # same fp32 math, different association order of the matmuls: a few ulp
    torch.testing.assert_close(out, torch.from_numpy(d[f"{case}_output"]), rtol=2e-5, atol=2e-6)


def test_append_then_gather_roundtrip():
    """Appending rows through the descriptors and reading them back through the
    page table gives the rows in token order (index rule of the append call)."""
    from helpers import random_descriptors

    ps, hkv, dim = 16, 2, 64
    desc, pool_pages = random_descriptors(3, 5, 1, 90, ps, new_tokens=[1, 4, 17, 2, 90])
    pages = torch.zeros(pool_pages, 2, ps, hkv, dim)
    nnz = int(desc["indptr"][-1])
    g = torch.Generator().manual_seed(0)
    k, v = torch.randn(nnz, hkv, dim, generator=g), torch.randn(nnz, hkv, dim, generator=g)
    kv_math.append_paged(pages, k, v, desc, ps)
    for i in range(5):
        a, b = desc["indptr"][i], desc["indptr"][i + 1]
        gk, gv = kv_math.gather_kv(pages, desc, i, ps)
        assert torch.equal(gk[-(b - a):], k[a:b]) and torch.equal(gv[-(b - a):], v[a:b])
    used = np.unique(desc["kv_page_indices"])
    mask = torch.ones(pool_pages, dtype=torch.bool)
    mask[torch.as_tensor(used, dtype=torch.long)] = False
    assert pages[mask].abs().sum() == 0  # nothing written outside the batch's pages
