"""The product's host-side KV-cache classes (reference names and signatures)
replayed against traces recorded from the reference's own classes. Pure host
logic: runs without a GPU."""
import numpy as np
import pytest
import torch

import deserve_b200 as dk
from helpers import bits, host_traces

CPU = torch.device("cpu")


def _extend(cache, tokens, native):
    """Grow a cache through the Python class or through the native step builder."""
    if not native:
        return cache.extend(tokens)
    from deserve_b200.context import build_step

    t = dk.TaskData.empty("x", 0)
    t.init(tokens)
    build_step([t], [cache])
    return True


@pytest.mark.parametrize("native", [False, True])
@pytest.mark.parametrize("idx", [0, 1, 2])
def test_allocator_trace(idx, native):
    tr = host_traces()["alloc_traces"][idx]
    pool = dk.CpuPagePool(1, tr["num_pages"], tr["page_size"], torch.float16, n_kv_heads=1, head_dim=8)
    pta = dk.PageTableAllocator(tr["max_req"], 4096, tr["page_size"], CPU)
    live = {}
    for op in tr["ops"]:
        if op["op"] == "new":
            live[op["id"]] = dk.PagedKVCache.empty(pta, pool)
            assert live[op["id"]].page_table.offset == op["slot"]
        elif op["op"] == "extend":
            c = live[op["id"]]
            if "error" in op:
                with pytest.raises(ValueError, match="Not enough pages"):
                    _extend(c, op["tokens"], native)
            else:
                assert _extend(c, op["tokens"], native) is True
                assert c.page_table.retrieve().tolist() == op["table"]
            assert pool.num_avails == op["num_avails"]
            assert pool.page_buffer.tolist() == op["buffer"]
        else:
            live.pop(op["id"]).free()
            assert pool.num_avails == op["num_avails"]
            assert int(pool.page_bitmap.sum()) == op["bitmap_free"]


@pytest.mark.parametrize("idx", [0, 1, 2])
def test_descriptor_trace(idx):
    tr = host_traces()["desc_traces"][idx]
    ps = tr["page_size"]
    pool = dk.CpuPagePool(1, tr["num_pages"], ps, torch.float16, n_kv_heads=1, head_dim=8)
    pta = dk.PageTableAllocator(len(tr["prompts"]), 4096, ps, CPU)
    tasks = [dk.TaskData.empty(f"t{i}", p) for i, p in enumerate(tr["prompts"])]
    caches = [dk.PagedKVCache.empty(pta, pool) for _ in tr["prompts"]]
    for step in tr["steps"]:
        sel_t = [tasks[i] for i in step["tasks"]]
        sel_c = [caches[i] for i in step["tasks"]]
        for t, n in zip(sel_t, step["seqlens"]):
            t.init(n)
        ctx = dk.FlashForwardCtx.init_paged_forward_ctx(sel_t, sel_c)
        for key, want in step["desc"].items():
            got = getattr(ctx, key)
            assert got.dtype == torch.int32 and got.tolist() == want, key
        assert ctx.bsz == len(sel_t) and ctx.layer_id == 0 and ctx.page_pool is pool
        assert [c.page_table.occupied for c in sel_c] == step["occupied"]
        for t in sel_t:
            t.step()


def _check_vstate(pool, st):
    assert pool.on == st["on"]
    assert pool.num_avails == st["num_avails"]
    assert (pool.page_bitmap.numpy() == bits(st["bitmap"])).all()
    assert (pool.swap_bitmap.numpy() == bits(st["swap_bitmap"])).all()
    assert pool.swap_count == st["swap_count"]
    assert pool.page_buffer.tolist() == st["buffer"]


@pytest.mark.parametrize("native", [False, True])
@pytest.mark.parametrize("idx", [0, 1, 2])
def test_virtual_pool_trace(idx, native):
    tr = host_traces()["virtual_traces"][idx]
    pool = dk.VirtualPagePool(1, tr["main"], tr["swap"], tr["page_size"], CPU, torch.float16, n_kv_heads=1, head_dim=8)
    pta = dk.PageTableAllocator(64, 4096, tr["page_size"], CPU)
    rounds = tr["rounds"]
    pinned = [dk.CopiedPinnedMemory(16, tr["swap"], CPU) for _ in range(rounds)]
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
                assert live[int(cid)].page_table.retrieve().tolist() == table
        elif kind == "free":
            live.pop(op["id"]).free()
            _check_vstate(pool, op["state"])
        elif kind == "new":
            live[op["id"]] = dk.VirtualPagedKVCache.empty(pta, pool)
            assert live[op["id"]].page_table.offset == op["slot"]
        elif kind == "extend":
            c = live[op["id"]]
            if "error" in op:
                with pytest.raises(ValueError):
                    _extend(c, op["tokens"], native)
            else:
                _extend(c, op["tokens"], native)
                assert c.page_table.retrieve().tolist() == op["table"]
                assert c.isswap[: c.page_table.occupied].tolist() == op["isswap"]
            _check_vstate(pool, op["state"])
        elif kind == "swap2":
            mb = op["mb"]
            to = pinned[(mb - 1 + rounds) % rounds]
            pool._handoff(pinned[(mb + 1) % rounds], to)  # the bookkeeping half of swap2 (no device here)
            _check_vstate(pool, op["state"])
            assert to.count == op["to_count"]
            assert (np.asarray(to.bitmap).astype(bool) == bits(op["to_bitmap"])).all()


@pytest.mark.parametrize("idx", [0, 1])
def test_chunk_pool_trace(idx):
    tr = host_traces()["chunk_traces"][idx]
    cp = dk.CpuChunkPool(1, tr["height"], 1, torch.float16, n_kv_heads=1, head_dim=8)
    live = {}
    for op in tr["ops"]:
        if op["op"] == "alloc":
            if "error" in op:
                with pytest.raises(RuntimeError):
                    cp.alloc(op["size"])
            else:
                h = cp.alloc(op["size"])
                assert (h.id, h.level, h.initial_size) == (op["id"], op["level"], op["size"])
                live[(h.id, h.level)] = h
        else:
            live.pop((op["id"], op["level"])).free()
        assert cp.available_ids == op["available"]


def test_chunk_handle_rows():
    cp = dk.CpuChunkPool(3, 4, 2, torch.float16, n_kv_heads=1, head_dim=8)
    a, b = cp.alloc(2), cp.alloc(1)
    assert a.retrieve().shape == (2 * 3, 2, 2, 1, 8)
    assert (a.id, a.level, b.id, b.level) == (2, 1, 6, 0)  # split pops the last parent, alloc the first child
    assert (a.row_begin, b.row_begin) == (12, 18)
    assert b.retrieve().data_ptr() == cp.chunks[18:].data_ptr()


def test_errors_match_reference_types():
    pool = dk.CpuPagePool(1, 4, 16, torch.float16, n_kv_heads=1, head_dim=8)
    with pytest.raises(ValueError, match="Not enough pages"):
        pool.alloc(5)
    pta = dk.PageTableAllocator(1, 64, 16, CPU)
    pta.alloc()
    with pytest.raises(ValueError, match="No available slots"):
        pta.alloc()
    cp = dk.CpuChunkPool(1, 3, 1, torch.float16, n_kv_heads=1, head_dim=8)
    cp.alloc(4)
    with pytest.raises(RuntimeError):
        cp.alloc(1)


def test_page_tensor_layout_and_defaults():
    pool = dk.CpuPagePool(2, 3, 16, torch.bfloat16)
    assert pool.pages.shape == (2, 3, 2, 16, 8, 128)
    assert pool.get_layered_pages(1).data_ptr() == pool.pages[1].data_ptr()
    assert pool.page_bytes == 2 * 16 * 8 * 128 * 2
    assert pool.calc_num_pages(17) == 2
    v = dk.VirtualPagePool(2, 4, 2, 8, CPU, torch.float16)
    assert v.calc_swap_size() == 2 * 2 * 2 * 8 * 8 * 128
    assert v.slices == [(4, 6), (6, 8)] and v.num_avails == 6


def test_task_manager_page_arithmetic():
    tm = dk.TaskManager(100, 16)
    t = dk.TaskData.empty("a", 100)
    tm.add(t)
    t.init(40)
    assert tm.calc_extended_space(["a"]) == 3 and tm.calc_rest_space("a") == 7
    t.step()
    assert (t.start_pos, t.seqlen) == (40, 0)
    t.init(60)
    assert tm.calc_delta_space("a", 60) == 4 and t.finished_prefill()
    t.step()
    assert (t.start_pos, t.seqlen, t.round) == (100, 1, 2)
    assert tm.calc_occupied_space(["a"]) == 7 and tm.calc_initial_space(["a"]) == 7


def test_kernels_refuse_cpu_tensors():
    """No CPU fallback: an operator handed host tensors fails loudly."""
    pages = torch.zeros(4, 2, 16, 2, 64)
    k = torch.zeros(1, 2, 64)
    i32 = torch.zeros(2, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        dk.append_paged_kv_cache(k, k, i32, pages, i32, i32, i32[:1])
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        dk.apply_rope(k, k, i32, i32[:1])


@pytest.mark.parametrize("native", [False, True])
@pytest.mark.parametrize("seed", range(6))
def test_allocator_agrees_with_oracle_on_random_histories(seed, native):
    """Differential check beyond the recorded traces: random create / grow / free
    histories (pool exhaustion included) through the product's classes, grown either by
    the Python classes or by the native step builder, against the CPU oracle that the
    reference traces pin."""
    import random

    from oracle.paged_alloc import OracleKVCache, OraclePagePool, OraclePageTables

    rng = random.Random(1000 + seed)
    ps = rng.choice([4, 8, 16])
    num_pages, max_req = rng.choice([40, 90, 200]), rng.choice([4, 9, 16])
    pool = dk.CpuPagePool(1, num_pages, ps, torch.float16, n_kv_heads=1, head_dim=8)
    pta = dk.PageTableAllocator(max_req, 4096, ps, CPU)
    opool, otab = OraclePagePool(num_pages, ps), OraclePageTables(max_req, 4096, ps)
    live = {}
    for step in range(300):
        r = rng.random()
        if (r < 0.25 or not live) and len(live) < max_req:
            live[step] = [dk.PagedKVCache.empty(pta, pool), OracleKVCache(otab, opool), 0]
            assert live[step][0].page_table.offset == live[step][1].slot
        elif r < 0.8:
            cid = rng.choice(list(live))
            mine, theirs, tokens = live[cid]
            tokens += rng.choice([1, 1, 1, 2, ps, ps + 1, 5 * ps, 23 * ps])
            try:
                theirs.extend(tokens)
                ok = True
            except ValueError:
                ok = False
            if ok:
                assert _extend(mine, tokens, native) is True
                live[cid][2] = tokens
                assert mine.page_table.retrieve().tolist() == theirs.page_ids().tolist()
            else:
                with pytest.raises(ValueError, match="Not enough pages"):
                    _extend(mine, tokens, native)
        else:
            mine, theirs, _ = live.pop(rng.choice(list(live)))
            mine.free()
            theirs.free()
        assert pool.num_avails == opool.num_avails
        assert pool.page_buffer.tolist() == opool.buffer.tolist()
        assert pool.page_bitmap.numpy().tolist() == opool.bitmap.tolist()


def test_reserve_takes_chosen_pages_out_of_the_free_set():
    pool = dk.CpuPagePool(1, 32, 4, torch.float32, n_kv_heads=1, head_dim=4)
    ids = np.array([30, 2, 17], dtype=np.int32)
    pool.reserve(ids)
    assert pool.num_avails == 29 and not pool.page_bitmap[ids.astype(np.int64)].any()
    got = pool.alloc(4).tolist()
    assert got == [0, 1, 3, 4]  # lowest free ids, the reserved ones skipped
    with pytest.raises(ValueError):
        pool.reserve([2])        # already taken
    with pytest.raises(ValueError):
        pool.reserve([5, 5])     # listed twice
    with pytest.raises(ValueError):
        pool.reserve([32])       # outside the pool
    pool.free(ids)
    assert pool.num_avails == 28


def test_pinned_ring_hands_out_buffers_round_robin_and_grows():
    from deserve_b200.pinned import PinnedRing

    r = PinnedRing(slots=3, capacity=8, pin=False)
    a, sa = r.take(4)
    b, sb = r.take(8)
    c, sc = r.take(20)  # larger than the slot: the slot grows
    assert (sa, sb, sc) == (0, 1, 2) and a.numel() == 4 and c.numel() == 20
    a[:] = 7
    r.done(sa)
    a2, sa2 = r.take(2)
    assert sa2 == 0 and a2.data_ptr() == a.data_ptr()


def test_kvconfig_builds_the_stage_objects_and_ownership_check_finds_planted_faults():
    cfg = dk.KVConfig(num_layers=2, n_q_heads=4, n_kv_heads=2, head_dim=8, page_size=4, dtype=torch.float32,
                      num_pages_main=10, num_pages_swap=3, max_requests=4, max_context_len=64, buddy_height=3)
    assert cfg.pool_bytes() == 2 * 16 * 2 * 4 * 2 * 8 * 4
    pool, tables, chunks, mgr = cfg.build("cpu")
    assert pool.pages.shape == (2, 16, 2, 4, 2, 8) and pool.num_pages_swap == 3 and mgr.virtual_page_pool is pool
    a, b = dk.VirtualPagedKVCache.empty(tables, pool), dk.VirtualPagedKVCache.empty(tables, pool)
    a.extend(17)   # 5 pages
    b.extend(30)   # 8 pages: the main area runs out, the last ones come from the active region
    assert int(b.isswap.sum()) + int(a.isswap.sum()) == 3
    dk.check_page_ownership(pool, [a, b])
    with pytest.raises(AssertionError, match="in flight"):      # the caches do own pages of region 0 ...
        dk.check_page_ownership(pool, [a, b], in_flight=pool.slices[0])
    dk.check_page_ownership(pool, [a, b], in_flight=pool.slices[1])  # ... and none of region 1
    stolen = int(a.page_table.retrieve_np()[2])
    b.page_table.retrieve_np()[0] = stolen                          # plant: one page in two tables
    with pytest.raises(AssertionError, match="owned twice"):
        dk.check_page_ownership(pool, [a, b])
    b.page_table.retrieve_np()[0] = 99                               # plant: an id outside the pool
    with pytest.raises(AssertionError, match="outside the pool"):
        dk.check_page_ownership(pool, [a, b])
    b.page_table.retrieve_np()[0] = 15                               # plant: a page of the region that is away
    with pytest.raises(AssertionError, match="in flight"):
        dk.check_page_ownership(pool, [b], in_flight=pool.slices[1 - pool.on])
    b.page_table.retrieve_np()[0] = 5
    b.pool._bitmap[5] = True                                         # plant: an owned page marked free
    with pytest.raises(AssertionError, match="marked free"):
        dk.check_page_ownership(pool, [b])


def test_bind_host_to_gpu_leaves_the_process_alone_without_nvml():
    import os

    from deserve_b200.pinned import bind_host_to_gpu

    before = os.sched_getaffinity(0)
    info = bind_host_to_gpu(0)
    assert isinstance(info, dict) and "bound" in info
    if not info["bound"]:
        assert os.sched_getaffinity(0) == before
    os.sched_setaffinity(0, before)


def test_swap_regions_learn_the_token_rows_of_their_pages_from_the_step_builder():
    """A pool with swap regions keeps, per region page, how many token rows hold data: the step builder
    lowers it for the pages a step describes (a request's last page holds kv_last_page_len rows, the others
    are full), a freed page counts as whole again, and the count of a region's head is the most any page in
    use holds. swap2 moves only that many rows of each half page."""
    from deserve_b200.context import pack_descriptors
    from deserve_b200.task import TaskData

    ps, main, swap = 8, 2, 3
    pool = dk.VirtualPagePool(1, main, swap, ps, CPU, torch.float16, n_kv_heads=1, head_dim=8)
    pta = dk.PageTableAllocator(4, 64, ps, CPU)
    assert pool.rows_used.tolist() == [ps] * (2 * swap)
    cache = dk.VirtualPagedKVCache.empty(pta, pool)
    task = TaskData.empty("t", 19, dk.SamplingParams()) if hasattr(TaskData, "empty") else None
    if task is None:
        pytest.skip("TaskData.empty is not available")
    task.start_pos, task.seqlen = 0, 19          # 19 tokens: pages 0, 1 (main) and the first page of the region on
    d = pack_descriptors([task], [cache])
    ids = d["kv_page_indices"].tolist()
    assert ids[:2] == [0, 1] and ids[2] == main and d["kv_last_page_lens"].tolist() == [3]
    assert pool.rows_used[0] == 3                # the request's last page sits in the region: 3 rows
    assert pool._rows_of(main, 1, np.array([False, True, True])) == 3
    assert pool._rows_of(main, 0, np.array([True, True, True])) == 0
    task.start_pos, task.seqlen = 19, 6          # 25 tokens: the region page is full, a second one holds 1 row
    d = pack_descriptors([task], [cache])
    assert d["kv_page_indices"].tolist()[2:] == [main, main + 1]
    assert pool.rows_used[:2].tolist() == [ps, 1]
    assert pool._rows_of(main, 2, np.array([False, False, True])) == ps
    pool.rows_used[0] = 2
    pool.free(np.array([main]))                  # whoever gets the page next holds a whole page until told otherwise
    assert pool.rows_used[0] == ps
    plain = dk.GpuPagePool(1, 4, ps, CPU, torch.float16, n_kv_heads=1, head_dim=8) if hasattr(dk, "GpuPagePool") else None
    assert plain is None or getattr(plain, "rows_used", None) is None
