"""The device-resident allocator / page tables / descriptor build (DevicePageState,
csrc/device_step.cu) against the CPU oracle that the reference's own traces pin:
random create / grow / free histories must leave the same page ids in the same
table rows, the same free bitmap and the same prefetch buffer, and every step's
descriptors must equal the oracle's; then a decode step fed by these descriptors
must give the host path's attention output bit for bit."""
import random

import numpy as np
import pytest
import torch

import deserve_b200 as dk
from deserve_b200 import _lib, ops
from deserve_b200.device_state import DevicePageState
from oracle.descriptors import OracleTask, build_descriptors
from oracle.paged_alloc import OracleKVCache, OraclePagePool, OraclePageTables

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.mark.parametrize("seed", range(4))
def test_device_state_follows_the_oracle_on_random_histories(seed):
    rng = random.Random(2000 + seed)
    ps = rng.choice([4, 8, 16])
    num_pages, max_req = rng.choice([90, 200, 700]), rng.choice([4, 9, 16])
    st = DevicePageState(num_pages, ps, max_req, 4096, DEV)
    opool, otab = OraclePagePool(num_pages, ps), OraclePageTables(max_req, 4096, ps)
    live = {}   # id -> [slot, oracle cache, oracle task]
    for step in range(120):
        r = rng.random()
        if (r < 0.25 or not live) and len(live) < max_req:
            kv = OracleKVCache(otab, opool)
            slot = st.alloc_slot()
            assert slot == kv.slot
            live[step] = [slot, kv, OracleTask(initial_seqlen=rng.choice([1, 5, 3 * ps, 40 * ps]))]
        elif r < 0.85:
            # one step of a random subset of the live requests, in a random order
            ids = rng.sample(list(live), rng.randint(1, len(live)))
            for i in ids:
                t = live[i][2]
                t.init(min(rng.choice([1, 1, ps, 5 * ps + 1]), max(1, t.initial_seqlen - t.start_pos))
                       if t.start_pos < t.initial_seqlen else 1)
            tasks, caches = [live[i][2] for i in ids], [live[i][1] for i in ids]
            args = ([live[i][0] for i in ids], [t.start_pos for t in tasks], [t.seqlen for t in tasks],
                    [t.initial_seqlen for t in tasks])
            try:
                want = build_descriptors(tasks, caches, ps)
            except ValueError:
                with pytest.raises(ValueError, match="Not enough pages"):
                    st.build_step(*args)
                want = None
            if want is not None:
                dev, host = st.build_step(*args)
                for name in ("indptr", "kv_page_indptr", "kv_last_page_lens", "kv_page_indices"):
                    assert dev[name].cpu().numpy().tolist() == want[name].tolist(), (step, name)
                for name in ("indptr", "kv_page_indptr", "kv_last_page_lens"):
                    assert host[name].tolist() == want[name].tolist()
                for t in tasks:
                    t.step()
        else:
            i = rng.choice(list(live))
            slot, kv, _ = live.pop(i)
            st.free_slots([slot])
            kv.free()
        snap = st.snapshot()
        assert st.num_avails == snap["num_avails"] == opool.num_avails, step
        assert snap["bitmap"].tolist() == opool.bitmap.tolist(), step
        assert snap["buffer"].tolist() == opool.buffer.tolist(), step
        for slot, kv, _ in live.values():
            ids = kv.page_ids().tolist()
            assert snap["occupied"][slot] == len(ids) and snap["tables"][slot, : len(ids)].tolist() == ids
    assert _lib.read_device_status() == 0


def test_decode_step_from_device_built_descriptors_equals_the_host_path():
    hq, hkv, d, ps, dtype = 32, 8, 128, 16, torch.bfloat16
    lens = [37, 512, 16, 1200, 255, 3000, 64, 700]
    B = len(lens)
    pool = dk.GpuPagePool(1, 600, ps, DEV, dtype, n_kv_heads=hkv, head_dim=d)
    pta = dk.PageTableAllocator(B, 4096, ps, DEV)
    st = DevicePageState(600, ps, B, 4096, DEV)
    g = torch.Generator(device=DEV).manual_seed(3)
    pool.pages.normal_(0.0, 0.5, generator=g)
    tasks = [dk.TaskData.empty(f"t{i}", n) for i, n in enumerate(lens)]
    caches = [dk.PagedKVCache.empty(pta, pool) for _ in lens]
    slots = [st.alloc_slot() for _ in lens]
    assert slots == [c.page_table.offset for c in caches]
    for t, c in zip(tasks, caches):   # the context is already in the cache
        t.init(t.initial_seqlen)
    ws = torch.empty(32 << 20, dtype=torch.uint8, device=DEV)
    wrapper = dk.BatchDecodeWithPagedKVCacheWrapper(ws)
    q = torch.randn(B, hq, d, device=DEV, generator=g).to(dtype)
    outs = []
    for step in range(3):
        ctx = dk.FlashDecodeCtx.init_paged_decode_ctx(tasks, caches, wrapper) if step else \
            dk.FlashPrefillCtx.init_paged_prefill_ctx(tasks, caches, None)
        dev, host = st.build_step(slots, [t.start_pos for t in tasks], [t.seqlen for t in tasks],
                                  [t.initial_seqlen for t in tasks])
        for name in ("indptr", "kv_page_indices", "kv_page_indptr", "kv_last_page_lens", "offsets", "seqlens"):
            assert torch.equal(dev[name], getattr(ctx, name)), (step, name)
        if step:
            got = []
            for desc, h in ((ctx, ctx.host), (None, host)):
                kvp, idx, last = (desc.kv_page_indptr, desc.kv_page_indices, desc.kv_last_page_lens) if desc else \
                    (dev["kv_page_indptr"], dev["kv_page_indices"], dev["kv_last_page_lens"])
                wrapper.begin_forward(kvp, idx, last, hq, hkv, d, ps, data_type=dtype, indptr_host=h["kv_page_indptr"])
                got.append(wrapper.forward(q, pool.pages[0]).clone())
                wrapper.end_forward()
            assert torch.equal(got[0], got[1])
            outs.append(got[1])
        for t in tasks:
            t.step()
    assert len(outs) == 2 and _lib.read_device_status() == 0
