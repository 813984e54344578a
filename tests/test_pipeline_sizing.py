"""Page accounting of the pipelined job on the host (no GPU): with the pools
sized by pipeline_driver.size_pools, the allocator, the region state machine and
the descriptor builder run the whole schedule of the 70B-shaped configuration —
8 microbatches x 128 sequences, 512-token prompts, 256 generated tokens — without
ever running out of pages, and the last page of every sequence ends up in its
microbatch's swap region (that is what makes the region swap carry live data)."""
import numpy as np
import pytest
import torch

import deserve_b200 as dk
from deserve_b200.context import build_step
from deserve_b200.pipeline_driver import size_pools


def _simulate(model, M, S, prompt, new_tokens, prefill_seqs, sz):
    ps = model.page_size
    pool = dk.VirtualPagePool(1, sz["main_pages"], sz["swap_pages"], ps, torch.device("cpu"), torch.float32,
                              n_kv_heads=1, head_dim=1)
    Mw = sz["concurrent"]
    pta = dk.PageTableAllocator(Mw * S, (prompt + new_tokens + ps) // ps * ps, ps, torch.device("cpu"))
    pinned = [dk.CopiedPinnedMemory(8, sz["swap_pages"], torch.device("cpu"), torch.float32) for _ in range(Mw)]
    tasks = [[dk.TaskData.empty(f"m{m}s{i}", prompt) for i in range(S)] for m in range(Mw)]
    caches = [[None] * S for _ in range(Mw)]
    P = -(-S // prefill_seqs)
    live_out = []
    for s in range(P + new_tokens - 1):
        for m in range(Mw):
            pool.switch()
            if Mw % 2 == 1:
                off = pool.num_pages_swap if pool.on == 1 else -pool.num_pages_swap
                for kv in caches[m]:
                    if kv is not None:
                        kv.adjust(off)
            sel = range(s * prefill_seqs, min(S, (s + 1) * prefill_seqs)) if s < P else range(S)
            for i in sel:
                if caches[m][i] is None:
                    caches[m][i] = dk.VirtualPagedKVCache.empty(pta, pool)
                tasks[m][i].init(prompt if s < P else 1)
            build_step([tasks[m][i] for i in sel], [caches[m][i] for i in sel])  # raises ValueError when out of pages
            for i in sel:
                tasks[m][i].step()
            if sz["swap_pages"]:
                pool._handoff(pinned[(m + 1) % Mw], pinned[(m - 1) % Mw])
                live_out.append(pool._live_pages(pinned[(m - 1) % Mw].bitmap))
    in_region = [sum(int(kv.isswap[: kv.page_table.occupied].sum()) for kv in caches[m]) for m in range(Mw)]
    pages = [sum(kv.page_table.occupied for kv in caches[m]) for m in range(Mw)]
    return pool, in_region, pages, live_out


@pytest.mark.parametrize("stages,layers_here,budget_gb,new_tokens", [(8, 10, 150, 256), (4, 20, 140, 256), (2, 40, 105, 256),
                                                                    (8, 10, 150, 26)])
def test_config4_schedule_never_runs_out_of_pages_and_fills_the_regions(stages, layers_here, budget_gb, new_tokens):
    from deserve_b200.model import llama_3_70b_args as model

    sz = size_pools(model, layers_here, 8, 128, 512, new_tokens, int(budget_gb * 1e9), stages, sized_for_tokens=256)
    assert sz["concurrent"] == (4 if stages == 2 else 8)
    assert sz["swap_pages"] == 128 + 64
    pool, in_region, pages, live_out = _simulate(model, 8, 128, 512, new_tokens, 8, sz)
    want = -(-(512 + new_tokens) // 16) * 128
    assert pages == [want] * sz["concurrent"]
    # the last growth round of every microbatch landed in its region: one page per sequence, give or take
    # the pages the prefetch buffer took from the main area's slack
    assert all(64 <= n <= 128 for n in in_region), in_region
    assert max(live_out) <= sz["swap_pages"] and max(live_out) >= 64


def test_one_gpu_holds_one_microbatch_and_swaps_nothing():
    from deserve_b200.model import llama_3_70b_args as model

    sz = size_pools(model, 80, 8, 128, 512, 256, int(45e9), 1)
    assert sz["concurrent"] == 1 and sz["swap_pages"] == 0
    with pytest.raises(ValueError):
        size_pools(model, 40, 8, 128, 512, 256, int(20e9), 2)  # two stages cannot run on one microbatch
