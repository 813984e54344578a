"""Generate the golden fixtures of tests/golden/ by running the REFERENCE's own
classes (CoLearn-Dev/deserve) on CPU.

Run once, in a container that has the reference tree:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's Python modules unmodified and records what they do;
the fixtures it writes (JSON / NPZ, a few hundred KB) are committed so that the
tests never need the reference tree. Environment stubs used (none of them
touches reference code):
  * torch.utils.cpp_extension.load -> a dummy module, so that importing
    kvcache/virtual.py does not JIT-compile swap.cpp (its only use, the DMA
    inside swap2, needs a GPU; the bookkeeping half of swap2 is what is traced);
  * torch.cuda.Stream -> a no-op object (the reference creates streams in
    constructors);
  * torch.empty(..., pin_memory=True) -> pageable memory (no CUDA driver here);
  * Tensor.to("cuda") -> identity (KVCacheManager.copy_cpu_to_gpu hard-codes it).
"""
from __future__ import annotations

import ast
import hashlib
import json
import os
import random
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def install_stubs() -> None:
    import torch.utils.cpp_extension as cpp

    dummy = types.SimpleNamespace(swap=lambda *a, **k: None)
    cpp.load = lambda *a, **k: dummy
    torch.cuda.Stream = lambda *a, **k: types.SimpleNamespace(synchronize=lambda: None)
    real_empty = torch.empty

    def empty(*a, **k):
        k.pop("pin_memory", None)
        return real_empty(*a, **k)

    torch.empty = empty
    real_to = torch.Tensor.to

    def to(self, *a, **k):
        if a and isinstance(a[0], str) and a[0].startswith("cuda"):
            return self
        return real_to(self, *a, **k)

    torch.Tensor.to = to


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    os.chdir(ref_root)
    install_stubs()
    import deserve_worker.task as task_mod  # sets default dtype fp16 (task.py:9)

    torch.set_default_dtype(torch.float32)
    import deserve_worker.model.context.flash as flash

    cpu = torch.device("cpu")
    flash.main_device = cpu
    from deserve_worker.kvcache.manager import KVCacheManager
    from deserve_worker.kvcache.paged.chunk_pool import CpuChunkPool
    from deserve_worker.kvcache.paged.kvcache import PagedKVCache
    from deserve_worker.kvcache.paged.page_pool import CpuPagePool
    from deserve_worker.kvcache.paged.page_table import PageTableAllocator
    from deserve_worker.kvcache.virtual import CopiedPinnedMemory, VirtualPagedKVCache, VirtualPagePool
    from deserve_worker.task import SamplingParams, TaskData

    sp = SamplingParams()
    out: dict = {}

    # ---- 1. allocator / page-table op trace --------------------------------
    def alloc_trace(seed: int, num_pages: int, page_size: int, max_req: int, n_ops: int):
        rng = random.Random(seed)
        pool = CpuPagePool(1, num_pages, page_size, torch.float16)
        pta = PageTableAllocator(max_req, 4096, page_size, cpu)
        live: dict[int, tuple] = {}
        ops = []
        next_id = 0
        for _ in range(n_ops):
            r = rng.random()
            if (r < 0.3 or not live) and len(live) < max_req:
                c = PagedKVCache.empty(pta, pool)
                live[next_id] = [c, 0]
                ops.append({"op": "new", "id": next_id, "slot": c.page_table.offset})
                next_id += 1
            elif r < 0.8:
                cid = rng.choice(list(live))
                c, tokens = live[cid]
                tokens += rng.choice([1, 1, 1, 7, 33, 150, 400])
                rec = {"op": "extend", "id": cid, "tokens": tokens}
                try:
                    c.extend(tokens)
                    live[cid][1] = tokens
                    rec["table"] = c.page_table.retrieve().tolist()
                except ValueError:
                    rec["error"] = "ValueError"
                rec["num_avails"] = pool.num_avails
                rec["buffer"] = pool.page_buffer.tolist()
                ops.append(rec)
            else:
                cid = rng.choice(list(live))
                c, _ = live.pop(cid)
                c.free()
                ops.append({"op": "free", "id": cid, "num_avails": pool.num_avails,
                            "bitmap_free": int(pool.page_bitmap.sum())})
        return {"seed": seed, "num_pages": num_pages, "page_size": page_size, "max_req": max_req, "ops": ops}

    out["alloc_traces"] = [alloc_trace(0, 100, 16, 8, 120), alloc_trace(1, 300, 8, 16, 200),
                           alloc_trace(2, 70, 16, 4, 80)]

    # ---- 2. descriptor traces ------------------------------------------------
    def desc_to_json(ctx):
        return {"indptr": ctx.indptr.tolist(), "kv_page_indices": ctx.kv_page_indices.tolist(),
                "kv_page_indptr": ctx.kv_page_indptr.tolist(), "kv_last_page_lens": ctx.kv_last_page_lens.tolist(),
                "offsets": ctx.offsets.tolist(), "seqlens": ctx.seqlens.tolist()}

    def desc_trace(seed: int, prompts: list[int], chunk: int, steps: int, page_size: int, num_pages: int):
        """Every task is prefilled in chunks of at most `chunk` tokens (one task's
        chunk per step, like the join stage), then all tasks decode together."""
        pool = CpuPagePool(1, num_pages, page_size, torch.float16)
        pta = PageTableAllocator(len(prompts), 4096, page_size, cpu)
        tasks = [TaskData.empty(f"t{i}", p, sp) for i, p in enumerate(prompts)]
        caches = [PagedKVCache.empty(pta, pool) for _ in prompts]
        trace = []
        for i, t in enumerate(tasks):
            while t.start_pos < t.initial_seqlen:
                t.init(min(chunk, t.initial_seqlen - t.start_pos))
                ctx = flash.FlashForwardCtx.init_paged_forward_ctx([t], [caches[i]])
                trace.append({"tasks": [i], "seqlens": [t.seqlen], "desc": desc_to_json(ctx),
                              "occupied": [caches[i].page_table.occupied]})
                t.step()
        for _ in range(steps):
            ctx = flash.FlashForwardCtx.init_paged_forward_ctx(tasks, caches)
            trace.append({"tasks": list(range(len(tasks))), "seqlens": [t.seqlen for t in tasks],
                          "desc": desc_to_json(ctx), "occupied": [c.page_table.occupied for c in caches]})
            for t in tasks:
                t.step()
        return {"seed": seed, "prompts": prompts, "chunk": chunk, "page_size": page_size, "num_pages": num_pages,
                "steps": trace}

    out["desc_traces"] = [
        desc_trace(0, [100, 37, 16], 4096, 3, 16, 200),
        desc_trace(1, [100], 40, 2, 16, 100),
        desc_trace(2, [random.Random(2).randint(1, 300) for _ in range(6)], 64, 20, 8, 400),
    ]

    # ---- 3. virtual pool region state machine ---------------------------------
    def vstate(pool):
        return {"on": pool.on, "num_avails": pool.num_avails,
                "bitmap": "".join("1" if b else "0" for b in pool.page_bitmap.tolist()),
                "swap_bitmap": "".join("1" if b else "0" for b in pool.swap_bitmap.tolist()),
                "swap_count": pool.swap_count, "buffer": pool.page_buffer.tolist()}

    def virtual_trace(seed: int, main: int, swap: int, page_size: int, rounds: int, n_steps: int):
        rng = random.Random(seed)
        pool = VirtualPagePool(1, main, swap, page_size, cpu, torch.float16)
        pta = PageTableAllocator(64, 4096, page_size, cpu)
        pinned = [CopiedPinnedMemory(16, swap, cpu) for _ in range(rounds)]
        mbs: list[dict[int, list]] = [dict() for _ in range(rounds)]
        ops = [{"op": "init", "state": vstate(pool)}]
        nid = 0
        for step in range(n_steps):
            mb = step % rounds
            pool.switch()
            ops.append({"op": "switch", "state": vstate(pool)})
            if rounds % 2 == 1:
                offset = pool.num_pages_swap if pool.on == 1 else -pool.num_pages_swap
                for cid, (c, _) in mbs[mb].items():
                    c.adjust(offset)
                ops.append({"op": "adjust", "mb": mb, "offset": offset,
                            "tables": {str(cid): c.page_table.retrieve().tolist() for cid, (c, _) in mbs[mb].items()}})
            # free one, add one, grow some
            if mbs[mb] and rng.random() < 0.3:
                cid = rng.choice(list(mbs[mb]))
                c, _ = mbs[mb].pop(cid)
                c.free()
                ops.append({"op": "free", "mb": mb, "id": cid, "state": vstate(pool)})
            if rng.random() < 0.6:
                c = VirtualPagedKVCache.empty(pta, pool)
                mbs[mb][nid] = [c, 0]
                ops.append({"op": "new", "mb": mb, "id": nid, "slot": c.page_table.offset})
                nid += 1
            for cid in list(mbs[mb]):
                c, tokens = mbs[mb][cid]
                tokens += rng.choice([1, 1, page_size, 3 * page_size])
                rec = {"op": "extend", "mb": mb, "id": cid, "tokens": tokens}
                try:
                    c.extend(tokens)
                    mbs[mb][cid][1] = tokens
                    rec["table"] = c.page_table.retrieve().tolist()
                    rec["isswap"] = c.isswap[: c.page_table.occupied].tolist()
                except ValueError:
                    rec["error"] = "ValueError"
                rec["state"] = vstate(pool)
                ops.append(rec)
            nxt, prv = pinned[(mb + 1) % rounds], pinned[(mb - 1 + rounds) % rounds]
            pool.swap2(nxt, prv)
            ops.append({"op": "swap2", "mb": mb, "state": vstate(pool),
                        "to_count": prv.count, "to_bitmap": "".join("1" if b else "0" for b in prv.bitmap.tolist())})
        return {"seed": seed, "main": main, "swap": swap, "page_size": page_size, "rounds": rounds, "ops": ops}

    out["virtual_traces"] = [virtual_trace(0, 6, 4, 16, 2, 12), virtual_trace(1, 20, 10, 8, 3, 18),
                             virtual_trace(2, 12, 8, 16, 4, 16)]

    # a hand-written scenario: two microbatches alternating over a 6 + 4 + 4 page pool
    pool = VirtualPagePool(1, 6, 4, 16, cpu, torch.float16)
    pta = PageTableAllocator(8, 4096, 16, cpu)
    a2 = [{"op": "init", "state": vstate(pool)}]
    mb0 = VirtualPagedKVCache.empty(pta, pool)
    mb0.extend(8 * 16)
    a2.append({"op": "mb0.extend(8p)", "state": vstate(pool), "table": mb0.page_table.retrieve().tolist(),
               "isswap": mb0.isswap[:8].tolist()})
    pool.switch()
    a2.append({"op": "switch", "state": vstate(pool)})
    mb1 = VirtualPagedKVCache.empty(pta, pool)
    mb1.extend(3 * 16)
    a2.append({"op": "mb1.extend(3p)", "state": vstate(pool), "table": mb1.page_table.retrieve().tolist(),
               "isswap": mb1.isswap[:3].tolist()})
    pool.switch()
    a2.append({"op": "switch", "state": vstate(pool)})
    mb0.extend(9 * 16)
    a2.append({"op": "mb0.extend(9p)", "state": vstate(pool), "table": mb0.page_table.retrieve().tolist()})
    mb0.adjust(4)
    a2.append({"op": "mb0.adjust(4)", "table": mb0.page_table.retrieve().tolist()})
    out["virtual_a2"] = a2

    # ---- 4. buddy chunk pool ----------------------------------------------------
    def chunk_trace(seed: int, height: int, n_ops: int):
        rng = random.Random(seed)
        cp = CpuChunkPool(1, height, 1, torch.float16)
        live = []
        ops = []
        for _ in range(n_ops):
            if rng.random() < 0.55 or not live:
                size = rng.choice([1, 1, 2, 3, 5, 8, 13, 2 ** (height - 2)])
                rec = {"op": "alloc", "size": size}
                try:
                    h = cp.alloc(size)
                    live.append(h)
                    rec.update(id=h.id, level=h.level)
                except RuntimeError:
                    rec["error"] = "RuntimeError"
                ops.append(rec)
            else:
                h = live.pop(rng.randrange(len(live)))
                h.free()
                ops.append({"op": "free", "id": h.id, "level": h.level})
            ops[-1]["available"] = [list(x) for x in cp.available_ids]
        return {"seed": seed, "height": height, "ops": ops}

    out["chunk_traces"] = [chunk_trace(0, 6, 120), chunk_trace(1, 8, 200)]

    # ---- 5. per-task offload / reload (layout + data) ---------------------------
    g = torch.Generator().manual_seed(5)
    L, ps = 3, 4
    vpool = VirtualPagePool(L, 10, 3, ps, cpu, torch.float16)
    vpool.pages.copy_(torch.randn(vpool.pages.shape, generator=g).to(torch.float16))
    before = vpool.pages.clone()
    pta = PageTableAllocator(8, 4096, ps, cpu)
    cpool = CpuChunkPool(L, 5, ps, torch.float16)
    mgr = KVCacheManager(vpool, cpool, pta)
    c0 = VirtualPagedKVCache.empty(pta, vpool)
    c0.extend(2 * ps)      # pages 0,1
    c1 = VirtualPagedKVCache.empty(pta, vpool)
    c1.extend(5 * ps)      # pages 2..6
    ids1 = c1.page_table.retrieve().tolist()
    h = mgr.copy_gpu_to_cpu(c1, "x")
    rows = h.retrieve()[: len(ids1) * L].clone()
    c1.free()
    c2 = VirtualPagedKVCache.empty(pta, vpool)
    c2.extend(3 * ps)      # takes buffer pages first
    new = mgr.copy_cpu_to_gpu(h, "x")
    out["offload"] = {
        "seed": 5, "L": L, "ps": ps, "main": 10, "swap": 3, "height": 5,
        "pages_before_sha": sha(before), "ids": ids1, "chunk_id": h.id, "chunk_level": h.level,
        "rows_sha": sha(rows), "new_ids": new.page_table.retrieve().tolist(),
        "isswap": new.isswap[: new.page_table.occupied].tolist(),
        "new_slot": new.page_table.offset, "pages_after_sha": sha(vpool.pages),
        "c2_ids": c2.page_table.retrieve().tolist(),
    }

    (HERE / "host_traces.json").write_text(json.dumps(out, separators=(",", ":")))

    # ---- 6. dense attention + rotary embedding -----------------------------------
    # The function that builds the rotary table lives in a module that allocates
    # CUDA memory at import (execution/exec.py:20); its own source is compiled in
    # isolation instead.
    src = Path(ref_root, "deserve_worker/execution/exec.py").read_text()
    fn = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "precompute_freqs_cis")
    ns: dict = {"torch": torch}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "exec.py", "exec"), ns)
    from deserve_utils.trace import ComponentId
    from deserve_worker.model.args import ModelArgs
    from deserve_worker.model.context.trace import TraceForwardCtx
    from deserve_worker.model.layer.attention import Attention

    arrays = {}
    cases = [("a", 8, 2, 64, 17, 10000.0), ("b", 4, 4, 128, 9, 500000.0), ("c", 8, 1, 128, 12, 500000.0),
             ("d", 4, 4, 64, 1, 500000.0)]
    g = torch.Generator().manual_seed(6)
    for name, hq, hkv, d, n, theta in cases:
        args = ModelArgs(dim=hq * d, n_heads=hq, n_kv_heads=hkv)
        att = Attention(ComponentId(layer="l0", component="attn"), args)
        freqs = ns["precompute_freqs_cis"](d, 256, theta, False)
        xq = torch.randn(1, n, hq, d, generator=g)
        xk = torch.randn(1, n, hkv, d, generator=g)
        xv = torch.randn(1, n, hkv, d, generator=g)
        att.wo.weight.data = torch.eye(hq * d)
        t = TaskData.empty("t", n, sp)
        t.init(n)
        traces: dict = {}
        ctx = TraceForwardCtx.init_trace_forward_ctx([t], freqs, traces, {})
        with torch.inference_mode():
            att.traced_forward(xq, xk, xv, ctx)
        got = {str(k).split(".")[-1]: v for k, v in traces.items()}
        arrays[f"{name}_meta"] = np.array([hq, hkv, d, n, theta], dtype=np.float64)
        arrays[f"{name}_xq"] = xq[0].numpy()
        arrays[f"{name}_xk"] = xk[0].numpy()
        arrays[f"{name}_xv"] = xv[0].numpy()
        arrays[f"{name}_xq_rotary"] = got["xq_rotary"][0].numpy()
        arrays[f"{name}_xk_rotary"] = got["xk_rotary"][0].numpy()
        arrays[f"{name}_output"] = got["output"].reshape(n, hq, d).numpy()
    np.savez_compressed(HERE / "dense_attention.npz", **arrays)
    print("wrote", HERE / "host_traces.json", HERE / "dense_attention.npz")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
