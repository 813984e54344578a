"""Mixed prefill / decode under page churn at full size: the stage loop of one GPU
(StageProcessor) fed by the first stage's admission and swap policies
(StepPlanner), on a Llama-3-8B-shaped random-init model.

512 requests arrive a few per iteration; prompt lengths ~ LogNormal(6.5, 0.8)
clipped to [16, 8192]; prompts are prefilled in chunks of at most 512 rows per
step through the tensor-core paged attention kernel, mixed with the decode rows
of the running requests; every request generates a seeded number of tokens in
[16, 128] and then leaves, its pages go back to the pool and are handed to later
arrivals. The pool holds well under half of the pages the whole job touches, so
pages are recycled all the time and, when the running requests outgrow the pool,
the swap policy offloads parked requests to pinned host memory and brings them
back.

It plays the role of the reference's mixed benchmark
(deserve_worker/benchmark/mixed.py:19-88: prefill + decode rows in one
BatchPrefill step) under the scheduling of
deserve_worker/engine/pipeline/stage/join.py:11-179 and scheduler.py:66-90.
Synthetic prompts (random token ids) stand in for the reference's datasets.
"""
from __future__ import annotations

import time

import numpy as np
import torch

from . import _lib
from .engine import StageProcessor, StepRequest
from .kvcache import CpuChunkPool, KVCacheManager, PageTableAllocator, VirtualPagePool
from .model import LlamaStage, ModelArgs, llama_3_8b_args
from .scheduling import StepPlanner
from .task import SamplingParams, TaskManager


def longest_free_run(free: np.ndarray) -> int:
    """Length of the longest run of consecutive free pages in a bitmap (True = free)."""
    if not free.any():
        return 0
    edges = np.diff(np.concatenate([[0], free.astype(np.int8), [0]]))
    return int((np.flatnonzero(edges == -1) - np.flatnonzero(edges == 1)).max())


def make_arrivals(n: int, seed: int, vocab: int, lo: int = 16, hi: int = 8192, new_lo: int = 16, new_hi: int = 128):
    rng = np.random.default_rng(seed)
    lens = np.clip(rng.lognormal(6.5, 0.8, size=n), lo, hi).astype(np.int64)
    new = rng.integers(new_lo, new_hi + 1, size=n)
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(1, vocab, (int(l),), generator=g, dtype=torch.int32) for l in lens]
    return lens, new, prompts


def run_fragmentation(dev: torch.device, policy: str = "prefill_first", n_arrivals: int = 512, per_iteration: int = 4,
                      model: ModelArgs | None = None, pool_fraction: float = 0.4, max_batch_rows: int = 512,
                      chunk_pool_height: int = 13, seed: int = 0, stats_every: int = 16, max_iterations: int = 20000,
                      prompt_hi: int = 8192) -> dict:
    model = model or llama_3_8b_args
    ps, dtype, rounds = model.page_size, torch.bfloat16, 2
    lens, new, prompts = make_arrivals(n_arrivals, seed, model.vocab_size, hi=prompt_hi)
    demand = int(sum(-(-(int(l) + int(k)) // ps) for l, k in zip(lens, new)))
    biggest = int(max(-(-(int(l) + int(k)) // ps) for l, k in zip(lens, new)))
    main_pages = max(int(demand * pool_fraction), 3 * biggest)
    stage = LlamaStage(model, 0, model.n_layers, dev, dtype, seed=seed)
    pool = VirtualPagePool(model.n_layers, main_pages, 0, ps, dev, dtype, n_kv_heads=model.n_kv_heads,
                           head_dim=model.head_dim)
    pta = PageTableAllocator(n_arrivals, (prompt_hi + 128 + 2 * ps) // ps * ps, ps, dev)
    chunks = CpuChunkPool(model.n_layers, chunk_pool_height, ps, dtype, n_kv_heads=model.n_kv_heads,
                          head_dim=model.head_dim)
    mgr = KVCacheManager(pool, chunks, pta)
    tm = TaskManager(pool.num_pages, ps)
    proc = StageProcessor(mgr, tm, stage, pta, rounds, ignore_eos=True)
    planner = StepPlanner(tm, rounds, policy, max_batch_size=max_batch_rows)
    reqs = [StepRequest.empty(mb, torch.int32, dev) for mb in range(rounds)]

    done: set = set()
    produced = {i: 0 for i in range(n_arrivals)}
    next_arrival = 0
    ever_used = np.zeros(pool.num_pages, dtype=bool)
    prev_free = np.ones(pool.num_pages, dtype=bool)
    samples, events = [], []
    prompt_rows = generated = offloads = reloads = steps = reused_total = 0
    torch.cuda.synchronize(dev)
    t_wall = time.perf_counter()
    e_first = torch.cuda.Event(enable_timing=True)
    e_first.record()
    it = 0
    while len(done) < n_arrivals and it < max_iterations:
        for _ in range(per_iteration):
            if next_arrival < n_arrivals:
                i = next_arrival
                planner.add_prompt(f"r{i}", prompts[i].to(dev, non_blocking=True), SamplingParams(max_new_tokens=int(new[i]), max_seq_len=prompt_hi + 256))
                next_arrival += 1
        for mb in range(rounds):
            req = planner.convert(reqs[mb], free_pages=pool.num_avails)
            offloads += len(req.offload_task_ids)
            reloads += len(req.reload_task_ids)
            ids = list(req.exec_task_ids)
            seqlens = list(req.exec_seqlens)[: len(ids)]
            in_prompt = [tm.get(t).start_pos < tm.get(t).initial_seqlen for t in ids]  # before the step
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            proc.synchronize()
            reqs[mb], result = proc.process_step(req)
            e1.record()
            if result is None:
                continue
            steps += 1
            rows_prompt = sum(n for n, p in zip(seqlens, in_prompt) if p)
            events.append((e0, e1, rows_prompt, len(result.all_task_ids)))
            prompt_rows += rows_prompt
            generated += len(result.all_task_ids)
            for t in result.all_task_ids:
                produced[int(t[1:])] += 1
            done.update(result.done_task_ids)
            free = pool.page_bitmap.numpy().copy()
            used = ~free
            reused_total += int((used & prev_free & ever_used).sum())  # taken now, free a step ago, used before
            ever_used |= used
            prev_free = free
            if steps % stats_every == 0:
                samples.append({"step": steps, "pages_free": int(pool.num_avails), "longest_free_run": longest_free_run(free),
                                "pages_reused_so_far": reused_total, "tasks_resident": sum(
                                    len(m.ongoing_paged_kvcaches) for m in proc.microbatches),
                                "tasks_offloaded": len(proc.offloaded_kvcaches)})
        it += 1
    e_last = torch.cuda.Event(enable_timing=True)
    e_last.record()
    torch.cuda.synchronize(dev)
    total_ms = e_first.elapsed_time(e_last)
    wall_s = time.perf_counter() - t_wall
    ms_prefill = sum(a.elapsed_time(b) for a, b, rp, _ in events if rp > 0)
    ms_decode = sum(a.elapsed_time(b) for a, b, rp, _ in events if rp == 0)
    status = _lib.read_device_status()
    keep = samples if len(samples) <= 24 else samples[:: max(1, len(samples) // 24)]
    return {
        "workload": f"{n_arrivals} requests, prompts ~ LogNormal(6.5, 0.8) in [16, {prompt_hi}], chunks of <= {max_batch_rows} rows per "
                    f"step, 16-128 generated tokens each, {model.n_layers}-layer {model.dim}-wide model, join policy {policy}",
        "finished": len(done), "iterations": it, "steps": steps, "prompt_tokens": int(prompt_rows),
        "generated_tokens": int(generated), "expected_generated_tokens": int(new.sum()),
        "all_requests_produced_their_tokens": all(produced[i] == int(new[i]) for i in range(n_arrivals)),
        "total_ms": total_ms, "wall_s": wall_s,
        "prompt_tokens_per_s": prompt_rows / (total_ms * 1e-3), "generated_tokens_per_s": generated / (total_ms * 1e-3),
        "ms_in_steps_with_prompt_rows": ms_prefill, "ms_in_pure_decode_steps": ms_decode,
        "pool_pages": pool.num_pages, "pages_the_job_touches": demand, "pool_fraction": pool.num_pages / demand,
        "pages_reused": reused_total, "offloaded_tasks": offloads, "reloaded_tasks": reloads,
        "pages_free_at_end": int(pool.num_avails), "samples_every_%d_steps" % stats_every: keep,
        "device_status": status,
    }
