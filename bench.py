#!/usr/bin/env python
"""Benchmark of the paged KV-cache hot path (the Llama-3-8B-shaped decode configuration).

Workload "llama3-8b-decode-kv": 32 layers, 32 q / 8 kv heads, head_dim 128,
bf16, page size 16; 256 sequences with context lengths uniform in [512, 4096];
physical pages dealt from a seeded random permutation of a pool of 1.25x the
pages in use; K/V ~ 0.5*N(0,1). One step = one decode token for every sequence:
in each of the 32 layers, append the new K/V row and run paged GQA decode
attention (layer l's output is layer l+1's query). Synthetic data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 (launched with torch.distributed.run): the layers are split evenly over N
pipeline stages and N microbatches of 256 sequences rotate through them (weak
scaling: the KV bytes per GPU stay the same); activations hop between stages
with NCCL send/recv.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = "llama3-8b-decode-kv"
METRIC = "decode_tokens_per_s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    # shape overrides for small profiling captures; the defaults are the benchmark
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx-lo", type=int, default=512)
    ap.add_argument("--ctx-hi", type=int, default=4096)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end pass")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the chunked-prefill attention measurement")
    ap.add_argument("--prefill-only", action="store_true", help="run only the chunked-prefill measurement (profiling)")
    ap.add_argument("--prefill-reqs", type=int, default=32)
    ap.add_argument("--prefill-ctx", type=int, default=4096)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--no-swap", action="store_true", help="skip the KV swap stress (16 GiB of scattered pages out and back)")
    ap.add_argument("--swap-seqs", type=int, default=64)
    ap.add_argument("--swap-tokens", type=int, default=2048)
    ap.add_argument("--hop", default="nccl", choices=["auto", "peer", "nccl"],
                    help="N > 1: how a stage hands its activations on. peer = the sender's kernel stores into the "
                         "next GPU's inbox over NVLink (deserve_b200.peer); nccl = grouped send/recv; auto = peer, "
                         "and nccl if peer memory cannot be set up")
    ap.add_argument("--measure-hop", action="store_true",
                    help="N > 1 only: time one 2 MiB hop around the ring, NCCL send/recv against the peer-memory "
                         "transport, with nothing else on the GPUs; prints its own JSON line")
    ap.add_argument("--compare-library", action="store_true",
                    help="only time flashinfer (the library the reference calls) and this package on the same "
                         "one-layer decode and chunked-prefill inputs; prints its own JSON line")
    return ap.parse_args()


def make_lengths(args, seed=0):
    rng = np.random.default_rng(seed)
    return rng.integers(args.ctx_lo, args.ctx_hi + 1, size=args.batch)


def algorithmic_bytes_per_layer(kv_tokens, n_pages, args, es=2):
    """decode attention: every live K/V element once, q in and out once, the
    page list and the three per-request descriptor arrays once."""
    B = args.batch
    return (kv_tokens * 2 * args.kv_heads * args.head_dim * es + 2 * B * args.q_heads * args.head_dim * es
            + 4 * (n_pages + 2 * (B + 1)))


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with NVML while the timed
    region runs (read-only queries)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            if visible:
                index = int(visible.split(",")[index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ---------------------------------------------------------------------------
# CPU oracle arm (cpu_baseline of our line, and the whole --impl reference run)
# ---------------------------------------------------------------------------
def cpu_reference_arm(args, steps, warmup, n_seq=128):
    """The reference's torch path restated on the host (oracle/): one layer of
    the workload on the first n_seq sequences per sample — append one token by
    index assignment, gather K/V through the page table, dense fp32 attention.
    tok/s is scaled to the full step: n_seq tokens per (sample time * layers)."""
    from oracle import kv_math

    torch.set_num_threads(os.cpu_count())
    n_seq = min(n_seq, args.batch)
    lens = make_lengths(args)[:n_seq] + 1
    ps, hkv, d, hq = args.page_size, args.kv_heads, args.head_dim, args.q_heads
    n_pages = (lens + ps - 1) // ps
    total = int(n_pages.sum())
    perm = np.random.default_rng(1).permutation(int(total * 1.25) + 1)[:total].astype(np.int32)
    desc = {"indptr": np.arange(n_seq + 1, dtype=np.int32), "kv_page_indices": perm,
            "kv_page_indptr": np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32),
            "kv_last_page_lens": ((lens - 1) % ps + 1).astype(np.int32)}
    g = torch.Generator().manual_seed(2)
    pages = (torch.randn(int(total * 1.25) + 1, 2, ps, hkv, d, generator=g) * 0.5).to(torch.bfloat16)
    q = torch.randn(n_seq, hq, d, generator=g).to(torch.bfloat16)
    k = torch.randn(n_seq, hkv, d, generator=g).to(torch.bfloat16)
    v = torch.randn(n_seq, hkv, d, generator=g).to(torch.bfloat16)

    def sample():
        kv_math.append_paged(pages, k, v, desc, ps)
        return kv_math.paged_attention(q, pages, desc, ps, causal=False)

    for _ in range(warmup):
        sample()
    t0 = time.perf_counter()
    for _ in range(steps):
        sample()
    dt = (time.perf_counter() - t0) / steps
    tok_s = n_seq / (dt * args.layers)
    info = {"value": tok_s, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"1 of {args.layers} layers x first {n_seq} of {args.batch} sequences per step "
                      f"({dt * 1e3:.1f} ms/sample, CPU torch, scaled to the full step)"}
    return info, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    info, dt = cpu_reference_arm(args, max(1, args.steps), max(1, args.warmup))
    line = {"impl": "reference", "metric": METRIC, "value": info["value"], "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(args, args.gpus), "cpu_baseline": info,
            "e2e": {"value": info["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def config_dict(args, n):
    return {"workload": WORKLOAD, "layers": args.layers, "q_heads": args.q_heads, "kv_heads": args.kv_heads,
            "head_dim": args.head_dim, "page_size": args.page_size, "sequences_per_microbatch": args.batch,
            "microbatches": n, "context": f"U[{args.ctx_lo},{args.ctx_hi}]", "pool": "1.25x pages, seeded permutation",
            "parallelism": f"pp{n}" if n > 1 else "single", "l2": "inputs larger than L2 (KV read per step >> 126 MB)"}


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def build_microbatch(dk, pool, pta, lens, page_ids, tag):
    """Tasks + caches of one microbatch whose pages are the given (permuted) ids."""
    tasks, caches = [], []
    at = 0
    ps = pool.page_size
    for i, n in enumerate(lens):
        n_pg = (int(n) + ps - 1) // ps
        t = dk.TaskData.empty(f"{tag}-{i}", int(n))
        t.start_pos, t.seqlen = int(n), 1
        kv = dk.PagedKVCache.empty(pta, pool)
        kv.page_table.extend(page_ids[at : at + n_pg])
        at += n_pg
        tasks.append(t)
        caches.append(kv)
    return tasks, caches


def host_link_peak(dev, nbytes=1 << 30, reps=5):
    """Best-of-reps pinned cudaMemcpyAsync bandwidth in each direction (GB/s)."""
    host = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    devb = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    out = {}
    for name, dst, src in (("h2d", devb, host), ("d2h", host, devb)):
        best = 0.0
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dst.copy_(src, non_blocking=True)
            b.record()
            torch.cuda.synchronize()
            best = max(best, nbytes / (a.elapsed_time(b) * 1e-3) / 1e9)
        out[name] = best
    return out


def prefill_measure(dk, args, dev, iters=5):
    """Chunked-prefill attention (mixed prefill/decode configuration's shape): prefill_reqs requests that already hold
    prefill_ctx tokens each get a chunk of prefill_chunk new tokens; ragged causal attention of the
    chunk against the paged K/V on the tcgen05 kernel, one layer. Reports dense-equivalent TFLOP/s
    (4 * Hq * D * visible (q, kv) pairs) against the measured bf16 GEMM peak."""
    from deserve_b200 import ops

    ps, hq, hkv, d = args.page_size, args.q_heads, args.kv_heads, args.head_dim
    B, ctx, n = args.prefill_reqs, args.prefill_ctx, args.prefill_chunk
    lens = np.full(B, ctx + n)
    n_pages = (lens + ps - 1) // ps
    total = int(n_pages.sum())
    pool_pages = int(total * 1.25) + 1
    g = torch.Generator(device=dev).manual_seed(7)
    pages = torch.empty(pool_pages, 2, ps, hkv, d, dtype=torch.bfloat16, device=dev).normal_(0, 0.5, generator=g)
    q = torch.randn(B * n, hq, d, device=dev, generator=g).to(torch.bfloat16)
    qo = (np.arange(B + 1) * n).astype(np.int32)
    kvp = np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32)
    idx = np.random.default_rng(3).permutation(pool_pages)[:total].astype(np.int32)
    last = ((lens - 1) % ps + 1).astype(np.int32)
    plan = np.zeros(ops.prefill_plan_capacity(B * n, B, hq // hkv), dtype=np.int32)
    used = ops.make_prefill_plan(qo, lens.astype(np.int32), hq, hkv, d, ps, torch.bfloat16, True, plan)
    t = lambda a: torch.from_numpy(a).to(dev)
    qo_d, kvp_d, idx_d, last_d, plan_d = t(qo), t(kvp), t(idx), t(last), t(plan[:used].copy())
    out = torch.empty_like(q)

    def run():
        ops.paged_prefill(q, qo_d, pages, idx_d, kvp_d, last_d, plan, plan_d, out=out)

    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    pairs = B * sum(ctx + j + 1 for j in range(n))
    flops = 4.0 * hq * d * pairs
    peak = 1646.8
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except Exception:
        peak = 1590.0
    tf = flops / (ms * 1e-3) / 1e12
    return {"workload": f"{B} requests x ({ctx} context + {n}-token chunk), causal, 1 layer", "ms": ms,
            "tflops": tf, "peak_tflops": peak, "frac": tf / peak, "prefill_tokens_per_s_per_layer": B * n / (ms * 1e-3),
            "bound": "tensor"}


def library_compare(dk, args, dev, iters=20):
    """flashinfer's paged decode / prefill wrappers (what the reference calls) and this package's on the
    same tensors: one layer of the benchmark's decode shape and the chunked-prefill case. Plans are made
    outside the timed loops on both sides; K/V read per decode launch is far larger than L2."""
    import flashinfer as fi
    from deserve_b200 import ops

    ps, hq, hkv, d = args.page_size, args.q_heads, args.kv_heads, args.head_dim
    out = {"flashinfer": fi.__version__}

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    def case(lens, new):
        n_pages = (lens + ps - 1) // ps
        total = int(n_pages.sum())
        pool_pages = int(total * 1.25) + 1
        g = torch.Generator(device=dev).manual_seed(7)
        pages = torch.empty(pool_pages, 2, ps, hkv, d, dtype=torch.bfloat16, device=dev).normal_(0, 0.5, generator=g)
        q = torch.randn(int(new.sum()), hq, d, device=dev, generator=g).to(torch.bfloat16)
        host = {"qo": np.concatenate([[0], np.cumsum(new)]).astype(np.int32),
                "kvp": np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32),
                "idx": np.random.default_rng(3).permutation(pool_pages)[:total].astype(np.int32),
                "last": ((lens - 1) % ps + 1).astype(np.int32)}
        return pages, q, host, {k: torch.from_numpy(v).to(dev) for k, v in host.items()}

    ws_fi = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ws = torch.empty(128 << 20, dtype=torch.uint8, device=dev)
    # decode: one layer of the benchmark batch
    lens = make_lengths(args).astype(np.int64)
    pages, q, host, t = case(lens, np.ones(len(lens), dtype=np.int64))
    alg = algorithmic_bytes_per_layer(int(lens.sum()), int(((lens + ps - 1) // ps).sum()), args)
    w = fi.BatchDecodeWithPagedKVCacheWrapper(ws_fi, "NHD")
    w.plan(t["kvp"], t["idx"], t["last"], hq, hkv, d, ps, pos_encoding_mode="NONE", q_data_type=torch.bfloat16,
           kv_data_type=torch.bfloat16)
    ref = w.run(q, pages)
    ms_fi = timed(lambda: w.run(q, pages))
    mine = dk.BatchDecodeWithPagedKVCacheWrapper(ws)
    mine.begin_forward(t["kvp"], t["idx"], t["last"], hq, hkv, d, ps, data_type=torch.bfloat16, indptr_host=host["kvp"])
    got = mine.forward(q, pages)
    ms_us = timed(lambda: mine.forward(q, pages))
    out["decode"] = {"workload": f"{len(lens)} sequences U[{args.ctx_lo},{args.ctx_hi}], one layer",
                     "flashinfer_ms": ms_fi, "ours_ms": ms_us, "flashinfer_GBps": alg / ms_fi / 1e6,
                     "ours_GBps": alg / ms_us / 1e6, "max_abs_diff": (got.float() - ref.float()).abs().max().item()}
    del pages, q
    # chunked prefill
    B, ctx, n = args.prefill_reqs, args.prefill_ctx, args.prefill_chunk
    lens = np.full(B, ctx + n, dtype=np.int64)
    pages, q, host, t = case(lens, np.full(B, n, dtype=np.int64))
    flops = 4.0 * hq * d * B * sum(ctx + j + 1 for j in range(n))
    wp = fi.BatchPrefillWithPagedKVCacheWrapper(ws_fi, "NHD")
    wp.plan(t["qo"], t["kvp"], t["idx"], t["last"], hq, hkv, d, ps, causal=True, pos_encoding_mode="NONE",
            q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16)
    ref = wp.run(q, pages)
    ms_fi = timed(lambda: wp.run(q, pages))
    minep = dk.BatchPrefillWithPagedKVCacheWrapper(ws)
    minep.begin_forward(t["qo"], t["kvp"], t["idx"], t["last"], hq, hkv, d, ps, data_type=torch.bfloat16,
                        qo_indptr_host=host["qo"], kv_indptr_host=host["kvp"], last_page_len_host=host["last"])
    got = minep.forward(q, pages, causal=True)
    ms_us = timed(lambda: minep.forward(q, pages, causal=True))
    out["prefill"] = {"workload": f"{B} requests x ({ctx} context + {n}-token chunk), causal, one layer",
                      "flashinfer_ms": ms_fi, "ours_ms": ms_us, "flashinfer_TFLOPs": flops / ms_fi / 1e9,
                      "ours_TFLOPs": flops / ms_us / 1e9, "max_abs_diff": (got.float() - ref.float()).abs().max().item()}
    return out


def measure_hop(args, rank, world, dev, dist, iters=200):
    """Every rank sends [batch, q_heads, head_dim] bf16 to its successor and receives from its predecessor,
    `iters` times back to back, once with a grouped NCCL send/recv and once through deserve_b200.peer.PeerHop.
    Device time per hop, max over ranks."""
    from deserve_b200.peer import PeerHop

    shape = (args.batch, args.q_heads, args.head_dim)
    y = torch.randn(shape, device=dev).to(torch.bfloat16)
    buf = torch.empty_like(y)
    nxt, prv = (rank + 1) % world, (rank - 1) % world

    def nccl_hop():
        for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, y, nxt), dist.P2POp(dist.irecv, buf, prv)]):
            w.wait()

    hop = PeerHop(rank, world, shape, torch.bfloat16, dev, dist.group.WORLD)

    def peer_hop():
        hop.send(y)
        got = hop.recv()
        buf.copy_(got)  # a consumer kernel, as the first layer's attention would be
        hop.release()

    out = {}
    for name, fn in (("nccl", nccl_hop), ("peer", peer_hop)):
        for _ in range(10):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[f"{name}_us_per_hop"] = float(t.item())
    hop.close()
    out["bytes"] = y.numel() * 2
    out["n_gpus"] = world
    return out


def swap_stress(dk, pool, free_ids, args, dev, decode_step):
    """KV swap stress: the KV of swap_seqs x swap_tokens tokens, all layers, scattered over the
    permuted pool, is swapped out to pinned host chunks and back into DIFFERENT pages while decode
    attention of another microbatch runs on the main stream. Bit-exactness is checked with a 32-bit
    checksum of every (layer, page) before and after, and exactly on the first and last layer."""
    ps, L = pool.page_size, pool.num_layers
    n_seq, n_pg = args.swap_seqs, (args.swap_tokens + ps - 1) // ps
    total = n_seq * n_pg
    free_ids = free_ids[pool._bitmap[free_ids]]  # pages the decode microbatch grew into since are not free
    ids_a = torch.from_numpy(np.ascontiguousarray(free_ids[:total]).astype(np.int64)).to(dev)
    height = int(np.ceil(np.log2(max(total, 2)))) + 1
    peak = host_link_peak(dev)
    chunks = dk.CpuChunkPool(L, height, ps, pool.main_dtype, n_kv_heads=pool.n_kv_heads, head_dim=pool.head_dim)
    pta = dk.PageTableAllocator(n_seq, n_pg * ps, ps, dev)
    mgr = dk.KVCacheManager(pool, chunks, pta, staging_bytes=4 * total * pool.page_bytes + 1024)
    caches = []
    for i in range(n_seq):
        kv = dk.VirtualPagedKVCache.empty(pta, pool)
        kv.page_table.extend(free_ids[i * n_pg : (i + 1) * n_pg])
        caches.append(kv)
    pool._bitmap[free_ids[:total]] = False
    pool.num_avails -= total

    def checksums(ids):
        return torch.stack([pool.pages[l, ids].view(torch.int32).sum(dim=(1, 2, 3, 4), dtype=torch.int64)
                            for l in range(L)])

    before = checksums(ids_a)
    first, last = pool.pages[0, ids_a].clone(), pool.pages[L - 1, ids_a].clone()
    nbytes = total * L * pool.page_bytes
    decode_stream = torch.cuda.Stream(device=dev)
    steps = 24

    def timed(fn):
        torch.cuda.synchronize()
        cur = torch.cuda.current_stream(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(cur)
        res = fn()  # asynchronous: pack/unpack kernels and DMA bursts are only queued here
        with torch.cuda.stream(decode_stream):  # meanwhile another microbatch decodes
            for _ in range(steps):
                decode_step()
        cur.wait_stream(mgr.stream)
        cur.wait_stream(mgr.dma_stream)
        e1.record(cur)
        torch.cuda.synchronize()
        return res, nbytes / (e0.elapsed_time(e1) * 1e-3) / 1e9

    handles, out_gbs = timed(lambda: mgr.offload_many(caches))
    for kv in caches:
        kv.free()
    pool.pages[:, ids_a] = 0  # the old pages are gone
    new_caches, in_gbs = timed(lambda: mgr.reload_many(handles))
    ids_b = torch.from_numpy(np.concatenate([c.page_table.retrieve_np() for c in new_caches]).astype(np.int64)).to(dev)
    moved = int((ids_a != ids_b).sum().item())
    ok = bool(torch.equal(before, checksums(ids_b)) and torch.equal(first, pool.pages[0, ids_b])
              and torch.equal(last, pool.pages[L - 1, ids_b]))
    for h in handles:
        h.free()
    return {"bytes_each_way": nbytes, "out_GBps": out_gbs, "in_GBps": in_gbs, "host_link_peak_d2h_GBps": peak["d2h"],
            "host_link_peak_h2d_GBps": peak["h2d"], "frac_out": out_gbs / peak["d2h"], "frac_in": in_gbs / peak["h2d"],
            "bit_exact": ok, "pages_that_changed_id": moved, "pages": total, "layers": L,
            "concurrent": f"{steps} decode steps of the 256-sequence microbatch on another stream"}


def run_ours(args):
    import torch.distributed as dist

    import deserve_b200 as dk
    from deserve_b200 import _lib
    from deserve_b200.engine import KVStage, RingPipeline, prepare_decode_step

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.compare_library:
        torch.cuda.set_device(local)
        print(json.dumps({"library_comparator": library_compare(dk, args, torch.device("cuda", local))}), flush=True)
        return
    if args.prefill_only:
        torch.cuda.set_device(local)
        print(json.dumps({"prefill": prefill_measure(dk, args, torch.device("cuda", local))}), flush=True)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only
        dist.init_process_group("nccl", device_id=dev)
    if args.measure_hop:
        if world < 2:
            raise SystemExit("--measure-hop needs --gpus 2 or more")
        res = measure_hop(args, rank, world, dev, dist)
        if rank == 0:
            print(json.dumps({"hop": res}), flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return
    if args.layers % world:
        raise SystemExit("--layers must be divisible by --gpus")
    L = args.layers // world
    M = world  # microbatches
    B, ps, hq, hkv, d = args.batch, args.page_size, args.q_heads, args.kv_heads, args.head_dim
    K, Wm = args.steps, args.warmup
    total_steps = Wm + K
    sm_count = _lib.device_info()[0]

    # ---- pool: M microbatches, pages from a seeded permutation ---------------------
    lens0 = make_lengths(args)
    final_pages = int(((lens0 + 2 * total_steps + 2 + ps - 1) // ps).sum())  # room for value + e2e passes
    pool_pages = int(np.ceil(1.25 * final_pages * M)) + 64
    do_swap = world == 1 and not args.no_swap
    swap_pages = args.swap_seqs * ((args.swap_tokens + ps - 1) // ps) if do_swap else 0
    pool_pages += 2 * swap_pages  # the swapped tasks' pages, and the different pages they come back to
    pool = dk.VirtualPagePool(L, pool_pages, 0, ps, dev, torch.bfloat16, n_kv_heads=hkv, head_dim=d)
    perm = np.random.default_rng(1).permutation(pool_pages).astype(np.int32)
    pta = dk.PageTableAllocator(B * M, 8192, ps, dev)
    gen = torch.Generator(device=dev).manual_seed(2 + rank)
    for layer in range(L):  # K/V ~ 0.5 * N(0,1)
        pool.pages[layer].normal_(0.0, 0.5, generator=gen)
    mbs = []
    at = 0
    for m in range(M):
        n_now = int(((lens0 + ps - 1) // ps).sum())
        tasks, caches = build_microbatch(dk, pool, pta, lens0, perm[at : at + n_now], f"mb{m}")
        at += n_now
        mbs.append((tasks, caches))
    used = perm[:at]
    pool._bitmap[used] = False
    pool.num_avails -= len(used)

    k_new = (torch.randn(M, L, B, hkv, d, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    v_new = (torch.randn(M, L, B, hkv, d, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    q0 = [torch.randn(B, hq, d, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + m)).to(torch.bfloat16)
          for m in range(M)]
    stage = KVStage(pool, hq, 0, L)

    # ---- descriptors + plans of every (microbatch, token step), device resident ------
    descs = {}
    for s in range(total_steps):
        for m, (tasks, caches) in enumerate(mbs):
            descs[(m, s)] = prepare_decode_step(tasks, caches, hq, sm_count)
            for t in tasks:
                t.step()
    torch.cuda.synchronize()

    attn_events = []
    launches = [0]

    def stage_fn(u, m, s, x):
        launches[0] += L * (2 + (1 if descs[(m, s)].workspace_bytes > 0 else 0))
        return stage.forward(x, k_new[m], v_new[m], descs[(m, s)])

    peer_hop, hop_name = None, "none"
    if world > 1:
        hop_name = "nccl send/recv"
        if args.hop in ("auto", "peer"):
            ok = torch.ones(1, device=dev)
            try:
                from deserve_b200.peer import PeerHop
                peer_hop = PeerHop(rank, world, (B, hq, d), torch.bfloat16, dev, dist.group.WORLD)
            except Exception as exc:  # no peer mapping on this node: every rank must take the same path
                if args.hop == "peer":
                    raise
                print(f"[bench] rank {rank}: peer memory hop unavailable ({exc!r})", file=sys.stderr, flush=True)
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                peer_hop = None
            else:
                hop_name = "peer-memory stores + flags"
    pipe = RingPipeline(rank, world, stage_fn, lambda m: q0[m], total_steps, dist=dist, peer_hop=peer_hop)

    def barrier():
        if world > 1:
            dist.barrier()

    # ---- warm-up (also fills the ring), then the timed K steps -----------------------
    pipe.advance(Wm * M)
    torch.cuda.synchronize()
    barrier()
    launches[0] = 0
    hop_launches0 = peer_hop.launches if peer_hop is not None else 0
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        torch.cuda.synchronize()
        t_start.record()
        pipe.advance(K * M)
        t_end.record()
        torch.cuda.synchronize()
    barrier()
    ms = t_start.elapsed_time(t_end)
    if world > 1:
        tmax = torch.tensor([ms], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms = float(tmax.item())
        pipe.advance(world - 1)  # drain so that every rank leaves with matching send/recv counts
    tokens = K * M * B
    value = tokens / (ms * 1e-3)
    timed_launches = launches[0] + ((peer_hop.launches - hop_launches0) if peer_hop is not None else 0)

    result = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": Wm,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": dict(config_dict(args, world), hop=hop_name), "gpu_launches": timed_launches,
        "clocks": clocks.summary(),
    }

    # ---- roofline of the dominant kernel: every attention launch bracketed by events --
    if rank == 0:
        m, s = 0, total_steps - 1
        sd = descs[(m, s)]
        x = q0[0]
        evs = []

        def on_attention(i):
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            evs.append(e)

        for _ in range(2):
            evs.clear()
            stage.forward(x, k_new[m], v_new[m], sd, on_attention)
        torch.cuda.synchronize()
        per_launch_ms = float(np.mean([evs[2 * i].elapsed_time(evs[2 * i + 1]) for i in range(L)]))
        n_pages = int(sd.kv_page_indices.numel())
        alg = algorithmic_bytes_per_layer(sd.kv_tokens, n_pages, args)
        peak, peak_src = 6520.5, "MEASURED_PEAKS.json hbm_gbs (burst copy)"
        try:
            peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
        except Exception:
            peak, peak_src = 6650.0, "fallback"
        achieved = alg / (per_launch_ms * 1e-3) / 1e9
        # DRAM bytes per algorithmic byte of this kernel, from the ncu capture of a small case whose
        # summary is committed under profiles/; every live page is read exactly once, so traffic
        # scales with the algorithmic bytes
        traffic_ratio = 1.024
        result["roofline"] = {"bound": "hbm", "kernel": "decode_tma_kernel + merge_kernel (one dsv_paged_decode call)",
                              "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                              "frac_of_8000": achieved / 8000.0, "traffic": alg * traffic_ratio,
                              "traffic_note": "ncu dram bytes of a 615 MB launch scaled by algorithmic bytes", "peak_source": peak_src,
                              "algorithmic_bytes_per_launch": alg, "ms_per_launch": per_launch_ms}

    # ---- end to end through the public API with host buffers (N = 1) -------------------
    if world == 1 and not args.no_e2e:
        tasks, caches = mbs[0]
        e2e_steps = K
        # new K/V rows of every layer in pinned host memory: [layer, K|V, sequence, kv head, head_dim]
        hkv_host = torch.randn(L, 2, B, hkv, d).mul_(0.5).to(torch.bfloat16).pin_memory()
        dkv = torch.empty(L, 2, B, hkv, d, dtype=torch.bfloat16, device=dev)
        copy_stream = torch.cuda.Stream(device=dev)
        layer_ready = [torch.cuda.Event() for _ in range(L)]
        small_inputs_done = torch.cuda.Event()
        hq_host = torch.randn(B, hq, d).to(torch.bfloat16).pin_memory()
        hout = torch.empty(B, hq, d, dtype=torch.bfloat16).pin_memory()
        ws = torch.empty(128 << 20, dtype=torch.uint8, device=dev)
        wrapper = dk.BatchDecodeWithPagedKVCacheWrapper(ws)

        desc_bytes = [0]

        def e2e_step():
            # The step's small inputs (q, descriptors, plan) go first on the compute stream; the new K/V
            # rows of all layers follow on a copy stream, layer by layer, while earlier layers compute. The
            # copy stream starts behind the small inputs (else the copy engine may serve the 33 MB first and
            # layer 0 waits for all of it) and thereby behind the previous step; the compute stream waits
            # for each layer's event.
            main = torch.cuda.current_stream()
            x = hq_host.to(dev, non_blocking=True)
            ctx = dk.FlashDecodeCtx.init_paged_decode_ctx(tasks, caches, wrapper)
            wrapper.begin_forward(ctx.kv_page_indptr, ctx.kv_page_indices, ctx.kv_last_page_lens, hq, hkv, d, ps,
                                  data_type=torch.bfloat16, indptr_host=ctx.host["kv_page_indptr"])
            small_inputs_done.record(main)
            copy_stream.wait_event(small_inputs_done)  # which also orders it behind the previous step
            with torch.cuda.stream(copy_stream):
                for layer in range(L):
                    dkv[layer].copy_(hkv_host[layer], non_blocking=True)
                    layer_ready[layer].record(copy_stream)
            for layer in range(L):
                pages = pool.get_layered_pages(layer)
                main.wait_event(layer_ready[layer])
                dk.append_paged_kv_cache(dkv[layer, 0], dkv[layer, 1], ctx.indptr, pages, ctx.kv_page_indices,
                                         ctx.kv_page_indptr, ctx.kv_last_page_lens)
                x = wrapper.forward(x, pages)
            wrapper.end_forward()
            desc_bytes[0] = 4 * (sum(len(a) for a in ctx.host.values()) + int(wrapper._plan_host[6]) + 2 * B)
            hout.copy_(x, non_blocking=True)
            for t in tasks:
                t.step()

        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        e_ms = e0.elapsed_time(e1)
        result["e2e"] = {"value": e2e_steps * B / (e_ms * 1e-3), "unit": "tok/s",
                         "h2d_bytes_per_step": int(hkv_host.numel() * 2 + hq_host.numel() * 2 + desc_bytes[0]),
                         "d2h_bytes_per_step": int(hout.numel() * 2), "ms_per_step": e_ms / e2e_steps,
                         "api": "FlashDecodeCtx.init_paged_decode_ctx + BatchDecodeWithPagedKVCacheWrapper + "
                                "append_paged_kv_cache, pinned host K/V/q in (K/V per layer on a copy stream), pinned host out"}
    if world == 1 and not args.no_prefill:
        result["prefill"] = prefill_measure(dk, args, dev)
    if do_swap:
        result["swap"] = swap_stress(dk, pool, perm[at:], args, dev, lambda: stage.forward(
            q0[0], k_new[0], v_new[0], descs[(0, total_steps - 1)]))
    status = _lib.read_device_status()
    if status != 0:
        raise SystemExit(f"device self-check fired: status {status}")
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"], _ = cpu_reference_arm(args, 15, 1)  # ~10 s of host work
        print(json.dumps(result), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
