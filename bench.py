#!/usr/bin/env python
"""Benchmark of the paged KV-cache hot path on 1 / 2 / 4 / 8 B200.

Headline (`value`): decode tokens/s of the Llama-3-70B-shaped pipeline —
80 layers split evenly over the N GPUs (pipeline stages), 64 q / 8 kv heads,
head_dim 128, hidden 8192, FFN 28672, bf16, random-init weights; 8 microbatches
x 128 sequences, each with a 512-token prompt of random ids (vocab 128256),
greedy decoding; every stage owns the KV pages of its layers and runs the
reference's per-step order (page allocation, descriptors, rotary + append,
paged attention, region swap) on them; activations hop between stages over
NCCL links; the output head is split between the last and the first stage. A
step = one decode token for all 8 x 128 sequences. The same job
runs at every N (strong scaling); `token_sha256` of the generated tokens must be
the same at every N. On one GPU the 141 GB of weights leave room for one
microbatch's KV, so the microbatches run one after the other and nothing is
swapped; from 2 GPUs on several microbatches are in flight and the region swap is
on (see `pipeline` in the line).

`kv_step` in the same line: the Llama-3-8B-shaped KV-only decode step (32
layers, 32 q / 8 kv heads, 256 sequences with contexts U[512, 4096] on a seeded
random permutation of a 1.25x pool; per layer append one token + paged decode
attention) that the `roofline` of the decode-attention kernel is measured on; on
N > 1 GPUs its layers are split over the stages and N microbatches rotate (weak
scaling of the pure KV path). On one GPU the line also carries the chunked-
prefill kernel (`prefill_kernel`), the KV swap stress (`swap`), the same
pipeline through host token buffers (`e2e`), the library the reference calls
on the same tensors (`library`) and the CPU restatement of the reference timed
on the host cores (`cpu_baseline`).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line on rank 0. Synthetic data throughout.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = "llama3-70b-pipeline"
KV_WORKLOAD = "llama3-8b-decode-kv"
METRIC = "decode_tokens_per_s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--parts", default="kv,pipe",
                    help="comma list: kv = the 8B KV-only step (roofline, swap, prefill kernel), pipe = the 70B pipeline")
    # the pipeline job; the defaults are the benchmark
    ap.add_argument("--pipe-layers", type=int, default=80)
    ap.add_argument("--pipe-microbatches", type=int, default=8)
    ap.add_argument("--pipe-seqs", type=int, default=128)
    ap.add_argument("--pipe-prompt", type=int, default=512)
    ap.add_argument("--pipe-prefill-seqs", type=int, default=8, help="prompts per prefill step")
    ap.add_argument("--pipe-sized-for", type=int, default=256,
                    help="generated tokens per sequence the pools are sized for (the configuration's 256)")
    ap.add_argument("--pipe-kv-budget-gb", type=float, default=0.0,
                    help="HBM for a stage's KV pool; 0 = what is free after the weights minus a reserve")
    ap.add_argument("--pipe-swap", default="auto", choices=["auto", "off", "zero"],
                    help="auto = region swap on when two or more microbatches are in flight; off = no swap regions; "
                         "zero = regions exist and rotate but the main pages hold everything, so nothing live travels "
                         "(isolates the cost of the swap calls from the cost of the bytes)")
    # shape overrides of the KV step for small profiling captures; the defaults are the benchmark
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx-lo", type=int, default=512)
    ap.add_argument("--ctx-hi", type=int, default=4096)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end passes")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the chunked-prefill attention measurement")
    ap.add_argument("--prefill-only", action="store_true", help="run only the chunked-prefill measurement (profiling)")
    ap.add_argument("--prefill-reqs", type=int, default=32)
    ap.add_argument("--prefill-ctx", type=int, default=4096)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--no-swap", action="store_true", help="skip the KV swap stress (16 GiB of scattered pages out and back)")
    ap.add_argument("--swap-seqs", type=int, default=64)
    ap.add_argument("--swap-tokens", type=int, default=2048)
    ap.add_argument("--swap-repeats", type=int, default=3)
    ap.add_argument("--hop", default="auto", choices=["auto", "peer", "nccl"],
                    help="KV step on N > 1: how a stage hands its activations on. peer = the stage's last attention "
                         "kernel stores its output straight into the next GPU's inbox over NVLink and a flag follows "
                         "(deserve_b200.peer); nccl = isend/irecv on one communicator per link; auto = peer, and "
                         "nccl if peer memory cannot be set up")
    ap.add_argument("--measure-hop", action="store_true",
                    help="N > 1 only: time one 2 MiB hop around the ring, NCCL send/recv against the peer-memory "
                         "transport, with nothing else on the GPUs; prints its own JSON line")
    ap.add_argument("--compare-library", action="store_true",
                    help="only time flashinfer (the library the reference calls) and this package on the same "
                         "one-layer decode and chunked-prefill inputs; prints its own JSON line")
    ap.add_argument("--no-library", action="store_true",
                    help="N = 1: do not run the flashinfer comparator (a child process, at most 240 s) for the `library` field")
    ap.add_argument("--frag-policy", default="prefill_first", choices=["vanilla", "prefill_first", "decode_first"],
                    help="join policy of the first stage's scheduler in the --fragmentation run")
    ap.add_argument("--fragmentation", action="store_true",
                    help="only run the mixed prefill/decode fragmentation workload (512 arrivals, lognormal prompts, "
                         "512-token chunks, 128 decode steps, seeded departures); prints its own JSON line")
    return ap.parse_args()


def make_lengths(args, seed=0):
    rng = np.random.default_rng(seed)
    return rng.integers(args.ctx_lo, args.ctx_hi + 1, size=args.batch)


def algorithmic_bytes_per_layer(kv_tokens, n_pages, args, es=2, batch=None):
    """decode attention: every live K/V element once, q in and out once, the
    page list and the three per-request descriptor arrays once."""
    B = args.batch if batch is None else batch
    return (kv_tokens * 2 * args.kv_heads * args.head_dim * es + 2 * B * args.q_heads * args.head_dim * es
            + 4 * (n_pages + 2 * (B + 1)))


def measured_peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16 burst)"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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
        self._stop.clear()
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
# configuration record (identical in both arms)
# ---------------------------------------------------------------------------
def config_dict(args, n):
    return {"workload": WORKLOAD, "layers": args.pipe_layers, "stages": n, "q_heads": 64, "kv_heads": 8,
            "head_dim": 128, "hidden": 8192, "ffn": 28672, "vocab": 128256, "page_size": 16,
            "microbatches": args.pipe_microbatches, "sequences_per_microbatch": args.pipe_seqs,
            "prompt_tokens": args.pipe_prompt, "decode_steps_timed": args.steps, "decode_steps_warmup": args.warmup,
            "pools_sized_for_new_tokens": args.pipe_sized_for, "parallelism": f"pp{n}" if n > 1 else "single",
            "l2": "inputs larger than L2 (a stage reads its weights and KV, >= 17 GB, per microbatch step)",
            "kv_step": {"workload": KV_WORKLOAD, "layers": args.layers, "q_heads": args.q_heads,
                        "kv_heads": args.kv_heads, "head_dim": args.head_dim, "page_size": args.page_size,
                        "sequences_per_microbatch": args.batch, "context": f"U[{args.ctx_lo},{args.ctx_hi}]",
                        "pool": "1.25x pages, seeded permutation"}}


# ---------------------------------------------------------------------------
# CPU arms (cpu_baseline of our line, and the whole --impl reference run)
# ---------------------------------------------------------------------------
def cpu_kv_layer_sample(args, steps, warmup, n_seq=None):
    """The reference's torch path restated on the host (oracle/): one layer of the KV step on all
    sequences of the microbatch per sample — append one token by index assignment, gather K/V
    through the page table, dense fp32 attention. tok/s is scaled to the full step."""
    from oracle import kv_math

    torch.set_num_threads(os.cpu_count())
    n_seq = args.batch if n_seq is None else min(n_seq, args.batch)
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
    return {"value": n_seq / (dt * args.layers), "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"1 of {args.layers} layers x {n_seq} of {args.batch} sequences per step "
                      f"({dt * 1e3:.1f} ms/sample, CPU torch, scaled to the full step)"}


def cpu_config1_full():
    """The small CPU configuration in full on the host: 2 layers, 8 q / 2 kv heads, head_dim 64, fp32, page
    size 16, 4 sequences with contexts U[100,300] from seed 0, 32 decode steps (allocator, descriptors,
    append, paged attention), all through the oracle."""
    from oracle import kv_math
    from oracle.descriptors import OracleTask, build_descriptors
    from oracle.paged_alloc import OracleKVCache, OraclePagePool, OraclePageTables

    L, hq, hkv, d, ps, B, steps = 2, 8, 2, 64, 16, 4, 32
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(100, 301, (B,), generator=g).tolist()
    pool, tab = OraclePagePool(256, ps), OraclePageTables(B, 4096, ps)
    pages = torch.zeros(L, 256, 2, ps, hkv, d)
    tasks = [OracleTask(initial_seqlen=n) for n in lens]
    caches = [OracleKVCache(tab, pool) for _ in lens]
    for t, c in zip(tasks, caches):
        c.extend(t.initial_seqlen)
        t.start_pos, t.seqlen = t.initial_seqlen, 1
    t0 = time.perf_counter()
    for _ in range(steps):
        desc = build_descriptors(tasks, caches, ps)
        for layer in range(L):
            k, v = torch.randn(B, hkv, d, generator=g), torch.randn(B, hkv, d, generator=g)
            q = torch.randn(B, hq, d, generator=g)
            kv_math.append_paged(pages[layer], k, v, desc, ps)
            kv_math.paged_attention(q, pages[layer], desc, ps, causal=False)
        for t in tasks:
            t.start_pos += 1
    dt = time.perf_counter() - t0
    return {"value": B * steps / dt, "unit": "tok/s", "seconds": dt, "steps": steps, "sequences": B}


def cpu_pipeline_layer_sample(args, steps, warmup):
    """One decode step of one microbatch of the 70B-shaped model on the host, restated from the
    reference's torch statements (oracle/): ONE transformer layer per sample — RMSNorm, fused q|k|v
    projection, rotary embedding, append into pages, paged attention through the page table, output
    projection, SwiGLU feed-forward, bf16 weights — plus the final norm + output projection + argmax
    once; a step is layers x the layer time + the head time."""
    from oracle import kv_math

    torch.set_num_threads(os.cpu_count())
    S, D, hq, hkv, hd, F, V, ps = args.pipe_seqs, 8192, 64, 8, 128, 28672, 128256, 16
    ctx = args.pipe_prompt + args.warmup + 1
    g = torch.Generator().manual_seed(5)
    w = lambda r, c: (torch.randn(r, c, generator=g) * 0.02).to(torch.bfloat16)
    wqkv, wo, w13, w2, wout = w((hq + 2 * hkv) * hd, D), w(D, hq * hd), w(2 * F, D), w(D, F), w(V, D)
    ones = torch.ones(D, dtype=torch.bfloat16)
    n_pg = (ctx + ps - 1) // ps
    total = S * n_pg
    desc = {"indptr": np.arange(S + 1, dtype=np.int32),
            "kv_page_indices": np.random.default_rng(1).permutation(total + total // 4)[:total].astype(np.int32),
            "kv_page_indptr": (np.arange(S + 1) * n_pg).astype(np.int32),
            "kv_last_page_lens": np.full(S, (ctx - 1) % ps + 1, dtype=np.int32),
            "offsets": np.full(S, ctx - 1, dtype=np.int32)}
    pages = (torch.randn(total + total // 4, 2, ps, hkv, hd, generator=g) * 0.5).to(torch.bfloat16)
    x = torch.randn(S, D, generator=g).to(torch.bfloat16)
    pos = torch.full((S,), ctx - 1, dtype=torch.int64)

    def layer(x):
        qkv = kv_math.rmsnorm(x, ones, 1e-5) @ wqkv.t()
        q = kv_math.apply_rope(qkv[:, : hq * hd].reshape(S, hq, hd), pos, 500000.0)
        k = kv_math.apply_rope(qkv[:, hq * hd : (hq + hkv) * hd].reshape(S, hkv, hd), pos, 500000.0)
        v = qkv[:, (hq + hkv) * hd :].reshape(S, hkv, hd)
        kv_math.append_paged(pages, k, v, desc, ps)
        attn = kv_math.paged_attention(q, pages, desc, ps, causal=False).to(torch.bfloat16)
        h = x + attn.reshape(S, hq * hd) @ wo.t()
        gu = kv_math.rmsnorm(h, ones, 1e-5) @ w13.t()
        return h + (torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]) @ w2.t()

    def head(x):
        return kv_math.greedy_tokens(kv_math.rmsnorm(x, ones, 1e-5) @ wout.t())

    for _ in range(warmup):
        layer(x)
    head(x)
    t0 = time.perf_counter()
    for _ in range(steps):
        layer(x)
    t_layer = (time.perf_counter() - t0) / steps
    t0 = time.perf_counter()
    head(x)
    t_head = time.perf_counter() - t0
    step_s = args.pipe_layers * t_layer + t_head
    info = {"value": S / step_s, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"1 of {args.pipe_layers} layers of one {S}-sequence microbatch at context {ctx} per step "
                      f"({t_layer * 1e3:.1f} ms/layer) + the output head once ({t_head * 1e3:.0f} ms), CPU torch bf16 "
                      f"weights, scaled to the {args.pipe_layers}-layer step"}
    return info, step_s


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    info, step_s = cpu_pipeline_layer_sample(args, max(1, args.steps), max(1, args.warmup))
    line = {"impl": "reference", "metric": METRIC, "value": info["value"], "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * args.pipe_microbatches * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(args, args.gpus), "cpu_baseline": info,
            "e2e": {"value": info["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# KV step (8B shape): helpers
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


def prefill_case(dk, args, dev, lens, new, label, iters=5):
    """Ragged causal attention of `new[i]` new rows per request against paged K/V holding lens[i]
    tokens (after the append), one layer, on the tcgen05 kernel. Dense-equivalent TFLOP/s
    (4 * Hq * D * visible (q, kv) pairs) against the measured bf16 GEMM peak."""
    from deserve_b200 import ops

    ps, hq, hkv, d = args.page_size, args.q_heads, args.kv_heads, args.head_dim
    lens, new = np.asarray(lens, dtype=np.int64), np.asarray(new, dtype=np.int64)
    B = len(lens)
    n_pages = (lens + ps - 1) // ps
    total = int(n_pages.sum())
    pool_pages = int(total * 1.25) + 1
    g = torch.Generator(device=dev).manual_seed(7)
    pages = torch.empty(pool_pages, 2, ps, hkv, d, dtype=torch.bfloat16, device=dev).normal_(0, 0.5, generator=g)
    nnz = int(new.sum())
    q = torch.randn(nnz, hq, d, device=dev, generator=g).to(torch.bfloat16)
    qo = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    kvp = np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32)
    idx = np.random.default_rng(3).permutation(pool_pages)[:total].astype(np.int32)
    last = ((lens - 1) % ps + 1).astype(np.int32)
    plan = np.zeros(ops.prefill_plan_capacity(nnz, B, hq // hkv), dtype=np.int32)
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
    # q row j (of n) of a request with len tokens sees len - n + j + 1 positions
    pairs = float(sum(int(n) * (int(l) - int(n)) + int(n) * (int(n) + 1) // 2 for l, n in zip(lens, new)))
    flops = 4.0 * hq * d * pairs
    pk = measured_peaks()
    tf = flops / (ms * 1e-3) / 1e12
    return {"workload": label, "ms": ms, "tflops": tf, "peak_tflops": pk["bf16_tflops"], "frac": tf / pk["bf16_tflops"],
            "frac_of_sustained": tf / pk["bf16_tflops_sustained"], "new_tokens": nnz, "requests": B,
            "prefill_tokens_per_s_per_layer": nnz / (ms * 1e-3), "bound": "tensor"}


def prefill_measure(dk, args, dev):
    """Two shapes: the uniform one (prefill_reqs requests that hold prefill_ctx tokens each get a
    prefill_chunk-token chunk) and one chunked-prefill step of the mixed prefill/decode configuration
    (prompt lengths ~ LogNormal(6.5, 0.8) clipped to [16, 8192], every request at a seeded random
    chunk of its prompt, chunks of at most 512 tokens, 64 requests in the step)."""
    B, ctx, n = args.prefill_reqs, args.prefill_ctx, args.prefill_chunk
    uniform = prefill_case(dk, args, dev, np.full(B, ctx + n), np.full(B, n),
                           f"{B} requests x ({ctx} context + {n}-token chunk), causal, 1 layer")
    rng = np.random.default_rng(5)
    prompts = np.clip(rng.lognormal(6.5, 0.8, size=64), 16, 8192).astype(np.int64)
    n_chunks = (prompts + 511) // 512
    which = (rng.random(64) * n_chunks).astype(np.int64)           # the chunk each request is at
    done = which * 512
    new = np.minimum(512, prompts - done)
    ragged = prefill_case(dk, args, dev, done + new, new,
                          "64 requests, prompts ~ LogNormal(6.5, 0.8) in [16, 8192], each at a random 512-token chunk, "
                          "causal, 1 layer")
    uniform["ragged"] = ragged
    return uniform


def library_compare(dk, args, dev, iters=20):
    """flashinfer's paged decode / prefill wrappers (what the reference calls) and this package's on the
    same tensors: one layer of the KV step's decode shape and the chunked-prefill case. Plans are made
    outside the timed loops on both sides; K/V read per decode launch is far larger than L2."""
    import flashinfer as fi
    from deserve_b200 import ops  # noqa: F401

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
    t0 = time.perf_counter()
    w = fi.BatchDecodeWithPagedKVCacheWrapper(ws_fi, "NHD")
    w.plan(t["kvp"], t["idx"], t["last"], hq, hkv, d, ps, pos_encoding_mode="NONE", q_data_type=torch.bfloat16,
           kv_data_type=torch.bfloat16)
    ref = w.run(q, pages)
    torch.cuda.synchronize()
    out["flashinfer_first_decode_call_s"] = time.perf_counter() - t0  # includes its JIT build on a fresh machine
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


def library_in_child(limit_s=240):
    """The flashinfer comparator (`--compare-library`) in a child process with a time limit: flashinfer
    builds or loads its kernels on first use, which on a machine without its cache can take minutes; the
    benchmark line then says so instead of waiting. The parent's device memory has been released by then."""
    import subprocess

    t0 = time.perf_counter()
    try:
        out = subprocess.run([sys.executable, os.path.abspath(__file__), "--compare-library"], capture_output=True,
                             text=True, timeout=limit_s)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"flashinfer did not finish building its kernels within {limit_s} s"}
    for ln in reversed(out.stdout.strip().splitlines()):
        if ln.startswith("{"):
            try:
                res = json.loads(ln)["library_comparator"]
                res["wall_s"] = time.perf_counter() - t0
                res["note"] = ("the library the reference calls (its paged decode / prefill wrappers), same tensors, "
                               "plans outside the timed loops on both sides")
                return res
            except Exception:
                break
    return {"unavailable": f"comparator exited with code {out.returncode}: {out.stderr.strip()[-200:]}"}


def measure_hop(args, rank, world, dev, dist, iters=200):
    """Every rank sends [batch, q_heads, head_dim] bf16 to its successor and receives from its predecessor,
    `iters` times back to back, once with NCCL isend/irecv on per-link communicators and once through
    deserve_b200.peer.PeerHop (push kernel + flag). Device time per hop, max over ranks."""
    from deserve_b200.engine import make_ring_links
    from deserve_b200.peer import PeerHop

    shape = (args.batch, args.q_heads, args.head_dim)
    y = torch.randn(shape, device=dev).to(torch.bfloat16)
    buf = torch.empty_like(y)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    send_g, recv_g = make_ring_links(dist, rank, world, dev)

    def nccl_hop():
        r = dist.irecv(buf, prv, group=recv_g)
        s = dist.isend(y, nxt, group=send_g)
        r.wait()
        s.wait()

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
    hop.close()  # raises if a wait of the peer transport gave up: its figure would be meaningless
    out["bytes"] = y.numel() * 2
    out["n_gpus"] = world
    return out


def swap_stress(dk, pool, free_ids, args, dev, decode_step, repeats):
    """KV swap stress: the KV of swap_seqs x swap_tokens tokens, all layers, scattered over the
    permuted pool, is swapped out to pinned host chunks and back into DIFFERENT pages while decode
    attention of another microbatch runs on the main stream; `repeats` rounds, each round's pages
    being the previous round's reloaded ones. Bit-exactness is checked every round with a 32-bit
    checksum of every (layer, page) before and after, and exactly on the first and last layer."""
    ps, L = pool.page_size, pool.num_layers
    n_seq, n_pg = args.swap_seqs, (args.swap_tokens + ps - 1) // ps
    total = n_seq * n_pg
    free_ids = free_ids[pool.page_bitmap.numpy()[free_ids]]  # pages the decode microbatch grew into since are not free
    first_ids = np.ascontiguousarray(free_ids[:total]).astype(np.int32)
    height = int(np.ceil(np.log2(max(total, 2)))) + 1
    peak = host_link_peak(dev)
    chunks = dk.CpuChunkPool(L, height, ps, pool.main_dtype, n_kv_heads=pool.n_kv_heads, head_dim=pool.head_dim)
    pta = dk.PageTableAllocator(n_seq, n_pg * ps, ps, dev)
    mgr = dk.KVCacheManager(pool, chunks, pta, staging_bytes=4 * total * pool.page_bytes + 1024)
    caches = []
    for i in range(n_seq):
        kv = dk.VirtualPagedKVCache.empty(pta, pool)
        kv.page_table.extend(first_ids[i * n_pg : (i + 1) * n_pg])
        caches.append(kv)
    pool.reserve(first_ids)

    def checksums(ids):
        return torch.stack([pool.pages[l, ids].view(torch.int32).sum(dim=(1, 2, 3, 4), dtype=torch.int64)
                            for l in range(L)])

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

    outs, ins, ok, moved = [], [], True, 0
    for _ in range(max(1, repeats)):
        ids_a = torch.from_numpy(np.concatenate([c.page_table.retrieve_np() for c in caches]).astype(np.int64)).to(dev)
        before = checksums(ids_a)
        first, last = pool.pages[0, ids_a].clone(), pool.pages[L - 1, ids_a].clone()
        handles, out_gbs = timed(lambda: mgr.offload_many(caches))
        old_lists = [c.page_table.retrieve_np().copy() for c in caches]
        # hold the old pages while the tasks come back, so that every page changes its id, then let them go
        for kv in caches:
            kv.page_table.free()
        pool.pages[:, ids_a] = 0  # the old pages are gone
        caches, in_gbs = timed(lambda: mgr.reload_many(handles))
        for ids in old_lists:
            pool.free(ids)
        ids_b = torch.from_numpy(np.concatenate([c.page_table.retrieve_np() for c in caches]).astype(np.int64)).to(dev)
        moved = int((ids_a != ids_b).sum().item())
        ok = ok and bool(torch.equal(before, checksums(ids_b)) and torch.equal(first, pool.pages[0, ids_b])
                         and torch.equal(last, pool.pages[L - 1, ids_b]))
        for h in handles:
            h.free()
        outs.append(out_gbs)
        ins.append(in_gbs)
    med = lambda v: float(np.median(v))
    return {"bytes_each_way": nbytes, "repeats": len(outs), "out_GBps": med(outs), "in_GBps": med(ins),
            "out_GBps_min": min(outs), "in_GBps_min": min(ins), "out_GBps_all": outs, "in_GBps_all": ins,
            "host_link_peak_d2h_GBps": peak["d2h"], "host_link_peak_h2d_GBps": peak["h2d"],
            "frac_out": med(outs) / peak["d2h"], "frac_in": med(ins) / peak["h2d"],
            "frac_out_min": min(outs) / peak["d2h"], "frac_in_min": min(ins) / peak["h2d"],
            "bit_exact": ok, "pages_that_changed_id": moved, "pages": total, "layers": L,
            "concurrent": f"{steps} decode steps of the 256-sequence microbatch on another stream"}


# ---------------------------------------------------------------------------
# part 1: the 8B KV-only decode step
# ---------------------------------------------------------------------------
def kv_step_bench(args, dk, rank, world, local, dev, dist):
    from deserve_b200 import _lib
    from deserve_b200.engine import KVStage, RingPipeline, prepare_decode_step

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
    # K/V ~ 0.5 * N(0,1). Page contents and new rows are seeded by (microbatch, GLOBAL layer) and laid down in the
    # order of the microbatch's page list, so microbatch m is the same job whatever the stage count and wherever
    # the permutation put its pages: its final activations can be compared across N.
    mbs = []
    at = 0
    n_now = int(((lens0 + ps - 1) // ps).sum())
    gen = torch.Generator(device=dev)
    k_new = torch.empty(M, L, B, hkv, d, dtype=torch.bfloat16, device=dev)
    v_new = torch.empty(M, L, B, hkv, d, dtype=torch.bfloat16, device=dev)
    for layer in range(L):  # pages nobody owns still hold finite values
        pool.pages[layer].normal_(0.0, 0.5, generator=gen.manual_seed(7))
    for m in range(M):
        ids = perm[at : at + n_now]
        tasks, caches = build_microbatch(dk, pool, pta, lens0, ids, f"mb{m}")
        ids_dev = torch.from_numpy(ids.astype(np.int64)).to(dev)
        for layer in range(L):
            gen.manual_seed(100000 + 1000 * m + rank * L + layer)
            pool.pages[layer].index_copy_(0, ids_dev, torch.empty(
                n_now, 2, ps, hkv, d, dtype=torch.bfloat16, device=dev).normal_(0.0, 0.5, generator=gen))
            k_new[m, layer].normal_(0.0, 0.5, generator=gen)
            v_new[m, layer].normal_(0.0, 0.5, generator=gen)
        at += n_now
        mbs.append((tasks, caches))
    pool.reserve(perm[:at])
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

    mb0_final = {}

    def stage_fn(u, m, s, x, out=None):
        y = stage.forward(x, k_new[m], v_new[m], descs[(m, s)], out=out)
        if rank == world - 1 and m == 0 and s == total_steps - 1:
            mb0_final["y"] = y.clone()  # the job's output for microbatch 0 at the last timed token step
        return y

    peer_hop, hop_name = None, "none"
    if world > 1:
        hop_name = "nccl isend/irecv, one communicator per link"
        if args.hop in ("auto", "peer"):
            ok = torch.ones(1, device=dev)
            try:
                from deserve_b200.peer import PeerHop
                peer_hop = PeerHop(rank, world, (B, hq, d), torch.bfloat16, dev, dist.group.WORLD, depth=3)
            except Exception as exc:  # no peer mapping on this node: every rank must take the same path
                if args.hop == "peer":
                    raise
                print(f"[bench] rank {rank}: peer memory hop unavailable ({exc!r})", file=sys.stderr, flush=True)
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                peer_hop = None
            else:
                hop_name = "peer memory: the last attention kernel stores into the next GPU's inbox, then a flag"
    pipe = RingPipeline(rank, world, stage_fn, lambda m: q0[m], total_steps, dist=dist, peer_hop=peer_hop,
                        direct=peer_hop is not None)

    def barrier():
        if world > 1:
            dist.barrier()

    # ---- warm-up (also fills the ring), then the timed K steps -----------------------
    pipe.advance(Wm * M)
    torch.cuda.synchronize()
    barrier()
    _lib.LAUNCHES[0] = 0
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
    timed_launches = _lib.LAUNCHES[0] + ((peer_hop.launches - hop_launches0) if peer_hop is not None else 0)
    # microbatch 0's activations after its last timed step, as it leaves this stage: the same number at every N
    # for the stage that owns the same last layer (rank world-1 holds the job's final output)
    if world > 1:
        tmax = torch.tensor([ms], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms = float(tmax.item())
        pipe.advance(world - 1)  # drain so that every rank leaves with matching send/recv counts
        pipe.flush()
    checksum = None
    if "y" in mb0_final:
        checksum = int(mb0_final["y"].contiguous().view(torch.int16).to(torch.int64).sum().item())
    if world > 1:  # the last rank holds the job's output
        c = torch.tensor([checksum if checksum is not None else 0], dtype=torch.int64, device=dev)
        dist.all_reduce(c, op=dist.ReduceOp.SUM)
        checksum = int(c.item())
    if peer_hop is not None:
        peer_hop.close()  # raises if a bounded wait gave up
    tokens = K * M * B
    res = {"workload": KV_WORKLOAD, "value": tokens / (ms * 1e-3), "unit": "tok/s", "scaling": "weak",
           "microbatches": M, "ms_per_step": ms / K, "hop": hop_name, "gpu_launches": timed_launches,
           "clocks": clocks.summary(), "mb0_checksum": checksum}
    roof = None

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

        with ClockSampler(local) as rclocks:
            for _ in range(6):
                evs.clear()
                stage.forward(x, k_new[m], v_new[m], sd, on_attention)
            torch.cuda.synchronize()
        per_launch_ms = float(np.mean([evs[2 * i].elapsed_time(evs[2 * i + 1]) for i in range(L)]))
        n_pages = int(sd.kv_page_indices.numel())
        alg = algorithmic_bytes_per_layer(sd.kv_tokens, n_pages, args)
        pk = measured_peaks()
        achieved = alg / (per_launch_ms * 1e-3) / 1e9
        mhz = rclocks.summary()["sm_mhz"]
        # DRAM bytes per algorithmic byte of this kernel, from the ncu capture of a small case whose
        # summary is committed under profiles/; every live page is read exactly once, so traffic
        # scales with the algorithmic bytes
        traffic_ratio = 1.024
        roof = {"bound": "hbm", "kernel": "decode_tma_kernel + merge_kernel (one dsv_paged_decode call)",
                "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                "frac_of_8000": achieved / 8000.0, "traffic": alg * traffic_ratio,
                "traffic_note": "ncu dram bytes of a 615 MB launch scaled by algorithmic bytes",
                "peak_source": pk["source"], "algorithmic_bytes_per_launch": alg, "ms_per_launch": per_launch_ms,
                "sm_mhz_median": mhz, "ms_per_launch_x_sm_mhz": per_launch_ms * mhz if mhz else None,
                "workload": KV_WORKLOAD}

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
        from deserve_b200.pinned import COUNTERS

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
            hout.copy_(x, non_blocking=True)
            for t in tasks:
                t.step()

        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        COUNTERS["h2d_bytes"] = 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        e_ms = e0.elapsed_time(e1)
        res["e2e"] = {"value": e2e_steps * B / (e_ms * 1e-3), "unit": "tok/s",
                      "h2d_bytes_per_step": int(hkv_host.numel() * 2 + hq_host.numel() * 2
                                                + COUNTERS["h2d_bytes"] // e2e_steps),
                      "d2h_bytes_per_step": int(hout.numel() * 2), "ms_per_step": e_ms / e2e_steps,
                      "api": "FlashDecodeCtx.init_paged_decode_ctx + BatchDecodeWithPagedKVCacheWrapper + "
                             "append_paged_kv_cache, pinned host K/V/q in (K/V per layer on a copy stream), pinned host out"}
    extras = {}
    if world == 1 and not args.no_prefill:
        extras["prefill_kernel"] = prefill_measure(dk, args, dev)
    if do_swap:
        extras["swap"] = swap_stress(dk, pool, perm[at:], args, dev, lambda: stage.forward(
            q0[0], k_new[0], v_new[0], descs[(0, total_steps - 1)]), args.swap_repeats)
    status = _lib.read_device_status()
    if status != 0:
        raise SystemExit(f"device self-check fired: status {status}")
    return res, roof, extras


# ---------------------------------------------------------------------------
# part 2: the 70B-shaped pipeline
# ---------------------------------------------------------------------------
def pipeline_bench(args, dk, rank, world, local, dev, dist):
    from deserve_b200 import _lib
    from deserve_b200.model import ModelArgs, llama_3_70b_args
    from deserve_b200.pinned import COUNTERS
    from deserve_b200.pipeline_driver import PipelineConfig, make_stage, run_stage, size_pools, token_digest

    model = ModelArgs(**{**llama_3_70b_args.__dict__, "n_layers": args.pipe_layers})
    if model.n_layers % world:
        raise SystemExit("--pipe-layers must be divisible by --gpus")
    lb, le = rank * model.n_layers // world, (rank + 1) * model.n_layers // world
    t0 = time.perf_counter()
    stage = make_stage(model, rank, world, dev)
    torch.cuda.synchronize()
    init_s = time.perf_counter() - t0
    free, total = torch.cuda.mem_get_info(dev)
    # reserve: prefill activations (prefill_seqs prompts through the FFN), logits, workspaces, allocator slack
    reserve = int(6e9)
    budget = int(args.pipe_kv_budget_gb * 1e9) if args.pipe_kv_budget_gb else free - reserve
    if world > 1:
        t = torch.tensor([budget], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        budget = int(t.item())
    new_tokens = 1 + args.warmup + args.steps
    sz = size_pools(model, le - lb, args.pipe_microbatches, args.pipe_seqs, args.pipe_prompt, new_tokens, budget, world,
                    sized_for_tokens=max(args.pipe_sized_for, new_tokens))
    if args.pipe_swap in ("off", "zero") and sz["swap_pages"]:
        sz["main_pages"] += sz["concurrent"] * args.pipe_seqs + 64
        if args.pipe_swap == "off":
            sz["swap_pages"] = 0
    cfg = PipelineConfig(model=model, n_microbatches=args.pipe_microbatches, seqs=args.pipe_seqs,
                         prompt_len=args.pipe_prompt, new_tokens=new_tokens, prefill_seqs=args.pipe_prefill_seqs,
                         main_pages=sz["main_pages"], swap_pages=sz["swap_pages"], concurrent=sz["concurrent"],
                         warmup_tokens=args.warmup)
    from deserve_b200 import trace

    trace.enable_host_timing(True)
    with ClockSampler(local) as clocks:
        res = run_stage(rank, world, cfg, dev, dist if world > 1 else None, stage=stage)
    launches = res["launches_timed"]  # rank 0's kernels of this package inside the timed decode regions
    host_phases = {k: round(v["ms"] / max(v["calls"], 1), 4) for k, v in trace.host_totals().items()}
    trace.enable_host_timing(False)
    tm = torch.tensor([res["prefill_ms"], res["decode_ms"], res["decode_compute_ms"]], device=dev, dtype=torch.float64)
    if world > 1:
        mx = tm.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        prefill_ms, decode_ms = float(mx[0]), float(mx[1])
        comp = [torch.zeros_like(tm) for _ in range(world)]
        dist.all_gather(comp, tm)
        compute_ms = [float(c[2]) for c in comp]
    else:
        prefill_ms, decode_ms, compute_ms = float(tm[0]), float(tm[1]), [float(tm[2])]
    M, S, K = cfg.n_microbatches, cfg.seqs, args.steps
    # the tokens live on rank 0 (the first stage finishes the split output head)
    digest, tsum = None, 0
    if rank == 0:
        digest, tsum = token_digest(res["tokens"]), int(res["tokens"].long().sum())
    slots = K * M
    slot_ms = decode_ms / max(slots, 1)
    # per-stage roofline of a decode slot: the stage's weights once + the KV of its layers once, at HBM speed
    pk = measured_peaks()
    layer_w = 2 * ((model.n_heads + 2 * model.n_kv_heads) * model.head_dim * model.dim + model.dim * model.dim
                   + 3 * model.ffn_dim * model.dim)
    head_w = 2 * model.vocab_size * model.dim
    ctx_mid = args.pipe_prompt + args.warmup + (K + 1) / 2
    kv_layer = S * ctx_mid * 2 * model.n_kv_heads * model.head_dim * 2
    # the output head is split between the last and the first stage (one stage: both halves)
    worst_stage_bytes = (le - lb) * (layer_w + kv_layer) + (head_w if world == 1 else head_w // 2)
    bound_ms = worst_stage_bytes / (pk["hbm_gbs"] * 1e9) * 1e3
    out = {
        "value": M * S * K / (decode_ms * 1e-3) if decode_ms > 0 else 0.0, "ms_per_step": decode_ms / max(K, 1),
        "decode_ms": decode_ms, "prefill_ms": prefill_ms,
        "prefill_tokens_per_s": M * S * args.pipe_prompt / (prefill_ms * 1e-3),
        "token_sha256": digest, "token_checksum": tsum, "gpu_launches": launches, "clocks": clocks.summary(),
        "pipeline": {
            "stages": world, "layers_per_stage": le - lb, "microbatches_in_flight": sz["concurrent"],
            "waves": M // sz["concurrent"], "weights_init_s": init_s,
            "pool": {"main_pages": sz["main_pages"], "pages_per_swap_region": sz["swap_pages"],
                     "bytes": sz["pool_bytes"], "kv_budget_bytes": budget, "hbm_total_bytes": total},
            "swap": ("off: one microbatch in flight has nobody to swap with" if not sz["swap_pages"] else {
                "region_pages": sz["swap_pages"], "live_only": True,
                "mean_pages_out_per_slot": res["swap_pages_out"] / max(res["swap_slots"], 1),
                "mean_pages_in_per_slot": res["swap_pages_in"] / max(res["swap_slots"], 1),
                "max_pages_out_per_slot": res["swap_pages_out_max"],
                "mean_token_rows_out_per_page": res["swap_rows_out"] / max(res["swap_slots"], 1),
                "mean_token_rows_in_per_page": res["swap_rows_in"] / max(res["swap_slots"], 1),
                "rows_note": "of a travelling page (16 token rows of K, 16 of V) only the rows that hold tokens move",
                "dma_out_ms_per_slot": res["swap_dma_out_ms"] / max(res["swap_dma_slots"], 1),
                "dma_in_ms_per_slot": res["swap_dma_in_ms"] / max(res["swap_dma_slots"], 1),
                "dma_note": "time the region copies of one slot run on their side streams (device events); they start "
                            "when the compute stream reaches the slot's first layer and must end before the next "
                            "slot's first kernel, i.e. within slot_ms",
                "bytes_per_page_per_stage": (le - lb) * 2 * 16 * model.n_kv_heads * model.head_dim * 2}),
            "pages_free_min": res["pages_free_min"],
            "slot_ms": slot_ms, "stage_compute_ms_per_slot": [c / max(slots, 1) for c in compute_ms],
            "bubble_frac_per_stage": [1.0 - c / decode_ms if decode_ms > 0 else 0.0 for c in compute_ms],
            "stage_roofline": {"bound": "hbm", "bytes_per_slot_worst_stage": worst_stage_bytes,
                               "bound_ms": bound_ms, "frac": bound_ms / slot_ms if slot_ms > 0 else None,
                               "note": "weights of the stage's layers + its half of the output head (last and first "
                                       "stage; both halves on one GPU) + the KV of its layers, each read once per "
                                       "microbatch step, over the measured copy bandwidth; the projections are cuBLAS "
                                       "GEMMs"},
            "hop": "none" if world == 1 else "nccl isend/irecv, one communicator per directed link; a receive is posted right "
                   "after the slot's send, the compute stream waits for it only where the next slot reads it",
            "host_ms_per_call_rank0": host_phases,
        },
    }
    # ---- the same loop with the tokens going through pinned host memory every step (N = 1) ----
    if world == 1 and not args.no_e2e:
        main_tokens = res.pop("tokens")
        gc.collect()
        torch.cuda.empty_cache()
        sz1 = size_pools(model, le - lb, 1, S, args.pipe_prompt, new_tokens, budget, 1)
        cfg1 = PipelineConfig(model=model, n_microbatches=1, seqs=S, prompt_len=args.pipe_prompt, new_tokens=new_tokens,
                              prefill_seqs=args.pipe_prefill_seqs, main_pages=sz1["main_pages"], swap_pages=0,
                              concurrent=1, warmup_tokens=args.warmup, host_tokens=True)
        COUNTERS["h2d_bytes"] = 0
        r1 = run_stage(0, 1, cfg1, dev, None, stage=stage)
        steps_all = cfg1.steps
        same = bool(torch.equal(r1["tokens"][0], main_tokens[0]))
        out["e2e"] = {"value": S * K / (r1["decode_ms"] * 1e-3), "unit": "tok/s",
                      "h2d_bytes_per_step": int(S * 4 + COUNTERS["h2d_bytes"] // max(steps_all, 1)),
                      "d2h_bytes_per_step": int(S * 4), "ms_per_microbatch_step": r1["decode_ms"] / max(K, 1),
                      "tokens_equal_device_loop": same,
                      "api": "StageProcessor.process_step per microbatch step: token ids come from pinned host memory, "
                             "the step's tokens go back to pinned host memory and the host waits for them before the "
                             "next step (one microbatch; on one GPU the microbatches run one after the other, so its "
                             "rate is the job's)"}
    # ---- N > 1: the same job with the serving loop's host round trip on the first stage -----------
    if world > 1 and not args.no_e2e:
        main_tokens = res.pop("tokens", None)
        res.pop("stage", None)
        gc.collect()
        torch.cuda.empty_cache()
        import dataclasses

        cfg_e = dataclasses.replace(cfg, host_tokens=True)
        COUNTERS["h2d_bytes"] = 0
        r1 = run_stage(rank, world, cfg_e, dev, dist, stage=stage)
        t1 = torch.tensor([r1["decode_ms"]], device=dev, dtype=torch.float64)
        dist.all_reduce(t1, op=dist.ReduceOp.MAX)
        e2e_ms = float(t1[0])
        if rank == 0:
            slots_all = max(cfg.steps * M, 1)
            out["e2e"] = {"value": M * S * K / (e2e_ms * 1e-3), "unit": "tok/s",
                          "h2d_bytes_per_step": int(M * (S * 4 + COUNTERS["h2d_bytes"] // slots_all)),
                          "d2h_bytes_per_step": int(M * S * 4), "ms_per_step": e2e_ms / max(K, 1),
                          "tokens_equal_device_loop": bool(torch.equal(r1["tokens"], main_tokens)),
                          "api": "StageProcessor.process_step per microbatch slot on every stage: on the first stage the "
                                 "step's tokens (finished from the last stage's message) go to pinned host memory, the "
                                 "host waits for them, and the next step's token ids come from there; bytes are the "
                                 "first stage's, per decode step of all microbatches"}
    status = _lib.read_device_status()
    if status != 0:
        raise SystemExit(f"device self-check fired: status {status}")
    return out


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist

    import deserve_b200 as dk

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.compare_library:
        torch.cuda.set_device(local)
        print(json.dumps({"library_comparator": library_compare(dk, args, torch.device("cuda", local))}), flush=True)
        return
    if args.prefill_only:
        torch.cuda.set_device(local)
        print(json.dumps({"prefill_kernel": prefill_measure(dk, args, torch.device("cuda", local))}), flush=True)
        return
    if args.fragmentation:
        from deserve_b200.fragmentation import run_fragmentation

        torch.cuda.set_device(local)
        print(json.dumps({"fragmentation": run_fragmentation(torch.device("cuda", local), policy=args.frag_policy)}),
              flush=True)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    from deserve_b200.pinned import bind_host_to_gpu

    host_binding = bind_host_to_gpu(local)  # before any pinned allocation: swap images on the GPU's NUMA node
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
    parts = set(args.parts.split(","))
    kv = roof = pipe = None
    extras = {}
    if "kv" in parts:
        kv, roof, extras = kv_step_bench(args, dk, rank, world, local, dev, dist)
        gc.collect()
        torch.cuda.empty_cache()
    pipe_error = None
    if "pipe" in parts:
        try:
            pipe = pipeline_bench(args, dk, rank, world, local, dev, dist)
        except (RuntimeError, ValueError) as exc:  # e.g. out of memory: keep the KV-step line
            if kv is None or world > 1:
                raise
            pipe_error = f"{type(exc).__name__}: {exc}"[:300]
    if rank == 0:
        if pipe is not None:
            line = {"metric": METRIC, "value": pipe["value"], "unit": "tok/s", "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": pipe["ms_per_step"], "higher_is_better": True,
                    "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": config_dict(args, world),
                    "gpu_launches": pipe["gpu_launches"],
                    "clocks": pipe["clocks"], "token_sha256": pipe["token_sha256"],
                    "token_checksum": pipe["token_checksum"], "prefill_tokens_per_s": pipe["prefill_tokens_per_s"],
                    "pipeline": pipe["pipeline"]}
            if "e2e" in pipe:
                line["e2e"] = pipe["e2e"]
        else:  # the KV step alone (--parts kv, or the pipeline did not fit)
            line = {"metric": METRIC, "value": kv["value"], "unit": "tok/s", "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": kv["ms_per_step"], "higher_is_better": True,
                    "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": dict(config_dict(args, world), workload=KV_WORKLOAD),
                    "gpu_launches": kv["gpu_launches"], "clocks": kv["clocks"]}
            if "e2e" in kv:
                line["e2e"] = kv["e2e"]
            if pipe_error:
                line["pipeline_error"] = pipe_error
        line["host_binding"] = host_binding
        if kv is not None:
            line["kv_step"] = kv
        if roof is not None:
            line["roofline"] = roof
        line.update(extras)
        if world == 1 and kv is not None and not args.no_library:
            gc.collect()
            torch.cuda.empty_cache()  # the child needs a few GB of the device
            line["library"] = library_in_child()
        if world == 1 and not args.no_cpu_baseline:
            if pipe is not None:
                line["cpu_baseline"], _ = cpu_pipeline_layer_sample(args, 10, 2)
            if kv is not None:
                cb = cpu_kv_layer_sample(args, 6, 1)  # the full 256-sequence one-layer slice, ~10 s of host work
                cb["config1_full"] = cpu_config1_full()
                if pipe is not None:
                    line["kv_step"]["cpu_baseline"] = cb
                else:
                    line["cpu_baseline"] = cb
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
