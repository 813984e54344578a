"""In-process pipeline driver: a Llama-shaped model split by layers over the
GPUs of one node, microbatches rotating through the stages, every stage running
the reference's per-step ordering on its own pool (StageProcessor) and handing
activations to the next stage over NCCL send/recv links (RingPipeline).

It replaces, for measurement and parity runs, the HTTP worker shell of the
reference (deserve_worker/worker_api.py, engine/pipeline/processor.py:142-183,
scheduler.py:110-169): the step metadata (which tasks run, with how many tokens)
is recomputed identically on every rank instead of travelling with the request,
like the reference replicates its id lists to every stage (processor.py:254-266).

Schedule of one microbatch of S sequences: ceil(S / c) prefill steps (c whole
prompts each — the reference's 512-token aggregation budget becomes "c prompts"),
then T-1 decode steps of all S sequences. A job of M microbatches runs in waves of
`concurrent` microbatches (the number whose KV fits beside the stage's weights);
inside a wave the microbatches rotate through the stages, so any number of stages
up to `concurrent` is kept busy.

    python -m torch.distributed.run --nproc-per-node N -m deserve_b200.pipeline_driver --model 70b ...
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
from dataclasses import dataclass, field

import numpy as np
import torch

from . import _lib
from .engine import RingPipeline, StageProcessor, StepRequest, make_ring_links
from .kvcache import CpuChunkPool, KVCacheManager, PageTableAllocator, VirtualPagePool
from .model import LlamaStage, ModelArgs, llama_3_8b_args, llama_3_70b_args
from .task import SamplingParams, TaskManager
from .trace import phase


@dataclass
class PipelineConfig:
    model: ModelArgs
    n_microbatches: int = 2
    seqs: int = 4                 # sequences per microbatch
    prompt_len: int = 32
    new_tokens: int = 8           # generated tokens per sequence (the first one comes out of the prefill)
    prefill_seqs: int = 2         # prompts per prefill step
    main_pages: int = 64
    swap_pages: int = 16
    dtype: torch.dtype = torch.bfloat16
    seed: int = 0
    output_gain: float = 1.0      # multiplies the output projection (tests use decisive logits)
    concurrent: int | None = None  # microbatches in flight at once (a wave); None = all of them
    warmup_tokens: int = 0        # decode steps of every wave that run before its timed region
    host_tokens: bool = False     # every step's tokens go to pinned host memory (first stage) and the next
    #                               step's input comes back from there (the serving loop a client sees)
    extra: dict = field(default_factory=dict)

    @property
    def prefill_steps(self) -> int:
        return -(-self.seqs // self.prefill_seqs)

    @property
    def steps(self) -> int:
        return self.prefill_steps + self.new_tokens - 1

    @property
    def wave_size(self) -> int:
        return self.n_microbatches if self.concurrent is None else self.concurrent


def make_prompts(cfg: PipelineConfig) -> torch.Tensor:
    rows = []
    for m in range(cfg.n_microbatches):  # one seed per microbatch: microbatch m is the same job at any stage count
        g = torch.Generator().manual_seed(cfg.seed + 12345 + m)
        rows.append(torch.randint(1, cfg.model.vocab_size, (cfg.seqs, cfg.prompt_len), generator=g, dtype=torch.int32))
    return torch.stack(rows)


def token_digest(tokens: torch.Tensor) -> str:
    """SHA-256 of the generated tokens [microbatch, sequence, new token] (int32, C order):
    equal digests at two stage counts mean that not one greedy token differs."""
    return hashlib.sha256(np.ascontiguousarray(tokens.cpu().numpy().astype(np.int32)).tobytes()).hexdigest()


def size_pools(model: ModelArgs, layers_here: int, n_microbatches: int, seqs: int, prompt_len: int, new_tokens: int,
               kv_budget_bytes: int, world: int, sized_for_tokens: int | None = None, elem_bytes: int = 2) -> dict:
    """How many microbatches run at once and how the stage's pages are split, from
    the memory left beside the weights.

    * concurrent = the largest divisor of n_microbatches whose KV (at the context
      length the job is sized for) fits the budget, but never fewer than the
      number of stages;
    * with two or more microbatches in flight the region swap is on: a region holds
      one page per sequence plus the allocator's prefetch slack, and the main pages
      hold every page of every microbatch except its last one, so that the last
      16 tokens of each sequence live in its microbatch's swap region and travel to
      pinned host memory and back while the other microbatches compute. A region of
      this size (seqs + 64 pages per layer) crosses the host link in less time than
      a stage needs for one microbatch at any stage count, because both scale with
      the stage's layer count.
    """
    ps = model.page_size
    page_bytes = 2 * ps * model.n_kv_heads * model.head_dim * elem_bytes * layers_here
    pages_seq = -(-(prompt_len + new_tokens) // ps)
    pages_seq_sized = -(-(prompt_len + (sized_for_tokens or new_tokens)) // ps)
    per_mb = seqs * pages_seq_sized * page_bytes
    fit = max(1, kv_budget_bytes // max(per_mb, 1))
    concurrent = max([d for d in range(1, n_microbatches + 1) if n_microbatches % d == 0 and d <= fit] or [1])
    if concurrent < world:
        raise ValueError(f"{world} stages need {world} microbatches in flight; the KV budget holds {fit}")
    swap = seqs + 64 if concurrent > 1 and pages_seq > 1 else 0
    if swap:
        main = concurrent * seqs * (pages_seq - 1) + 64
    else:
        main = concurrent * seqs * pages_seq + 128
    return {"concurrent": concurrent, "main_pages": main, "swap_pages": swap, "pages_per_sequence": pages_seq,
            "kv_bytes_per_microbatch": seqs * pages_seq * page_bytes, "pool_bytes": (main + 2 * swap) * page_bytes}


def make_stage(model: ModelArgs, rank: int, world: int, device, dtype=torch.bfloat16, seed: int = 0,
               output_gain: float = 1.0) -> LlamaStage:
    """This rank's layers of the model, with the output head split between the last and the first stage."""
    lb, le = rank * model.n_layers // world, (rank + 1) * model.n_layers // world
    stage = LlamaStage(model, lb, le, device, dtype, seed=seed, first=(rank == 0), last=(rank == world - 1),
                       split_head=True)
    if output_gain != 1.0:
        for name in ("output_lo", "output_hi"):
            if hasattr(stage, name):
                getattr(stage, name).mul_(output_gain)
    return stage


def run_stage(rank: int, world: int, cfg: PipelineConfig, device: torch.device, dist=None, stage: LlamaStage | None = None,
              links=None, barrier=None) -> dict:
    """Runs this rank's stage for the whole job. Returns timings and page / swap
    statistics and, on rank 0, the generated tokens
    [microbatch][sequence][new_tokens]. The output head is split: the last stage
    hands the first stage the normed rows and its half's (max, argmax), the first
    stage finishes the tokens when the message arrives (LlamaStage.finish_head).

    Timed regions (CUDA events on the compute stream, each bracketed by a device
    synchronisation and `barrier()`): the prefill slots of every wave, and the
    decode slots of every wave after its warm-up tokens; both summed over waves."""
    a, M, S = cfg.model, cfg.n_microbatches, cfg.seqs
    Mw = cfg.wave_size
    assert a.n_layers % world == 0 and M % Mw == 0 and Mw >= world, "layers / microbatches must split evenly"
    # one microbatch alone cannot rotate through two swap regions (there is nobody to swap with)
    assert Mw > 1 or cfg.swap_pages == 0, "a single microbatch in flight needs swap_pages = 0"
    lb, le = rank * a.n_layers // world, (rank + 1) * a.n_layers // world
    if stage is None:
        stage = make_stage(a, rank, world, device, cfg.dtype, cfg.seed, cfg.output_gain)
    pool = VirtualPagePool(le - lb, cfg.main_pages, cfg.swap_pages, a.page_size, device, cfg.dtype,
                           n_kv_heads=a.n_kv_heads, head_dim=a.head_dim)
    ctx_len = (cfg.prompt_len + cfg.new_tokens + a.page_size) // a.page_size * a.page_size
    pta = PageTableAllocator(Mw * S, ctx_len, a.page_size, device)
    chunks = CpuChunkPool(le - lb, 2, a.page_size, cfg.dtype, n_kv_heads=a.n_kv_heads, head_dim=a.head_dim)
    mgr = KVCacheManager(pool, chunks, pta)
    tasks = TaskManager(pool.num_pages, a.page_size)
    proc = StageProcessor(mgr, tasks, stage, pta, Mw, ignore_eos=True)
    prompts = make_prompts(cfg)
    P, c = cfg.prefill_steps, cfg.prefill_seqs
    Wm = cfg.warmup_tokens
    K = cfg.new_tokens - 1 - Wm
    assert K >= 0, "warmup_tokens exceeds the decode steps of the job"
    out_tokens = torch.zeros(M, S, cfg.new_tokens, dtype=torch.int32)
    if barrier is None:
        barrier = dist.barrier if (dist is not None and world > 1) else (lambda: None)
    if world > 1 and links is None:
        links = make_ring_links(dist, rank, world, device)
    elem = torch.empty(0, dtype=cfg.dtype).element_size()
    host_ring = ([torch.empty(max(S, 1), dtype=torch.int32, pin_memory=True) for _ in range(Mw + 2)]
                 if cfg.host_tokens else None)
    stats = {"prefill_ms": 0.0, "decode_ms": 0.0, "decode_compute_ms": 0.0, "pages_free_min": pool.num_avails,
             "swap_pages_out": 0, "swap_pages_in": 0, "swap_slots": 0, "swap_pages_out_max": 0, "slots_timed": 0,
             "launches_timed": 0, "swap_dma_out_ms": 0.0, "swap_dma_in_ms": 0.0, "swap_dma_slots": 0,
             "swap_rows_out": 0, "swap_rows_in": 0}

    def subset(s):
        return list(range(s * c, min(S, (s + 1) * c)))

    def timed(fn):
        torch.cuda.synchronize(device)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize(device)
        barrier()
        return e0.elapsed_time(e1)

    for wave in range(M // Mw):
        ids = [[f"w{wave}m{m}s{i}" for i in range(S)] for m in range(Mw)]
        first_tokens: dict = {m: [] for m in range(Mw)}  # rank 0: first generated tokens as they come back
        pending = []                                      # rank 0: (m, step, tokens) copied out at the end of the wave
        slot_events = []
        in_timed = [False]
        n_host = [0]

        def stage_fn(u, m, s, x):
            gm = wave * Mw + m
            if rank == 0 and s > 0 and x.dtype == torch.uint8:
                # the last stage's message of step s-1: normed rows + its half of the head; finish the tokens
                with phase("finish_head"):
                    x = stage.finish_head(x)
                if cfg.host_tokens:
                    # serving loop over several stages: the client reads the step's tokens from pinned host memory
                    # and the next step's input comes from there (the host waits for the copy)
                    with phase("tokens_to_host"):
                        h = host_ring[n_host[0] % len(host_ring)][: x.numel()]
                        n_host[0] += 1
                        h.copy_(x, non_blocking=True)
                        torch.cuda.current_stream(device).synchronize()
                    x = h  # pinned; stays intact until Mw + 1 further steps have passed
                pending.append((m, s - 1, x.clone() if cfg.host_tokens else x))
            req = StepRequest(microbatch_id=m, xs=x)
            if s < P:
                sel = subset(s)
                req.exec_task_ids = [ids[m][i] for i in sel]
                req.exec_seqlens = [cfg.prompt_len] * len(sel)
                req.init_tasks = {ids[m][i]: (cfg.prompt_len, SamplingParams()) for i in sel}
                if rank == 0:
                    if s > 0:  # first tokens of the previous subset
                        first_tokens[m].append(x if x.is_cuda else x.clone())
                    req.xs = prompts[gm, sel].reshape(-1).to(device, non_blocking=True)
            else:
                req.exec_task_ids = list(ids[m])
                req.exec_seqlens = [1] * S
                if rank == 0 and s == P:
                    first_tokens[m].append(x if x.is_cuda else x.clone())
                    req.xs = torch.cat(first_tokens[m])
                if rank == 0 and not req.xs.is_cuda:
                    req.xs = req.xs.to(device, non_blocking=True)  # host_tokens: the step's input comes from the host
            if in_timed[0]:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record()
            proc.synchronize()
            _, result = proc.process_step(req)
            y = result.ongoing_xs  # activations; on the last stage the packed partial head
            if cfg.host_tokens and world == 1:
                with phase("tokens_to_host"):
                    toks = stage.finish_head(y)  # one stage: finish at once, the client reads the tokens now
                    h = host_ring[n_host[0] % len(host_ring)][: toks.numel()]
                    n_host[0] += 1
                    h.copy_(toks, non_blocking=True)
                    torch.cuda.current_stream(device).synchronize()
                pending.append((m, s, h.clone()))
                y = h  # pinned; stays intact until Mw + 1 further steps have passed
            if in_timed[0]:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                slot_events.append((e0, e1))
                stats["pages_free_min"] = min(stats["pages_free_min"], pool.num_avails)
                if pool.num_pages_swap:
                    o, i_ = pool.last_swap_pages
                    stats["swap_pages_out"] += o
                    stats["swap_pages_in"] += i_
                    stats["swap_pages_out_max"] = max(stats["swap_pages_out_max"], o)
                    stats["swap_rows_out"] += pool.last_swap_rows[0]
                    stats["swap_rows_in"] += pool.last_swap_rows[1]
                    stats["swap_slots"] += 1
            return y

        def recv_spec(u):
            m, s = u % Mw, u // Mw
            if rank == 0:  # the packed partial head of unit (m, s-1): rows, then float maxima, then int indices
                n = len(subset(s - 1)) if s - 1 < P else S
                return (n * (a.dim * elem + 8),), torch.uint8, device
            n = len(subset(s)) * cfg.prompt_len if s < P else S
            return (n, a.dim), cfg.dtype, device

        first = lambda m: torch.empty(0, dtype=torch.int32, device=device)
        pipe = RingPipeline(rank, world, stage_fn, first, cfg.steps, dist=dist, recv_spec=recv_spec, microbatches=Mw,
                            links=links, send_final=True)
        stats["prefill_ms"] += timed(lambda: pipe.advance(P * Mw))
        pipe.advance(Wm * Mw)
        in_timed[0] = True
        if pool.num_pages_swap:
            pool.dma_events = []
        launches0 = _lib.LAUNCHES[0]
        stats["decode_ms"] += timed(lambda: pipe.advance(K * Mw))
        stats["launches_timed"] += _lib.LAUNCHES[0] - launches0  # this package's kernels inside the timed region
        in_timed[0] = False
        pipe.advance(world - 1)  # the last units of the later stages
        if not (cfg.host_tokens and world == 1):  # the last step's tokens: the first stage finishes the last stage's partial heads
            for m, packed in enumerate(pipe.take_finals()):
                pending.append((m, cfg.steps - 1, stage.finish_head(packed)))
        pipe.flush()
        torch.cuda.synchronize(device)
        stats["decode_compute_ms"] += sum(e0.elapsed_time(e1) for e0, e1 in slot_events)
        stats["slots_timed"] += len(slot_events)
        if pool.dma_events:  # how long the region DMA of a slot runs on its side streams (both directions overlap)
            stats["swap_dma_out_ms"] += sum(a.elapsed_time(b) for a, b, _, _ in pool.dma_events)
            stats["swap_dma_in_ms"] += sum(c.elapsed_time(d) for _, _, c, d in pool.dma_events)
            stats["swap_dma_slots"] += len(pool.dma_events)
        pool.dma_events = None
        if rank == 0:
            for m, s, toks in pending:
                toks = toks.cpu()
                gm = wave * Mw + m
                if s < P:
                    out_tokens[gm, subset(s), 0] = toks
                else:
                    out_tokens[gm, :, s - P + 1] = toks
        # the wave is done: its tasks leave, their pages and table rows return to the pool. Each
        # microbatch is cancelled in a slot of its own, through the stage loop, so that its swap
        # region is the active one when its pages go back to the bitmap
        for m in range(Mw):
            proc.synchronize()
            proc.process_step(StepRequest(microbatch_id=m, xs=first(m), cancel_task_ids=list(ids[m])))
            for t in ids[m]:
                tasks.task_datas.pop(t, None)
    res = dict(stats)
    res["total_ms"] = stats["prefill_ms"] + stats["decode_ms"]
    res["decode_steps_timed"] = K
    res["bubble_frac"] = (1.0 - stats["decode_compute_ms"] / stats["decode_ms"]) if stats["decode_ms"] > 0 else 0.0
    res["stage"] = stage
    if rank == 0:
        res["tokens"] = out_tokens
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="70b", choices=["8b", "70b"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the model's)")
    ap.add_argument("--microbatches", type=int, default=8)
    ap.add_argument("--microbatch-seqs", type=int, default=128)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--warmup-tokens", type=int, default=4)
    ap.add_argument("--prefill-seqs", type=int, default=8)
    ap.add_argument("--kv-budget-gb", type=float, default=0.0, help="0 = what is free after the weights, minus 8 GB")
    args = ap.parse_args()
    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    from .pinned import bind_host_to_gpu

    bind_host_to_gpu(local)  # before the pinned swap images are allocated
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    model = llama_3_70b_args if args.model == "70b" else llama_3_8b_args
    if args.layers:
        model = ModelArgs(**{**model.__dict__, "n_layers": args.layers})
    lb, le = rank * model.n_layers // world, (rank + 1) * model.n_layers // world
    stage = make_stage(model, rank, world, dev)
    free, _ = torch.cuda.mem_get_info(dev)
    budget = int(args.kv_budget_gb * 1e9) if args.kv_budget_gb else free - (8 << 30)
    if world > 1:
        t = torch.tensor([budget], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        budget = int(t.item())
    sz = size_pools(model, le - lb, args.microbatches, args.microbatch_seqs, args.prompt, args.new_tokens, budget, world)
    cfg = PipelineConfig(model=model, n_microbatches=args.microbatches, seqs=args.microbatch_seqs,
                         prompt_len=args.prompt, new_tokens=args.new_tokens, prefill_seqs=args.prefill_seqs,
                         main_pages=sz["main_pages"], swap_pages=sz["swap_pages"], concurrent=sz["concurrent"],
                         warmup_tokens=args.warmup_tokens)
    res = run_stage(rank, world, cfg, dev, dist if world > 1 else None, stage=stage)
    if world > 1:
        t = torch.tensor([res["prefill_ms"], res["decode_ms"]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res["prefill_ms"], res["decode_ms"] = float(t[0]), float(t[1])
    if rank == 0:
        n_decode = args.microbatches * args.microbatch_seqs * res["decode_steps_timed"]
        print(json.dumps({
            "workload": f"llama3-{args.model}-shaped pipeline, {model.n_layers} layers on {world} stages, "
                        f"{args.microbatches} microbatches x {args.microbatch_seqs} sequences ({sz['concurrent']} in "
                        f"flight), prompt {args.prompt}, {args.new_tokens} greedy tokens, region swap "
                        f"{'on' if sz['swap_pages'] else 'off'}",
            "n_gpus": world, "prefill_ms": res["prefill_ms"], "decode_ms": res["decode_ms"],
            "decode_tokens_per_s": n_decode / (res["decode_ms"] * 1e-3),
            "prefill_tokens_per_s": args.microbatches * args.microbatch_seqs * args.prompt / (res["prefill_ms"] * 1e-3),
            "bubble_frac": res["bubble_frac"], "pools": sz,
            "token_checksum": int(res["tokens"].long().sum()), "token_sha256": token_digest(res["tokens"])}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
