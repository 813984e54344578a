"""In-process pipeline driver: a Llama-shaped model split by layers over the
GPUs of one node, microbatches rotating through the stages, every stage running
the reference's per-step ordering on its own pool (StageProcessor) and handing
activations to the next stage with NCCL send/recv (RingPipeline).

It replaces, for measurement and parity runs, the HTTP worker shell of the
reference (deserve_worker/worker_api.py, engine/pipeline/processor.py:142-183,
scheduler.py:110-169): the step metadata (which tasks run, with how many tokens)
is recomputed identically on every rank instead of travelling with the request,
like the reference replicates its id lists to every stage (processor.py:254-266).

Schedule of one microbatch of S sequences: ceil(S / c) prefill steps (c whole
prompts each — the reference's 512-token aggregation budget becomes "c prompts"),
then T-1 decode steps of all S sequences.

    python -m torch.distributed.run --nproc-per-node N -m deserve_b200.pipeline_driver --model 70b ...
"""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import dataclass, field

import torch

from .engine import RingPipeline, StageProcessor, StepRequest
from .kvcache import CpuChunkPool, KVCacheManager, PageTableAllocator, VirtualPagePool
from .model import LlamaStage, ModelArgs, llama_3_8b_args, llama_3_70b_args
from .task import SamplingParams, TaskManager


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
    extra: dict = field(default_factory=dict)

    @property
    def prefill_steps(self) -> int:
        return -(-self.seqs // self.prefill_seqs)

    @property
    def steps(self) -> int:
        return self.prefill_steps + self.new_tokens - 1


def make_prompts(cfg: PipelineConfig) -> torch.Tensor:
    rows = []
    for m in range(cfg.n_microbatches):  # one seed per microbatch: microbatch m is the same job at any stage count
        g = torch.Generator().manual_seed(cfg.seed + 12345 + m)
        rows.append(torch.randint(1, cfg.model.vocab_size, (cfg.seqs, cfg.prompt_len), generator=g, dtype=torch.int32))
    return torch.stack(rows)


def run_stage(rank: int, world: int, cfg: PipelineConfig, device: torch.device, dist=None) -> dict:
    """Runs this rank's stage for the whole job. Returns, on the last rank, the
    generated tokens [microbatch][sequence][new_tokens] and timings."""
    a, M, S = cfg.model, cfg.n_microbatches, cfg.seqs
    assert a.n_layers % world == 0 and M == world, "layers must split evenly; one microbatch per stage"
    # one microbatch alone cannot rotate through two swap regions (there is nobody to swap with)
    assert M > 1 or cfg.swap_pages == 0, "a single microbatch needs swap_pages = 0"
    lb, le = rank * a.n_layers // world, (rank + 1) * a.n_layers // world
    stage = LlamaStage(a, lb, le, device, cfg.dtype, seed=cfg.seed, first=(rank == 0), last=(rank == world - 1))
    if stage.need_sample and cfg.output_gain != 1.0:
        stage.output.mul_(cfg.output_gain)
    pool = VirtualPagePool(le - lb, cfg.main_pages, cfg.swap_pages, a.page_size, device, cfg.dtype,
                           n_kv_heads=a.n_kv_heads, head_dim=a.head_dim)
    ctx_len = (cfg.prompt_len + cfg.new_tokens + a.page_size) // a.page_size * a.page_size
    pta = PageTableAllocator(M * S, ctx_len, a.page_size, device)
    chunks = CpuChunkPool(le - lb, 2, a.page_size, cfg.dtype, n_kv_heads=a.n_kv_heads, head_dim=a.head_dim)
    mgr = KVCacheManager(pool, chunks, pta)
    proc = StageProcessor(mgr, TaskManager(pool.num_pages, a.page_size), stage, pta, M, ignore_eos=True)
    prompts = make_prompts(cfg)
    P, c = cfg.prefill_steps, cfg.prefill_seqs
    ids = [[f"m{m}s{i}" for i in range(S)] for m in range(M)]
    first_tokens: dict = {m: [] for m in range(M)}     # rank 0: first generated tokens as they come back
    out_tokens = torch.zeros(M, S, cfg.new_tokens, dtype=torch.int32)
    pending = []                                        # last rank: (m, s, device tokens) copied out at the end
    marks = {}

    def subset(s):
        return list(range(s * c, min(S, (s + 1) * c)))

    def stage_fn(u, m, s, x):
        req = StepRequest(microbatch_id=m, xs=x)
        if s < P:
            sel = subset(s)
            req.exec_task_ids = [ids[m][i] for i in sel]
            req.exec_seqlens = [cfg.prompt_len] * len(sel)
            req.init_tasks = {ids[m][i]: (cfg.prompt_len, SamplingParams()) for i in sel}
            if rank == 0:
                if s > 0:
                    first_tokens[m].append(x)  # first tokens of the previous subset, back from the last stage
                req.xs = prompts[m, sel].reshape(-1).to(device, non_blocking=True)
        else:
            req.exec_task_ids = list(ids[m])
            req.exec_seqlens = [1] * S
            if rank == 0 and s == P:
                first_tokens[m].append(x)
                req.xs = torch.cat(first_tokens[m])
        if s == P and m == 0 and "decode_start" not in marks:
            marks["decode_start"] = torch.cuda.Event(enable_timing=True)
            marks["decode_start"].record()
        proc.synchronize()
        _, result = proc.process_step(req)
        if rank == world - 1:
            pending.append((m, s, result.all_xs))
        return result.ongoing_xs if rank < world - 1 else result.all_xs

    def recv_spec(u):
        m, s = u % M, u // M
        if rank == 0:  # tokens produced by unit (m, s-1)
            n = len(subset(s - 1)) if s - 1 < P else S
            return (n,), torch.int32, device
        n = len(subset(s)) * cfg.prompt_len if s < P else S
        return (n, a.dim), cfg.dtype, device

    first = lambda m: torch.empty(0, dtype=torch.int32, device=device)
    pipe = RingPipeline(rank, world, stage_fn, first, cfg.steps, dist=dist, recv_spec=recv_spec)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0.record()
    pipe.advance(cfg.steps * M + world - 1)
    t1.record()
    torch.cuda.synchronize()
    res = {"total_ms": t0.elapsed_time(t1)}
    if "decode_start" in marks:
        res["decode_ms"] = marks["decode_start"].elapsed_time(t1)
    if rank == world - 1:
        for m, s, toks in pending:
            toks = toks.cpu()
            if s < P:
                out_tokens[m, subset(s), 0] = toks
            else:
                out_tokens[m, :, s - P + 1] = toks
        res["tokens"] = out_tokens
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="70b", choices=["8b", "70b"])
    ap.add_argument("--microbatch-seqs", type=int, default=128)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--prefill-seqs", type=int, default=8)
    ap.add_argument("--swap-fraction", type=float, default=0.25, help="share of a microbatch's pages meant for its swap region")
    args = ap.parse_args()
    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    model = llama_3_70b_args if args.model == "70b" else llama_3_8b_args
    per_mb = args.microbatch_seqs * (-(-(args.prompt + args.new_tokens) // model.page_size))
    swap = int(per_mb * args.swap_fraction)
    cfg = PipelineConfig(model=model, n_microbatches=world, seqs=args.microbatch_seqs, prompt_len=args.prompt,
                         new_tokens=args.new_tokens, prefill_seqs=args.prefill_seqs,
                         main_pages=int(world * (per_mb - swap) * 1.1) + 64 + (per_mb if world == 1 else 0),
                         swap_pages=swap if world > 1 else 0)
    res = run_stage(rank, world, cfg, dev, dist if world > 1 else None)
    if world > 1:
        t = torch.tensor([res["total_ms"], res.get("decode_ms", 0.0)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res["total_ms"], res["decode_ms"] = float(t[0]), float(t[1])
    if rank == world - 1:
        n_decode = world * args.microbatch_seqs * (args.new_tokens - 1)
        print(json.dumps({
            "workload": f"llama3-{args.model}-shaped pipeline, {world} stages x {world} microbatches x "
                        f"{args.microbatch_seqs} sequences, prompt {args.prompt}, {args.new_tokens} greedy tokens, region swap on",
            "n_gpus": world, "total_ms": res["total_ms"], "decode_ms": res["decode_ms"],
            "decode_tokens_per_s": n_decode / (res["decode_ms"] * 1e-3),
            "all_tokens_per_s": world * args.microbatch_seqs * (args.prompt + args.new_tokens) / (res["total_ms"] * 1e-3),
            "token_checksum": int(res["tokens"].long().sum())}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
