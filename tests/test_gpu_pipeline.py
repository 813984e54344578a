"""The layer-sharded model pipeline: greedy tokens of a 2-stage NCCL pipeline must
equal those of the same job on one GPU, and both must match the dense fp32 CPU
model. The one-GPU half runs on any box; the 2-stage half needs two GPUs."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

import deserve_b200 as dk
from deserve_b200.pipeline_driver import PipelineConfig, make_prompts, make_stage, run_stage
from oracle.llama_ref import DenseLlama

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _cfg(n_mb):
    model = dk.ModelArgs(dim=512, n_layers=4, n_heads=8, n_kv_heads=2, vocab_size=640, ffn_dim=1024, page_size=16)
    # two microbatches: 12 main pages for 30 needed, so both also live in their swap regions
    return PipelineConfig(model=model, n_microbatches=n_mb, seqs=5, prompt_len=37, new_tokens=6, prefill_seqs=2,
                          main_pages=12 if n_mb > 1 else 20, swap_pages=10 if n_mb > 1 else 0, output_gain=12.0, seed=4)


def _dense_tokens(cfg):
    dev = torch.device("cuda:0")
    full = make_stage(cfg.model, 0, 1, dev, cfg.dtype, cfg.seed, cfg.output_gain)  # both halves of the split head
    ref = DenseLlama(cfg.model, full.layers, full.tok_embeddings, full.norm, full.full_output)
    prompts = make_prompts(cfg)
    out = torch.zeros(cfg.n_microbatches, cfg.seqs, cfg.new_tokens, dtype=torch.int32)
    gaps = []
    return ref, prompts, out, gaps


def _check_against_dense(cfg, tokens):
    ref, prompts, _, _ = _dense_tokens(cfg)
    bad = []
    for m in range(cfg.n_microbatches):
        for i in range(cfg.seqs):
            tid = f"m{m}s{i}"
            want = ref.step(tid, prompts[m, i])
            for j in range(cfg.new_tokens):
                got = int(tokens[m, i, j])
                if got != want:
                    bad.append((tid, j, got, want, float(ref.last_logits[want] - ref.last_logits[got])))
                if j + 1 < cfg.new_tokens:
                    want = ref.step(tid, torch.tensor([got], dtype=torch.int32))
    assert all(g < 0.05 for *_, g in bad), bad          # only ties within 16-bit resolution may differ
    assert len(bad) <= max(1, tokens.numel() // 20), bad


def test_split_head_gives_the_argmax_over_the_whole_vocabulary():
    """The last stage's half (max, argmax) + the first stage's half = the argmax over all logits, the lowest
    index among equal maxima; a maximum that occurs in both halves goes to the lower half."""
    dev = torch.device("cuda:0")
    model = dk.ModelArgs(dim=256, n_layers=1, n_heads=4, n_kv_heads=2, vocab_size=1000, ffn_dim=512, page_size=16)
    st = make_stage(model, 0, 1, dev, torch.bfloat16, seed=1)
    assert st.output_lo.shape[0] == 504 and st.output_hi.shape[0] == 496 and not st.need_sample
    st.output_hi[7] = st.output_lo[100] * 3      # rows 0..3 will peak at column 100 and, equally, at 504 + 7
    st.output_lo[100] *= 3
    g = torch.Generator(device=dev).manual_seed(0)
    hn = torch.randn(37, 256, device=dev, generator=g).to(torch.bfloat16)
    hn[:4] = st.output_lo[100].sign() * 0.5       # aligned with that row: its logit is the maximum
    packed = st.pack_partial(hn)
    assert packed.dtype == torch.uint8 and packed.numel() == 37 * (256 * 2 + 8) and st.partial_rows(packed) == 37
    got = st.finish_head(packed)
    logits = torch.cat([hn @ st.output_lo.t(), hn @ st.output_hi.t()], dim=1)
    want = dk.greedy_sample(logits)
    assert torch.equal(got, want)
    assert got[:4].tolist() == [100] * 4 and (logits[:4, 100] == logits[:4, 504 + 7]).all()
    assert (got >= 504).any() and (got < 504).any()


def _cfg_many(concurrent, host_tokens=False):
    """Four microbatches of five sequences (43 tokens = 3 pages each), `concurrent` of them in flight."""
    model = dk.ModelArgs(dim=512, n_layers=4, n_heads=8, n_kv_heads=2, vocab_size=640, ffn_dim=1024, page_size=16)
    swap = 12 if concurrent > 1 else 0
    main = concurrent * 5 * 3 - 8 if swap else concurrent * 5 * 3 + 8  # with swap: eight pages of the last microbatch spill
    return PipelineConfig(model=model, n_microbatches=4, seqs=5, prompt_len=37, new_tokens=6, prefill_seqs=2,
                          main_pages=main, swap_pages=swap, output_gain=12.0, seed=4, concurrent=concurrent,
                          warmup_tokens=2, host_tokens=host_tokens)


def test_waves_swap_and_the_host_token_loop_do_not_change_a_token():
    """The same four microbatches (a) all in flight with the region swap on, (b) in two waves of two,
    (c) one after the other without swap, (d) one after the other with every step's tokens going
    through pinned host memory: the generated tokens must be identical, bit for bit."""
    dev = torch.device("cuda:0")
    runs = {name: run_stage(0, 1, cfg, dev) for name, cfg in [
        ("all in flight", _cfg_many(4)), ("two waves", _cfg_many(2)), ("one at a time", _cfg_many(1)),
        ("host tokens", _cfg_many(1, host_tokens=True))]}
    base = runs["one at a time"]["tokens"]
    assert base.shape == (4, 5, 6) and (base > 0).any()
    for name, res in runs.items():
        assert torch.equal(res["tokens"], base), name
        assert res["decode_steps_timed"] == 3 and res["decode_ms"] > 0 and res["prefill_ms"] > 0
    assert runs["all in flight"]["swap_slots"] > 0 and runs["all in flight"]["swap_pages_out"] > 0, \
        "with four microbatches in flight live pages must travel through the swap regions"
    _check_against_dense(_cfg_many(1), base)


def test_one_stage_pipeline_matches_dense_model():
    cfg = _cfg(1)
    res = run_stage(0, 1, cfg, torch.device("cuda:0"))
    _check_against_dense(cfg, res["tokens"])


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    res = run_stage(rank, world, _cfg(world), dev, dist)
    # more microbatches than stages: four in flight on two stages, then two waves of two
    many = [run_stage(rank, world, _cfg_many(c), dev, dist) for c in (4, 2)]
    # the serving loop over two stages: the first stage passes every step's tokens through pinned host memory
    many.append(run_stage(rank, world, _cfg_many(4, host_tokens=True), dev, dist))
    if rank == 0:  # the first stage finishes the split output head, so the tokens are there
        q.put((res["tokens"].clone(), [m["tokens"].clone() for m in many]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_stage_pipeline_matches_one_stage_and_dense():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        tokens2, many2 = q.get(timeout=240)
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        for p in procs:  # a worker that is still here hangs: do not leave it behind
            if p.is_alive():
                p.kill()
    _check_against_dense(_cfg(2), tokens2)
    # microbatch 0 as a one-stage job on one GPU: splitting the layers must not change a token
    res = run_stage(0, 1, _cfg(1), torch.device("cuda:0"))
    assert torch.equal(res["tokens"][0], tokens2[0]), "stage split changed the greedy tokens"
    one_gpu = run_stage(0, 1, _cfg_many(1), torch.device("cuda:0"))["tokens"]
    for got in many2:  # four microbatches on two stages, all in flight, in two waves, or with host tokens: the one-GPU tokens
        assert torch.equal(got, one_gpu), "stage split / waves changed the greedy tokens"
