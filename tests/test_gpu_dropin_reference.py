"""Drop-in check with the REFERENCE's own caller code: its unmodified
Attention.paged_forward (deserve_worker/model/layer/attention.py:160-193), RMSNorm,
TransformerBlock, BatchDecode / BatchPrefill.prepare/step
(deserve_worker/execution/exec.py:178-243) and MicroBatchProcessor.join / step /
offload / reload (deserve_worker/engine/microbatch/processor.py:24-146) run on the
GPU with this package standing where the reference imports `flashinfer`, its
`deserve_worker.kvcache.*` modules and `deserve_worker.model.context.flash` — the
import swaps a maintainer would make. The activations they produce are compared
with a dense fp32 evaluation of the same blocks.

The reference's sources are not part of this repository: the test runs from a
working copy staged by tests/golden/stage_reference_tree.py and is skipped
where that copy is absent."""
import sys
import types
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (REF / "deserve_worker").is_dir(), reason="no staged copy of the reference")]


def _install_shims():
    import deserve_b200 as dk
    from deserve_b200 import context, kvcache, ops

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    norm = mod("flashinfer.norm", rmsnorm=ops.rmsnorm)
    mod("flashinfer", append_paged_kv_cache=ops.append_paged_kv_cache, apply_rope=ops.apply_rope,
        BatchDecodeWithPagedKVCacheWrapper=ops.BatchDecodeWithPagedKVCacheWrapper,
        BatchPrefillWithPagedKVCacheWrapper=ops.BatchPrefillWithPagedKVCacheWrapper, norm=norm)
    mod("deserve_worker.kvcache.paged.page_pool", PagePool=kvcache.PagePool, GpuPagePool=kvcache.GpuPagePool,
        CpuPagePool=kvcache.CpuPagePool)
    mod("deserve_worker.kvcache.paged.page_table", PageTableAllocator=kvcache.PageTableAllocator,
        PageTableHandle=kvcache.PageTableHandle)
    mod("deserve_worker.kvcache.paged.kvcache", PagedKVCache=kvcache.PagedKVCache)
    mod("deserve_worker.kvcache.paged.chunk_pool", ChunkPool=kvcache.ChunkPool, ChunkHandle=kvcache.ChunkHandle,
        CpuChunkPool=kvcache.CpuChunkPool)
    mod("deserve_worker.kvcache.pinned.pinned_memory", PinnedMemory=kvcache.PinnedMemory)
    mod("deserve_worker.kvcache.pinned.kvcache", PinnedKVCache=kvcache.PinnedKVCache)
    mod("deserve_worker.kvcache.virtual", VirtualPagePool=kvcache.VirtualPagePool,
        VirtualPagedKVCache=kvcache.VirtualPagedKVCache, CopiedPinnedMemory=kvcache.CopiedPinnedMemory)
    mod("deserve_worker.kvcache.manager", KVCacheManager=kvcache.KVCacheManager)
    mod("deserve_worker.model.context.flash", FlashForwardCtx=context.FlashForwardCtx,
        FlashDecodeCtx=context.FlashDecodeCtx, FlashPrefillCtx=context.FlashPrefillCtx)
    return dk


@pytest.fixture(scope="module")
def ref():
    """The reference's modules, imported from the staged copy with the shims in place."""
    saved = {k: v for k, v in sys.modules.items() if k.startswith(("deserve_worker", "deserve_utils", "flashinfer"))}
    for k in saved:
        del sys.modules[k]
    dtype0 = torch.get_default_dtype()
    sys.path.insert(0, str(REF))
    try:
        dk = _install_shims()
        import deserve_worker.task as task            # sets the default dtype to fp16 and main_device to "cuda"
        import deserve_worker.execution.exec as ex    # allocates its 128 MiB workspace and both wrappers at import
        import deserve_worker.engine.microbatch.processor as mbp
        from deserve_utils.trace import LayerId
        from deserve_worker.model.args import ModelArgs
        from deserve_worker.model.llama import TransformerBlock
        yield types.SimpleNamespace(dk=dk, task=task, ex=ex, mbp=mbp, LayerId=LayerId, ModelArgs=ModelArgs,
                                    TransformerBlock=TransformerBlock)
    finally:
        torch.set_default_dtype(dtype0)
        sys.path.remove(str(REF))
        for k in [k for k in sys.modules if k.startswith(("deserve_worker", "deserve_utils", "flashinfer"))]:
            del sys.modules[k]
        sys.modules.update(saved)


class _Layers:
    """What the reference's LayerStorage is to its callers (layer_storage.py:182-197), over blocks built here."""

    need_sample = False
    need_tokenize = False

    def __init__(self, blocks, model_args):
        self.blocks, self.model_args = blocks, model_args

    @torch.inference_mode()
    def forward(self, h, ctx):
        for b in self.blocks:
            h = b(h, ctx)
            ctx.layer_id += 1
        return h


def _dense_block(blk, x, k_cache, v_cache, start, n_heads, n_kv_heads, hd, eps):
    """One reference block in fp32 on the CPU for one request (x: its new rows)."""
    from oracle import kv_math

    f = lambda t: t.detach().float().cpu()
    a = blk.attention
    norm = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * f(w)
    h = norm(x, blk.attention_norm.weight)
    pos = torch.arange(start, start + x.shape[0])
    q = kv_math.apply_rope((h @ f(a.wq.weight).t()).reshape(-1, n_heads, hd), pos, 500000.0)
    k = kv_math.apply_rope((h @ f(a.wk.weight).t()).reshape(-1, n_kv_heads, hd), pos, 500000.0)
    v = (h @ f(a.wv.weight).t()).reshape(-1, n_kv_heads, hd)
    k_all = k if k_cache is None else torch.cat([k_cache, k])
    v_all = v if v_cache is None else torch.cat([v_cache, v])
    attn = kv_math.dense_attention(q, k_all, v_all, causal_tail=True)
    hh = x + attn.reshape(-1, n_heads * hd) @ f(a.wo.weight).t()
    ff = blk.feed_forward
    g = norm(hh, blk.ffn_norm.weight)
    out = hh + (torch.nn.functional.silu(g @ f(ff.w1.weight).t()) * (g @ f(ff.w3.weight).t())) @ f(ff.w2.weight).t()
    return out, k_all, v_all


def test_reference_callers_run_on_this_package(ref):
    dk, dev = ref.dk, torch.device("cuda")
    n_heads, n_kv_heads, hd, ps, n_layers = 16, 8, 128, 8, 2   # the reference's pool fixes 8 kv heads x 128
    args = ref.ModelArgs(dim=n_heads * hd, n_layers=n_layers, n_heads=n_heads, n_kv_heads=n_kv_heads, vocab_size=1000,
                         page_size=ps)
    g = torch.Generator().manual_seed(0)
    blocks = []
    for i in range(n_layers):
        blk = ref.TransformerBlock(ref.LayerId(layer=f"layers.{i}"), args)
        for p in blk.parameters():
            if p.dim() == 2:
                p.data = (torch.randn(p.shape, generator=g) * 0.03).to(torch.float16)
            else:
                p.data = (1.0 + 0.1 * torch.randn(p.shape, generator=g)).to(torch.float16)
        blocks.append(blk.to(dev))
    layers = _Layers(blocks, args)
    pool = dk.VirtualPagePool(n_layers, 40, 6, ps, dev, torch.float16)
    pool.pages.fill_(float("nan"))
    pta = dk.PageTableAllocator(8, 512, ps, dev)
    chunks = dk.CpuChunkPool(n_layers, 6, ps, torch.float16)
    mgr = dk.KVCacheManager(pool, chunks, pta)
    tm = ref.task.TaskManager(pool.num_pages, ps)
    mbs = [ref.mbp.MicroBatchProcessor(mgr, tm, layers, pta, True) for _ in range(2)]
    mb = mbs[0]
    lens = {"a": 21, "b": 5, "c": 40}
    for t, n in lens.items():
        tm.add(ref.task.TaskData.empty(t, n, ref.task.SamplingParams()))
    mb.join(list(lens))
    dense = {t: [[None, None] for _ in range(n_layers)] for t in lens}
    fed = {t: 0 for t in lens}
    worst = 0.0

    def run(ids, rows):
        nonlocal worst
        xs = torch.cat([rows[t] for t in ids]).to(dev)
        for t in ids:
            tm.get(t).init(rows[t].shape[0])
        pool.switch()
        res = mb.step(ids, xs, mbs[1], mbs[1])     # the reference's own step: prepare, swap2, layers
        got = res.all_xs.float().cpu().split([rows[t].shape[0] for t in ids])
        for t, y in zip(ids, got):
            x = rows[t].float()
            for li, blk in enumerate(blocks):
                x, dense[t][li][0], dense[t][li][1] = _dense_block(blk, x, dense[t][li][0], dense[t][li][1], fed[t],
                                                                   n_heads, n_kv_heads, hd, args.norm_eps)
            worst = max(worst, ((y - x).abs().max() / x.abs().max().clamp_min(1.0)).item())
            fed[t] += rows[t].shape[0]
            tm.get(t).step()

    # a prefill batch (BatchPrefill), then decode steps (BatchDecode); one task sits one step out on the host
    run(list(lens), {t: (torch.randn(n, args.dim, generator=g) * 0.5).to(torch.float16) for t, n in lens.items()})
    for step in range(4):
        ids = list(lens)
        if step == 1:
            handles = mb.offload(["b"])            # copy_gpu_to_cpu + free, the reference's loop
            mgr.synchronize()
            ids.remove("b")
        if step == 2:
            mb.reload(["b"], handles)              # copy_cpu_to_gpu into other pages
            mgr.synchronize()
        run(ids, {t: (torch.randn(1, args.dim, generator=g) * 0.5).to(torch.float16) for t in ids})
    assert worst <= 3e-2, f"relative max-abs error {worst} against the dense fp32 blocks"
    from deserve_b200 import _lib

    assert _lib.read_device_status() == 0
    mb.cancel(list(lens))
    assert not mb.ongoing_paged_kvcaches and pool.num_avails == 40 + 6  # every page is back
