"""Parity of the CUDA path (through the C ABI) with the CPU oracle on the same
seeded inputs. Data movement is compared bit for bit; attention within the
stated tolerance of an fp32 reference (2e-2 max-abs for 16-bit types, the bound
the target specification gives; 2e-5 for fp32)."""
import numpy as np
import pytest
import torch

import deserve_b200 as dk
from deserve_b200 import _lib, ops
from helpers import random_descriptors, to_device
from oracle import kv_math

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = {torch.float32: 2e-5, torch.float16: 2e-2, torch.bfloat16: 2e-2}


def _pages(pool_pages, ps, hkv, d, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(pool_pages, 2, ps, hkv, d, generator=g) * scale).to(dtype)


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    assert _lib.read_device_status() == 0, "a kernel self-check fired"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hkv,d,ps", [(2, 64, 16), (8, 128, 16), (8, 128, 8), (1, 64, 4)])
def test_append_bit_exact(dtype, hkv, d, ps):
    new = [1, 5, 1, 33, 2, 1, 64]
    desc, pool_pages = random_descriptors(11, len(new), 1, 200, ps, new_tokens=new)
    pages_cpu = _pages(pool_pages, ps, hkv, d, dtype, 1)
    nnz = int(desc["indptr"][-1])
    g = torch.Generator().manual_seed(2)
    k = torch.randn(nnz, hkv, d, generator=g).to(dtype)
    v = torch.randn(nnz, hkv, d, generator=g).to(dtype)
    pages_gpu = pages_cpu.to(DEV)
    dd = to_device(desc, DEV)
    dk.append_paged_kv_cache(k.to(DEV), v.to(DEV), dd["indptr"], pages_gpu, dd["kv_page_indices"],
                             dd["kv_page_indptr"], dd["kv_last_page_lens"])
    kv_math.append_paged(pages_cpu, k, v, desc, ps)
    assert torch.equal(pages_gpu.cpu().view(torch.uint8), pages_cpu.view(torch.uint8))


def test_append_from_strided_projection_output():
    """K and V as column slices of one fused projection output (token stride
    larger than a row), the shape the attention layer hands over."""
    hkv, d, ps = 8, 128, 16
    desc, pool_pages = random_descriptors(5, 9, 20, 300, ps)
    pages_cpu = _pages(pool_pages, ps, hkv, d, torch.bfloat16, 3)
    g = torch.Generator().manual_seed(4)
    fused = torch.randn(9, 3 * hkv * d, generator=g).to(torch.bfloat16)
    fused_gpu = fused.to(DEV)
    k_gpu = fused_gpu[:, hkv * d : 2 * hkv * d].unflatten(1, (hkv, d))
    v_gpu = fused_gpu[:, 2 * hkv * d :].unflatten(1, (hkv, d))
    pages_gpu = pages_cpu.to(DEV)
    dd = to_device(desc, DEV)
    dk.append_paged_kv_cache(k_gpu, v_gpu, dd["indptr"], pages_gpu, dd["kv_page_indices"], dd["kv_page_indptr"],
                             dd["kv_last_page_lens"])
    kv_math.append_paged(pages_cpu, fused[:, hkv * d : 2 * hkv * d].reshape(9, hkv, d),
                         fused[:, 2 * hkv * d :].reshape(9, hkv, d), desc, ps)
    assert torch.equal(pages_gpu.cpu().view(torch.uint8), pages_cpu.view(torch.uint8))


def _decode_case(seed, batch, lo, hi, hq, hkv, d, ps, dtype, scale=0.5):
    desc, pool_pages = random_descriptors(seed, batch, lo, hi, ps)
    pages_cpu = _pages(pool_pages, ps, hkv, d, dtype, seed + 100, scale)
    g = torch.Generator().manual_seed(seed + 200)
    q = torch.randn(batch, hq, d, generator=g).to(dtype)
    want = kv_math.paged_attention(q, pages_cpu, desc, ps, causal=False)
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=DEV)
    wrapper = dk.BatchDecodeWithPagedKVCacheWrapper(ws)
    dd = to_device(desc, DEV)
    wrapper.begin_forward(dd["kv_page_indptr"], dd["kv_page_indices"], dd["kv_last_page_lens"], hq, hkv, d, ps,
                          data_type=dtype, indptr_host=desc["kv_page_indptr"])
    got = wrapper.forward(q.to(DEV), pages_cpu.to(DEV))
    wrapper.end_forward()
    assert got.dtype == dtype and got.shape == (batch, hq, d)
    err = (got.float().cpu() - want).abs().max().item()
    return err, wrapper


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,d,ps", [(8, 2, 64, 16), (32, 8, 128, 16), (64, 8, 128, 16), (32, 8, 128, 8),
                                         (8, 8, 64, 16), (4, 2, 128, 4), (16, 1, 128, 16), (32, 32, 64, 16),
                                         (64, 2, 64, 16), (24, 4, 128, 32), (12, 4, 64, 16)])
def test_decode_attention_parity(dtype, hq, hkv, d, ps):
    err, _ = _decode_case(7, 13, 1, 700, hq, hkv, d, ps, dtype)
    assert err <= TOL[dtype], f"max-abs error {err}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_attention_split_kv_and_merge(dtype):
    """Few long sequences: every request is split into several work items and
    folded by the merge kernel."""
    err, wrapper = _decode_case(9, 3, 3000, 4100, 32, 8, 128, 16, dtype)
    plan = wrapper._plan_host
    assert plan[2] > 0 and plan[1] > 3, "the case must exercise split-KV"
    assert err <= TOL[dtype], f"max-abs error {err}"


def test_decode_edge_lengths():
    """Lengths that end exactly on, one before and one after a page boundary."""
    ps, hq, hkv, d = 16, 8, 2, 64
    lens = np.array([1, 15, 16, 17, 31, 32, 33, 256, 257])
    n_pages = (lens + ps - 1) // ps
    total = int(n_pages.sum())
    desc = {
        "indptr": np.arange(len(lens) + 1, dtype=np.int32),
        "kv_page_indices": np.random.default_rng(0).permutation(total + 5)[:total].astype(np.int32),
        "kv_page_indptr": np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32),
        "kv_last_page_lens": ((lens - 1) % ps + 1).astype(np.int32),
    }
    pages_cpu = _pages(total + 5, ps, hkv, d, torch.float32, 1)
    pages_cpu[torch.rand(pages_cpu.shape) < 0.01] = float("nan")  # stale slots must never leak ...
    for i in range(len(lens)):                                     # ... so clean only the live tokens
        for t in range(lens[i]):
            pg = desc["kv_page_indices"][desc["kv_page_indptr"][i] + t // ps]
            pages_cpu[pg, :, t % ps] = torch.nan_to_num(pages_cpu[pg, :, t % ps], nan=0.25)
    q = torch.randn(len(lens), hq, d, generator=torch.Generator().manual_seed(3))
    want = kv_math.paged_attention(q, pages_cpu, desc, ps, causal=False)
    assert not want.isnan().any()
    plan = np.zeros(ops.plan_capacity(len(lens)), dtype=np.int32)
    used, ws_bytes = ops.make_decode_plan(desc["kv_page_indptr"], hq, hkv, d, ps, torch.float32, 148, plan)
    dd = to_device(desc, DEV)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=DEV)
    got = ops.paged_decode(q.to(DEV), pages_cpu.to(DEV), dd["kv_page_indices"], dd["kv_page_indptr"],
                           dd["kv_last_page_lens"], plan, torch.from_numpy(plan[:used]).to(DEV), ws)
    assert (got.cpu() - want).abs().max().item() <= 2e-5


def test_decode_lse_output():
    ps, hq, hkv, d = 16, 8, 2, 64
    desc, pool_pages = random_descriptors(21, 6, 5, 900, ps)
    pages_cpu = _pages(pool_pages, ps, hkv, d, torch.float32, 5, 0.5)
    q = torch.randn(6, hq, d, generator=torch.Generator().manual_seed(6))
    plan = np.zeros(ops.plan_capacity(6), dtype=np.int32)
    used, ws_bytes = ops.make_decode_plan(desc["kv_page_indptr"], hq, hkv, d, ps, torch.float32, 148, plan)
    dd = to_device(desc, DEV)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=DEV)
    lse = torch.empty(6, hq, dtype=torch.float32, device=DEV)
    ops.paged_decode(q.to(DEV), pages_cpu.to(DEV), dd["kv_page_indices"], dd["kv_page_indptr"],
                     dd["kv_last_page_lens"], plan, torch.from_numpy(plan[:used]).to(DEV), ws, lse=lse)
    for i in range(6):
        k, _ = kv_math.gather_kv(pages_cpu, desc, i, ps)
        s = torch.einsum("hd,thd->ht", q[i], k.repeat_interleave(hq // hkv, dim=1)) / d ** 0.5
        torch.testing.assert_close(lse[i].cpu(), torch.logsumexp(s, dim=-1), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_rope_parity(dtype):
    hq, hkv, d = 8, 2, 128
    new = [1, 40, 3, 1]
    desc, _ = random_descriptors(31, 4, 50, 3000, 16, new_tokens=new)
    nnz = int(desc["indptr"][-1])
    g = torch.Generator().manual_seed(8)
    q = torch.randn(nnz, hq, d, generator=g).to(dtype)
    k = torch.randn(nnz, hkv, d, generator=g).to(dtype)
    pos = kv_math.token_positions(desc)
    want_q, want_k = kv_math.apply_rope(q, pos, 500000.0), kv_math.apply_rope(k, pos, 500000.0)
    dd = to_device(desc, DEV)
    got_q, got_k = dk.apply_rope(q.to(DEV), k.to(DEV), dd["indptr"], dd["offsets"], interleave=True, rope_theta=500000)
    # fp32: the angle pos*inv_freq is the same fp32 product on both sides; sin/cos
    # differ by an ulp or two between libm and CUDA. 16-bit: one rounding step.
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (got_q.float().cpu() - want_q.float()).abs().max().item() <= tol
    assert (got_k.float().cpu() - want_k.float()).abs().max().item() <= tol


def test_config1_decode_loop_bit_exact_pages():
    """The CPU-reference configuration: 2 layers, 8 q / 2 kv heads, head_dim 64, fp32, page 16,
    4 sequences with context U[100,300] from seed 0, 32 decode steps. Page
    contents are compared bit for bit after every step, attention to fp32."""
    L, hq, hkv, d, ps, B, steps = 2, 8, 2, 64, 16, 4, 32
    g = torch.Generator().manual_seed(0)
    ctx_lens = torch.randint(100, 301, (B,), generator=g).tolist()
    pool = dk.GpuPagePool(L, 128, ps, DEV, torch.float32, n_kv_heads=hkv, head_dim=d)
    pta = dk.PageTableAllocator(B, 4096, ps, DEV)
    from oracle.paged_alloc import OracleKVCache, OraclePagePool, OraclePageTables
    from oracle.descriptors import OracleTask, build_descriptors
    o_pool, o_tab = OraclePagePool(128, ps), OraclePageTables(B, 4096, ps)
    o_pages = torch.zeros(L, 128, 2, ps, hkv, d)
    pool.pages.zero_()
    tasks = [dk.TaskData.empty(f"t{i}", n) for i, n in enumerate(ctx_lens)]
    caches = [dk.PagedKVCache.empty(pta, pool) for _ in range(B)]
    o_tasks = [OracleTask(initial_seqlen=n) for n in ctx_lens]
    o_caches = [OracleKVCache(o_tab, o_pool) for _ in range(B)]
    ws = torch.empty(16 << 20, dtype=torch.uint8, device=DEV)
    wrapper = dk.BatchDecodeWithPagedKVCacheWrapper(ws)
    # prefill the context through the append path (whole prompt as one chunk)
    for t, ot in zip(tasks, o_tasks):
        t.init(t.initial_seqlen)
        ot.init(ot.initial_seqlen)
    for step in range(steps + 1):
        ctx = dk.FlashDecodeCtx.init_paged_decode_ctx(tasks, caches, wrapper)
        o_desc = build_descriptors(o_tasks, o_caches, ps)
        for key in ("indptr", "kv_page_indices", "kv_page_indptr", "kv_last_page_lens", "offsets"):
            assert getattr(ctx, key).cpu().numpy().tolist() == o_desc[key].tolist()
        nnz = int(o_desc["indptr"][-1])
        if step > 0:
            wrapper.begin_forward(ctx.kv_page_indptr, ctx.kv_page_indices, ctx.kv_last_page_lens, hq, hkv, d, ps,
                                  data_type=torch.float32, indptr_host=ctx.host["kv_page_indptr"])
        for layer in range(L):
            k = torch.randn(nnz, hkv, d, generator=g)
            v = torch.randn(nnz, hkv, d, generator=g)
            q = torch.randn(nnz, hq, d, generator=g)
            pages = pool.get_layered_pages(layer)
            dk.append_paged_kv_cache(k.to(DEV), v.to(DEV), ctx.indptr, pages, ctx.kv_page_indices,
                                     ctx.kv_page_indptr, ctx.kv_last_page_lens)
            kv_math.append_paged(o_pages[layer], k, v, o_desc, ps)
            if step > 0:
                got = wrapper.forward(q.to(DEV), pages)
                want = kv_math.paged_attention(q, o_pages[layer], o_desc, ps, causal=False)
                assert (got.cpu() - want).abs().max().item() <= 2e-5
        if step > 0:
            wrapper.end_forward()
        assert torch.equal(pool.pages.cpu().view(torch.uint8), o_pages.view(torch.uint8)), f"pages differ at step {step}"
        for t, ot in zip(tasks, o_tasks):
            t.step()
            ot.step()
    assert [t.start_pos for t in tasks] == [n + steps for n in ctx_lens]


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier nobody completes runs out of polls, the kernel returns, the status word
    says so and the device keeps working (no trap, no hang)."""
    assert _lib.read_device_status() == 0
    _lib.check(_lib.lib.dsv_selftest_wait_timeout(2000, _lib.current_stream_ptr(DEV)))
    assert _lib.read_device_status() == 4          # wait timeout, cleared by the read
    assert _lib.read_device_status() == 0
    x = torch.arange(8, device=DEV)
    assert int(x.sum()) == 28                      # the context is still usable


@pytest.mark.parametrize("name,batch,lo,hi,hq,hkv", [("llama3-8b decode step", 256, 512, 4096, 32, 8),
                                                    ("llama3-70b head shape", 128, 512, 768, 64, 8)])
def test_decode_at_benchmark_size_matches_oracle(name, batch, lo, hi, hq, hkv):
    """One layer of the benchmark's own decode batch — 256 sequences with contexts U[512, 4096] on a
    seeded permutation of a 1.25x pool, bf16, the real split-KV plan with its partial-state slots —
    and the 70B head shape (GQA group 8) at microbatch size 128, against the fp32 oracle."""
    d, ps, dtype = 128, 16, torch.bfloat16
    desc, pool_pages = random_descriptors(0, batch, lo, hi, ps)
    g = torch.Generator().manual_seed(2)
    pages_cpu = (torch.randn(pool_pages, 2, ps, hkv, d, generator=g) * 0.5).to(dtype)
    q = torch.randn(batch, hq, d, generator=g).to(dtype)
    k = (torch.randn(batch, hkv, d, generator=g) * 0.5).to(dtype)
    v = (torch.randn(batch, hkv, d, generator=g) * 0.5).to(dtype)
    ws = torch.empty(128 << 20, dtype=torch.uint8, device=DEV)
    wrapper = dk.BatchDecodeWithPagedKVCacheWrapper(ws)
    dd = to_device(desc, DEV)
    pages = pages_cpu.to(DEV)
    dk.append_paged_kv_cache(k.to(DEV), v.to(DEV), dd["indptr"], pages, dd["kv_page_indices"], dd["kv_page_indptr"],
                             dd["kv_last_page_lens"])
    wrapper.begin_forward(dd["kv_page_indptr"], dd["kv_page_indices"], dd["kv_last_page_lens"], hq, hkv, d, ps,
                          data_type=dtype, indptr_host=desc["kv_page_indptr"])
    got = wrapper.forward(q.to(DEV), pages).float().cpu()
    n_items, n_slots = int(wrapper._plan_host[1]), int(wrapper._plan_host[2])
    wrapper.end_forward()
    kv_math.append_paged(pages_cpu, k, v, desc, ps)
    assert torch.equal(pages.cpu().view(torch.uint8), pages_cpu.view(torch.uint8)), "pages differ after the append"
    want = kv_math.paged_attention(q, pages_cpu, desc, ps, causal=False)
    err = (got - want).abs().max().item()
    assert err <= 2e-2, f"{name}: max-abs error {err}"
    if hi > 2048:
        assert n_items > batch and n_slots > 0, "the benchmark batch must be split over more items than requests"
