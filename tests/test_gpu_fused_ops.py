"""RMSNorm, rotary-embedding-fused append and greedy sampling against the oracle."""
import numpy as np
import pytest
import torch

import deserve_b200 as dk
from deserve_b200 import _lib
from helpers import random_descriptors, to_device
from oracle import kv_math

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    assert _lib.read_device_status() == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1.0 / 128), (torch.float16, 1.0 / 1024)])
@pytest.mark.parametrize("rows,dim", [(7, 512), (256, 4096), (3, 8192), (5, 16384), (1, 40)])
def test_rmsnorm(dtype, tol, rows, dim):
    g = torch.Generator().manual_seed(rows * dim)
    x = (torch.randn(rows, dim, generator=g) * 3).to(dtype)
    w = (1 + 0.1 * torch.randn(dim, generator=g)).to(dtype)
    want = kv_math.rmsnorm(x, w, 1e-5)
    got = dk.rmsnorm(x.to(DEV), w.to(DEV), 1e-5).cpu()
    # one rounding step of the output type at most (fp32: summation order)
    assert ((got.float() - want.float()).abs() <= tol * want.float().abs() + 1e-6).all()


def test_rmsnorm_strided_rows_and_in_place():
    x = torch.randn(6, 3 * 256, device=DEV).to(torch.bfloat16)
    view = x[:, 256:512]
    w = torch.ones(256, device=DEV, dtype=torch.bfloat16)
    want = kv_math.rmsnorm(view.cpu(), w.cpu(), 1e-6)
    dk.rmsnorm(view, w, 1e-6, out=view)
    assert ((x[:, 256:512].cpu().float() - want.float()).abs() <= want.float().abs() / 128 + 1e-6).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hq,hkv,d,ps", [(32, 8, 128, 16), (8, 2, 64, 16), (4, 4, 64, 8)])
def test_fused_rope_append_equals_rope_then_append(dtype, hq, hkv, d, ps):
    new = [1, 37, 1, 5, 64]
    desc, pool_pages = random_descriptors(17, len(new), 70, 2500, ps, new_tokens=new)
    nnz = int(desc["indptr"][-1])
    g = torch.Generator().manual_seed(5)
    pages0 = torch.randn(pool_pages, 2, ps, hkv, d, generator=g).to(dtype).to(DEV)
    fused = torch.randn(nnz, (hq + 2 * hkv) * d, generator=g).to(dtype).to(DEV)  # one projection output
    dd = to_device(desc, DEV)

    def split(t):
        return (t[:, : hq * d].unflatten(1, (hq, d)), t[:, hq * d : (hq + hkv) * d].unflatten(1, (hkv, d)),
                t[:, (hq + hkv) * d :].unflatten(1, (hkv, d)))

    # two launches, as the reference does it
    a = fused.clone()
    qa, ka, va = split(a)
    pages_a = pages0.clone()
    dk.apply_rope_inplace(qa, ka, dd["indptr"], dd["offsets"], True, 500000.0)
    dk.append_paged_kv_cache(ka, va, dd["indptr"], pages_a, dd["kv_page_indices"], dd["kv_page_indptr"],
                             dd["kv_last_page_lens"])
    # one launch
    b = fused.clone()
    qb, kb, vb = split(b)
    pages_b = pages0.clone()
    dk.rope_append_paged_kv_cache(qb, kb, vb, dd["indptr"], dd["offsets"], pages_b, dd["kv_page_indices"],
                                  dd["kv_page_indptr"], dd["kv_last_page_lens"], 500000.0)
    assert torch.equal(pages_a.view(torch.uint8), pages_b.view(torch.uint8))
    assert torch.equal(qa.contiguous().view(torch.uint8), qb.contiguous().view(torch.uint8))
    assert torch.equal(kb, split(fused)[1]) and torch.equal(vb, split(fused)[2])  # k, v inputs untouched
    # and against the oracle: rotate on the CPU, append by index assignment
    pos = kv_math.token_positions(desc)
    k_rot = kv_math.apply_rope(split(fused.cpu())[1], pos, 500000.0)
    pages_c = pages0.cpu().clone()
    kv_math.append_paged(pages_c, k_rot, split(fused.cpu())[2], desc, ps)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (pages_b.cpu().float() - pages_c.float()).abs().max().item() <= tol
    # V is pure data movement: bit-exact against the oracle
    assert torch.equal(pages_b.cpu()[:, 1].contiguous().view(torch.uint8), pages_c[:, 1].contiguous().view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,vocab", [(256, 128256), (3, 640), (1, 32000), (5, 1001)])
def test_greedy_sample(dtype, rows, vocab):
    g = torch.Generator().manual_seed(vocab)
    vs = (vocab + 7) // 8 * 8
    padded = torch.randn(rows, vs, generator=g).to(dtype)  # rows padded to a 16-byte multiple, as a GEMM output is
    logits = padded[:, :vocab]
    logits[0, vocab // 2] = logits[0].max()      # a tie: the lower index must win
    lo = int(torch.argmax((logits[0] == logits[0].max()).to(torch.int8)))
    got = dk.greedy_sample(padded.to(DEV)[:, :vocab]).cpu()
    want = kv_math.greedy_tokens(logits)
    assert got.dtype == torch.int32
    assert torch.equal(got[1:], want[1:]) and int(got[0]) == lo


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1.0 / 128), (torch.float16, 1.0 / 1024)])
@pytest.mark.parametrize("rows,ffn", [(5, 1024), (128, 28672), (1, 8)])
def test_silu_mul(dtype, tol, rows, ffn):
    """The SwiGLU middle on a fused gate|up projection output against the reference's two torch
    statements (deserve_worker/model/layer/linear.py:121-123) on the CPU: at most one rounding step
    of the output type apart (the silu itself is evaluated by another exp)."""
    g = torch.Generator().manual_seed(rows + ffn)
    gu = (torch.randn(rows, 2 * ffn, generator=g) * 2).to(dtype)
    want = torch.nn.functional.silu(gu[:, :ffn].float()).to(dtype).float() * gu[:, ffn:].float()
    got = dk.ops.silu_mul(gu.to(DEV)).cpu().float()
    assert got.shape == (rows, ffn)
    assert ((got - want).abs() <= 2 * tol * want.abs() + 1e-6).all()
    # a strided input (the gate|up block as a column slice of a wider tensor)
    wide = torch.zeros(rows, 2 * ffn + 16, dtype=dtype, device=DEV)
    wide[:, : 2 * ffn] = gu.to(DEV)
    got2 = dk.ops.silu_mul(wide[:, : 2 * ffn]).cpu().float()
    assert torch.equal(got, got2)
