"""dsv_paged_decode_static: the decode entry point for hosts that cannot
allocate device memory (its split-KV scratch is a fixed array inside the
library). Called through the C ABI and compared with dsv_paged_decode and with
the CPU oracle on two calls in a row; the second call uses other inputs and a
plan with fewer partial states, so stale scratch contents from the first call
are still in the array. The amount of device memory in use (the driver's count,
and torch's) must be the same before and after a call.

Collected last (file name) so that a run stopping at the first failure has
already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

from deserve_b200 import _lib, ops
from helpers import random_descriptors, to_device
from oracle import kv_math

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _case(seed, batch, lo, hi, hq, hkv, d, ps, dtype):
    desc, pool_pages = random_descriptors(seed, batch, lo, hi, ps)
    g = torch.Generator().manual_seed(seed)
    pages = (torch.randn(pool_pages, 2, ps, hkv, d, generator=g) * 0.5).to(dtype).to(DEV)
    q = torch.randn(batch, hq, d, generator=g).to(dtype).to(DEV)
    plan = np.zeros(ops.plan_capacity(batch), dtype=np.int32)
    used, ws_bytes = ops.make_decode_plan(desc["kv_page_indptr"], hq, hkv, d, ps, dtype, 148, plan)
    return desc, pages, q, plan, used, ws_bytes


def _run_both(seed, batch, lo, hi, hq, hkv, d, ps, dtype):
    desc, pages, q, plan, used, ws_bytes = _case(seed, batch, lo, hi, hq, hkv, d, ps, dtype)
    assert 0 < ws_bytes <= _lib.STATIC_SCRATCH_BYTES, "the case must use split-KV scratch that fits"
    dd = to_device(desc, DEV)
    plan_dev = torch.from_numpy(plan[:used]).to(DEV)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
    want = ops.paged_decode(q, pages, dd["kv_page_indices"], dd["kv_page_indptr"], dd["kv_last_page_lens"], plan,
                            plan_dev, ws)
    got = torch.empty_like(want)

    def call():
        return _lib.lib.dsv_paged_decode_static(
            q.data_ptr(), hq * d, pages.data_ptr(), pages.stride(0), pages.shape[0], dd["kv_page_indices"].data_ptr(),
            dd["kv_page_indptr"].data_ptr(), dd["kv_last_page_lens"].data_ptr(), got.data_ptr(), hq * d, None,
            plan.ctypes.data, plan_dev.data_ptr(), batch, hq, hkv, d, ps, _lib.dtype_code(dtype), 1.0 / d ** 0.5,
            _lib.current_stream_ptr(DEV))

    _lib.check(call())  # on a fresh device this call also resolves the scratch array's address
    torch.cuda.synchronize()
    # the call allocates nothing: neither the driver's free-memory count nor torch's counters move
    free0, _ = torch.cuda.mem_get_info(DEV)
    stats0 = (torch.cuda.memory_allocated(DEV), torch.cuda.memory_reserved(DEV))
    got.zero_()
    _lib.check(call())
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(DEV)
    assert free1 == free0, f"device memory in use changed across the call by {free0 - free1} bytes"
    assert (torch.cuda.memory_allocated(DEV), torch.cuda.memory_reserved(DEV)) == stats0
    oracle = kv_math.paged_attention(q.cpu(), pages.cpu(), desc, ps, causal=False)
    return got, want, oracle


def test_static_scratch_decode_matches_workspace_decode_twice():
    # first call: long sequences, many partial states, bf16 through the TMA kernel
    got, want, oracle = _run_both(41, 5, 2500, 4096, 32, 8, 128, 16, torch.bfloat16)
    assert (got.float() - want.float()).abs().max().item() <= 2e-2
    assert torch.equal(got, want)  # same kernels, same plan: the bits agree too
    assert (got.float().cpu() - oracle).abs().max().item() <= 2e-2  # fp32 oracle, bf16 tolerance
    # second call right after: other shapes and dtype (fp32 CUDA-core kernel), fewer partials
    got, want, oracle = _run_both(42, 3, 900, 1500, 8, 2, 64, 16, torch.float32)
    assert (got - want).abs().max().item() <= 2e-5
    assert torch.equal(got, want)
    assert (got.cpu() - oracle).abs().max().item() <= 2e-5
    assert _lib.read_device_status() == 0


def test_static_scratch_rejects_plans_beyond_its_size():
    hq, hkv, d, ps = 64, 8, 128, 16
    n_pages = np.full(8, 1250)
    indptr = np.concatenate([[0], np.cumsum(n_pages)]).astype(np.int32)
    plan = np.zeros(ops.plan_capacity(8, 2048), dtype=np.int32)
    used, ws_bytes = ops.make_decode_plan(indptr, hq, hkv, d, ps, torch.bfloat16, 2048, plan)
    assert ws_bytes > _lib.STATIC_SCRATCH_BYTES
    dummy = torch.zeros(16, dtype=torch.int32, device=DEV)
    rc = _lib.lib.dsv_paged_decode_static(
        dummy.data_ptr(), hq * d, dummy.data_ptr(), 2 * ps * hkv * d, 4, dummy.data_ptr(), dummy.data_ptr(),
        dummy.data_ptr(), dummy.data_ptr(), hq * d, None, plan.ctypes.data, dummy.data_ptr(), 8, hq, hkv, d, ps,
        _lib.DSV_BF16, 0.1, None)
    assert rc == _lib.E_WORKSPACE
    assert "built-in scratch" in _lib.last_error()
