"""Results recorded from flashinfer itself on a B200 (tests/golden/make_flashinfer_golden.py)
for the operators the reference reaches only through that library: ragged append,
paged decode attention, causal paged prefill attention, rotary embedding, RMSNorm.
CPU tests pin the oracle to those results; GPU tests hold the CUDA path to the same
numbers. Integer work (append) is compared bit for bit through SHA-256 of the pool;
floating point within the stated tolerance (flashinfer rounds P to 16 bit before
P.V and accumulates in another order than the fp32 oracle)."""
import numpy as np
import pytest
import torch

import helpers
from helpers import FLASHINFER_CASES, flashinfer_case_inputs, flashinfer_golden, lattice, sha
from oracle import kv_math

ATTN_TOL = 2e-2  # max abs on outputs of magnitude <= 2, 16-bit types
LSE_TOL = 2e-3   # natural-log units
LN2 = 0.6931471805599453


def _from_raw16(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(dtype)


def _oracle_lse(c, pages):
    """Natural-log sum-exp of the scaled (and, for prompt chunks, causally masked)
    scores, per new row and q head."""
    step, ps = c["step"], c["ps"]
    out = []
    g = c["hq"] // c["hkv"]
    for i in range(len(step["seqlens"])):
        a, b = int(step["indptr"][i]), int(step["indptr"][i + 1])
        k, _ = kv_math.gather_kv(pages, step, i, ps)
        kf = k.float().repeat_interleave(g, dim=1)
        s = torch.einsum("nhd,thd->nht", c["q"][a:b].float(), kf) / np.sqrt(c["d"])
        n, length = b - a, k.shape[0]
        pos_q = torch.arange(n).view(n, 1, 1) + (length - n)
        s = s.masked_fill(torch.arange(length).view(1, 1, -1) > pos_q, float("-inf"))
        out.append(torch.logsumexp(s, dim=-1))
    return torch.cat(out)


def _oracle_pages(c):
    pages = torch.zeros(c["pool_pages"], 2, c["ps"], c["hkv"], c["d"], dtype=c["dtype"])
    kv_math.append_paged(pages, c["k_prefix"], c["v_prefix"], c["prefix"], c["ps"])
    after_prefix = sha(pages)
    kv_math.append_paged(pages, c["k_new"], c["v_new"], c["step"], c["ps"])
    return pages, after_prefix, sha(pages)


@pytest.mark.parametrize("name", list(FLASHINFER_CASES))
def test_oracle_matches_flashinfer(name):
    arrays, meta = flashinfer_golden()
    c = flashinfer_case_inputs(name)
    pages, h1, h2 = _oracle_pages(c)
    assert h1 == meta["cases"][name]["pages_after_prefix"]
    assert h2 == meta["cases"][name]["pages_after_step"]
    want = _from_raw16(arrays[f"{name}.out"], c["dtype"]).float()
    got = kv_math.paged_attention(c["q"], pages, c["step"], c["ps"], causal=True)
    assert (got - want).abs().max().item() <= ATTN_TOL
    lse = torch.from_numpy(arrays[f"{name}.lse"]) * LN2  # recorded in base 2
    assert (_oracle_lse(c, pages) - lse).abs().max().item() <= LSE_TOL


def test_oracle_rope_matches_flashinfer():
    arrays, meta = flashinfer_golden()
    r = meta["rope"]
    desc = {"indptr": np.array(r["indptr"]), "offsets": np.array(r["offsets"])}
    pos = kv_math.token_positions(desc)
    for dt, tol in (("float16", 4e-3), ("bfloat16", 2 ** -6)):
        dtype = getattr(torch, dt)
        for which in ("q", "k"):
            x = lattice(r[f"{which}_seed"], r[f"{which}_shape"], dtype)
            got = kv_math.apply_rope(x, pos, r["theta"]).float()
            rec = arrays[f"rope_{dt}.{which}"]
            want = _from_raw16(rec, dtype).float()
            # the library evaluates the angle on the fly in fp32; at position 8000 the
            # angle's rounding alone moves the result by ~1e-3 of |x| <= 2 (fp16); in
            # bf16 one ulp of a result in [2, 4)
            assert (got - want).abs().max().item() <= tol


def test_oracle_rmsnorm_matches_flashinfer():
    arrays, meta = flashinfer_golden()
    r = meta["rmsnorm"]
    x = lattice(r["x_seed"], r["shape"], torch.bfloat16)
    w = lattice(r["w_seed"], r["shape"][-1:], torch.bfloat16)
    got = kv_math.rmsnorm(x, w, r["eps"]).float()
    want = _from_raw16(arrays["rmsnorm.out"], torch.bfloat16).float()
    # one bf16 ulp where the two fp32 evaluation orders round differently
    assert ((got - want).abs() <= want.abs() * 2 ** -7 + 1e-6).all()


# ---------------------------------------------------------------- CUDA path
DEV = torch.device("cuda:0")


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(FLASHINFER_CASES))
def test_cuda_path_matches_flashinfer(name):
    import deserve_b200 as dk
    from deserve_b200 import _lib, ops
    arrays, meta = flashinfer_golden()
    c = flashinfer_case_inputs(name)
    hq, hkv, d, ps, dtype = c["hq"], c["hkv"], c["d"], c["ps"], c["dtype"]
    pages = torch.zeros(c["pool_pages"], 2, ps, hkv, d, dtype=dtype, device=DEV)
    pre, step = helpers.to_device(c["prefix"], DEV), helpers.to_device(c["step"], DEV)
    ops.append_paged_kv_cache(c["k_prefix"].to(DEV), c["v_prefix"].to(DEV), pre["indptr"], pages,
                              pre["kv_page_indices"], pre["kv_page_indptr"], pre["kv_last_page_lens"])
    assert sha(pages) == meta["cases"][name]["pages_after_prefix"]
    ops.append_paged_kv_cache(c["k_new"].to(DEV), c["v_new"].to(DEV), step["indptr"], pages,
                              step["kv_page_indices"], step["kv_page_indptr"], step["kv_last_page_lens"])
    assert sha(pages) == meta["cases"][name]["pages_after_step"]
    ws = torch.empty(32 << 20, dtype=torch.uint8, device=DEV)
    q = c["q"].to(DEV)
    if name.startswith("decode"):
        w = dk.BatchDecodeWithPagedKVCacheWrapper(ws)
        w.begin_forward(step["kv_page_indptr"], step["kv_page_indices"], step["kv_last_page_lens"], hq, hkv, d, ps,
                        data_type=dtype)
        got = w.forward(q, pages)
    else:
        w = dk.BatchPrefillWithPagedKVCacheWrapper(ws)
        w.begin_forward(step["indptr"], step["kv_page_indptr"], step["kv_page_indices"], step["kv_last_page_lens"],
                        hq, hkv, d, ps, data_type=dtype)
        got = w.forward(q, pages, causal=True)
    w.end_forward()
    torch.cuda.synchronize()
    want = _from_raw16(arrays[f"{name}.out"], dtype).float()
    assert (got.float().cpu() - want).abs().max().item() <= ATTN_TOL
    assert _lib.read_device_status() == 0


@pytest.mark.gpu
def test_cuda_rope_and_rmsnorm_match_flashinfer():
    from deserve_b200 import ops
    arrays, meta = flashinfer_golden()
    r = meta["rope"]
    indptr = torch.tensor(r["indptr"], dtype=torch.int32, device=DEV)
    offsets = torch.tensor(r["offsets"], dtype=torch.int32, device=DEV)
    for dt, tol in (("float16", 4e-3), ("bfloat16", 2 ** -6)):
        dtype = getattr(torch, dt)
        q = lattice(r["q_seed"], r["q_shape"], dtype).to(DEV)
        k = lattice(r["k_seed"], r["k_shape"], dtype).to(DEV)
        ops.apply_rope_inplace(q, k, indptr, offsets, interleave=True, rope_theta=r["theta"])
        for which, t in (("q", q), ("k", k)):
            rec = arrays[f"rope_{dt}.{which}"]
            want = _from_raw16(rec, dtype).float()
            assert (t.float().cpu() - want).abs().max().item() <= tol
    n = meta["rmsnorm"]
    x = lattice(n["x_seed"], n["shape"], torch.bfloat16).to(DEV)
    w = lattice(n["w_seed"], n["shape"][-1:], torch.bfloat16).to(DEV)
    got = ops.rmsnorm(x, w, n["eps"]).float().cpu()
    want = _from_raw16(arrays["rmsnorm.out"], torch.bfloat16).float()
    assert ((got - want).abs() <= want.abs() * 2 ** -7 + 1e-6).all()
