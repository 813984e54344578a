"""Record results of flashinfer itself for the operators the reference reaches only
through that library (deserve_worker/model/layer/attention.py:163-193,
deserve_worker/execution/exec.py:184-242, deserve_worker/model/layer/norm.py:34):
ragged append into pages, paged decode attention, causal paged prefill attention,
in-place rotary embedding and RMSNorm. Needs a GPU and the flashinfer package; run as

    python tests/golden/make_flashinfer_golden.py OUT_DIR

and copy OUT_DIR/flashinfer_golden.{npz,json} beside this file. Inputs are not
stored: tests rebuild them from the seeds in tests/helpers.py (FLASHINFER_CASES).
16-bit results are stored as their raw bit patterns (uint16)."""
from __future__ import annotations

import hashlib
import json
import sys
import traceback
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import helpers  # noqa: E402

DEV = torch.device("cuda:0")


def raw16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def dev(desc: dict) -> dict:
    return {k: torch.from_numpy(np.ascontiguousarray(v)).to(DEV) for k, v in desc.items()}


def append(fi, k, v, desc, pages, ps):
    """The reference's append_paged_kv_cache(k, v, indptr, pages, indices, indptr,
    last_page_len) in the library's current spelling (per-row batch index and
    position instead of the ragged indptr)."""
    if k.shape[0] == 0:
        return
    d = dev(desc)
    n_pages = d["kv_page_indptr"][1:] - d["kv_page_indptr"][:-1]
    seq_lens = torch.where(n_pages > 0, (n_pages - 1) * ps + d["kv_last_page_lens"], torch.zeros_like(n_pages))
    bi, pos = fi.get_batch_indices_positions(d["indptr"], seq_lens.to(torch.int32), k.shape[0])
    fi.append_paged_kv_cache(k, v, bi, pos, pages, d["kv_page_indices"], d["kv_page_indptr"],
                             d["kv_last_page_lens"], kv_layout="NHD")


def attention_case(fi, name, arrays, meta):
    c = helpers.flashinfer_case_inputs(name)
    hq, hkv, d, ps, dtype = c["hq"], c["hkv"], c["d"], c["ps"], c["dtype"]
    pages = torch.zeros(c["pool_pages"], 2, ps, hkv, d, dtype=dtype, device=DEV)
    append(fi, c["k_prefix"].to(DEV), c["v_prefix"].to(DEV), c["prefix"], pages, ps)
    torch.cuda.synchronize()
    info = {"pages_after_prefix": sha(pages)}
    append(fi, c["k_new"].to(DEV), c["v_new"].to(DEV), c["step"], pages, ps)
    torch.cuda.synchronize()
    info["pages_after_step"] = sha(pages)
    s = dev(c["step"])
    ws = torch.empty(128 << 20, dtype=torch.uint8, device=DEV)
    q = c["q"].to(DEV)
    if name.startswith("decode"):
        w = fi.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
        w.plan(s["kv_page_indptr"], s["kv_page_indices"], s["kv_last_page_lens"], hq, hkv, d, ps,
               pos_encoding_mode="NONE", q_data_type=dtype, kv_data_type=dtype)
        out, lse = w.run(q, pages, return_lse=True)
    else:
        w = fi.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
        w.plan(s["indptr"], s["kv_page_indptr"], s["kv_page_indices"], s["kv_last_page_lens"], hq, hkv, d, ps,
               causal=True, pos_encoding_mode="NONE", q_data_type=dtype, kv_data_type=dtype)
        out, lse = w.run(q, pages, return_lse=True)
    torch.cuda.synchronize()
    arrays[f"{name}.out"] = raw16(out)
    arrays[f"{name}.lse"] = lse.float().cpu().numpy()
    meta["cases"][name] = info


def rope_case(fi, arrays, meta):
    """apply_rope_inplace(xq, xk, indptr, offsets, interleave=True, rope_theta=500000)
    as called at deserve_worker/model/layer/attention.py:163-173."""
    for dt in ("bfloat16", "float16"):  # the library's rotary kernel takes 16-bit tensors only
        dtype = getattr(torch, dt)
        indptr = torch.tensor([0, 1, 6, 7, 40], dtype=torch.int32, device=DEV)
        offsets = torch.tensor([0, 100, 4095, 8000], dtype=torch.int32, device=DEV)
        q = helpers.lattice(201, (40, 8, 128), dtype).to(DEV)
        k = helpers.lattice(202, (40, 2, 128), dtype).to(DEV)
        fi.apply_rope_inplace(q, k, indptr, offsets, interleave=True, rope_theta=500000)
        torch.cuda.synchronize()
        arrays[f"rope_{dt}.q"], arrays[f"rope_{dt}.k"] = raw16(q), raw16(k)
    meta["rope"] = {"indptr": [0, 1, 6, 7, 40], "offsets": [0, 100, 4095, 8000], "theta": 500000,
                    "q_seed": 201, "k_seed": 202, "q_shape": [40, 8, 128], "k_shape": [40, 2, 128]}


def rmsnorm_case(fi, arrays, meta):
    """flashinfer.norm.rmsnorm(x, weight, eps) as called at
    deserve_worker/model/layer/norm.py:34."""
    x = helpers.lattice(301, (12, 4096), torch.bfloat16).to(DEV)
    w = helpers.lattice(302, (4096,), torch.bfloat16).to(DEV)
    out = fi.norm.rmsnorm(x, w, 1e-5)
    torch.cuda.synchronize()
    arrays["rmsnorm.out"] = raw16(out)
    meta["rmsnorm"] = {"x_seed": 301, "w_seed": 302, "shape": [12, 4096], "eps": 1e-5}


def main():
    out_dir = Path(sys.argv[1])
    out_dir.mkdir(parents=True, exist_ok=True)
    log = open(out_dir / "flashinfer_golden.log", "w")
    import flashinfer as fi
    arrays, meta = {}, {
        "flashinfer": fi.__version__, "torch": torch.__version__, "gpu": torch.cuda.get_device_name(0),
        "cases": {}, "failed": [],
    }
    jobs = [(n, lambda n=n: attention_case(fi, n, arrays, meta)) for n in helpers.FLASHINFER_CASES]
    jobs += [("rope", lambda: rope_case(fi, arrays, meta)), ("rmsnorm", lambda: rmsnorm_case(fi, arrays, meta))]
    for name, job in jobs:
        try:
            job()
            print("ok", name, file=log, flush=True)
        except Exception:
            meta["failed"].append(name)
            print("FAILED", name, file=log)
            traceback.print_exc(file=log)
            log.flush()
    np.savez(out_dir / "flashinfer_golden.npz", **arrays)
    (out_dir / "flashinfer_golden.json").write_text(json.dumps(meta, indent=1))
    print(json.dumps({k: v for k, v in meta.items() if k != "cases"}), file=log, flush=True)


if __name__ == "__main__":
    main()
