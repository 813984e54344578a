"""Append-scatter, page gather, rotary embedding and dense attention on CPU."""
from __future__ import annotations

import math

import numpy as np
import torch


def kv_lengths(desc, page_size: int) -> np.ndarray:
    """Post-append length of every request implied by the descriptors
    (deserve_worker/model/context/flash.py:35-37 inverted)."""
    n_pages = np.diff(desc["kv_page_indptr"])
    return (n_pages - 1) * page_size + desc["kv_last_page_lens"]


def append_paged(pages_layer: torch.Tensor, k: torch.Tensor, v: torch.Tensor, desc, page_size: int) -> None:
    """Semantics of the call at deserve_worker/model/layer/attention.py:174-183:
    the n_i new rows of request i fill the LAST n_i token slots of its page list
    (descriptors already include the new tokens). pages_layer:
    [P, 2, page_size, Hkv, D]; k, v: [nnz, Hkv, D]. Pure index assignment."""
    lens = kv_lengths(desc, page_size)
    indptr, kvp, idx = desc["indptr"], desc["kv_page_indptr"], desc["kv_page_indices"]
    for i in range(len(lens)):
        n_i = int(indptr[i + 1] - indptr[i])
        for j in range(n_i):
            t = int(lens[i]) - n_i + j
            page = int(idx[kvp[i] + t // page_size])
            pages_layer[page, 0, t % page_size] = k[indptr[i] + j]
            pages_layer[page, 1, t % page_size] = v[indptr[i] + j]


def gather_kv(pages_layer: torch.Tensor, desc, i: int, page_size: int):
    """K and V of request i in token order, read through its page list:
    [len_i, Hkv, D] each."""
    kvp, idx = desc["kv_page_indptr"], desc["kv_page_indices"]
    ids = torch.as_tensor(np.asarray(idx[kvp[i] : kvp[i + 1]], dtype=np.int64))
    length = int(kv_lengths(desc, page_size)[i])
    blk = pages_layer[ids]  # [n, 2, ps, Hkv, D]
    k = blk[:, 0].reshape(-1, *blk.shape[3:])[:length]
    v = blk[:, 1].reshape(-1, *blk.shape[3:])[:length]
    return k, v


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal_tail: bool) -> torch.Tensor:
    """The math of deserve_worker/model/layer/attention.py:237-266 for one
    request in fp32: GQA by repeating kv heads (attention.py:75-84), scores
    q.k / sqrt(D) (attention.py:249), optional causal mask, fp32 softmax
    (attention.py:254), P.V. q: [n, Hq, D]; k, v: [len, Hkv, D]. With
    causal_tail, q row j sees kv positions <= len - n + j (the mask of
    attention.py:216-221 shifted so that the last q row sees everything)."""
    n, hq, d = q.shape
    length, hkv, _ = k.shape
    rep = hq // hkv
    qf = q.float().transpose(0, 1)  # [Hq, n, D]
    kf = k.float().repeat_interleave(rep, dim=1).transpose(0, 1)  # [Hq, len, D]
    vf = v.float().repeat_interleave(rep, dim=1).transpose(0, 1)
    scores = torch.matmul(qf, kf.transpose(1, 2)) / math.sqrt(d)
    if causal_tail and n > 1:
        pos_q = torch.arange(n).unsqueeze(1) + (length - n)
        pos_k = torch.arange(length).unsqueeze(0)
        scores = scores.masked_fill((pos_k > pos_q).unsqueeze(0), float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.matmul(probs, vf).transpose(0, 1).contiguous()  # [n, Hq, D]


def paged_attention(q: torch.Tensor, pages_layer: torch.Tensor, desc, page_size: int, causal: bool) -> torch.Tensor:
    """Ragged batch: request i's rows q[indptr[i]:indptr[i+1]] against its paged
    K/V. Decode is the n_i = 1 case (no mask needed). fp32 result [nnz, Hq, D]."""
    out = torch.zeros(q.shape, dtype=torch.float32)
    indptr = desc["indptr"]
    for i in range(len(indptr) - 1):
        a, b = int(indptr[i]), int(indptr[i + 1])
        if b == a:
            continue
        k, v = gather_kv(pages_layer, desc, i, page_size)
        out[a:b] = dense_attention(q[a:b], k, v, causal)
    return out


def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """deserve_worker/execution/exec.py:44: 1 / theta**(arange(0,D,2)/D), fp32."""
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))


def apply_rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """deserve_worker/model/layer/attention.py:45-72 with the table of
    exec.py:44-52: adjacent pairs (2i, 2i+1) are a complex number multiplied by
    exp(i * pos * inv_freq[i]); fp32 math, result cast back. x: [nnz, H, D]."""
    ang = torch.outer(positions.float(), rope_inv_freq(x.shape[-1], theta))  # [nnz, D/2]
    cis = torch.polar(torch.ones_like(ang), ang).unsqueeze(1)  # [nnz, 1, D/2]
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    return torch.view_as_real(xc * cis).flatten(-2).to(x.dtype)


def token_positions(desc) -> torch.Tensor:
    """Position of every ragged row: offsets[i] + j (the indptr/offsets pair the
    reference hands to apply_rope, attention.py:166-173)."""
    pos = []
    for i in range(len(desc["offsets"])):
        n = int(desc["indptr"][i + 1] - desc["indptr"][i])
        pos.extend(int(desc["offsets"][i]) + j for j in range(n))
    return torch.tensor(pos, dtype=torch.int64)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """deserve_worker/model/layer/norm.py:18-19 (x * rsqrt(mean(x^2) + eps)) times the
    weight, evaluated in fp32 and rounded once to x's type, which is what the fused
    call at norm.py:34 computes."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def greedy_tokens(logits: torch.Tensor) -> torch.Tensor:
    """deserve_worker/layer_storage.py:250: argmax of each row (first maximum)."""
    return torch.argmax(logits.float(), dim=-1).to(torch.int32)
