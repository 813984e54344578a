"""Operator entry points of the paged KV path, with the call shapes the
reference uses at its flashinfer boundary (deserve_worker/model/layer/
attention.py:166-192, deserve_worker/execution/exec.py:20-22, 184-198,
227-242), implemented by libdeserve_kv.so through ctypes.

All tensors must live on a CUDA device; there is no CPU path.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from . import _lib
from .pinned import COUNTERS as _COUNTERS, ring as _pinned_ring

_PLAN_HEADER = 8


def _i32_dev(t: torch.Tensor, name: str) -> torch.Tensor:
    _lib.require_cuda(t)
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous int32 tensor")
    return t


def _row_stride(t: torch.Tensor, heads: int, dim: int, name: str) -> int:
    """Token stride (elements) of a [nnz, heads, dim] tensor whose heads and dims
    are dense (a plain tensor or a column slice of a fused projection output)."""
    if t.dim() != 3 or t.shape[1] != heads or t.shape[2] != dim:
        raise ValueError(f"{name} must have shape [nnz, {heads}, {dim}], got {tuple(t.shape)}")
    if t.shape[0] > 0 and (t.stride(2) != 1 or t.stride(1) != dim):
        raise ValueError(f"{name}: heads and head_dim must be contiguous")
    return t.stride(0) if t.shape[0] > 1 else heads * dim


def _pages_view(paged_kv_cache: torch.Tensor):
    """[P, 2, page_size, n_kv_heads, head_dim] view of one layer."""
    p = paged_kv_cache
    if p.dim() != 5 or p.shape[1] != 2:
        raise ValueError(f"paged_kv_cache must be [P, 2, page_size, n_kv_heads, head_dim], got {tuple(p.shape)}")
    _, _, ps, hkv, d = p.shape
    if p.stride(4) != 1 or p.stride(3) != d or p.stride(2) != hkv * d or p.stride(1) != ps * hkv * d:
        raise ValueError("paged_kv_cache: a page must be contiguous")
    return ps, hkv, d, p.stride(0)


def append_paged_kv_cache(append_key: torch.Tensor, append_value: torch.Tensor, append_indptr: torch.Tensor,
                          paged_kv_cache: torch.Tensor, kv_indices: torch.Tensor, kv_indptr: torch.Tensor,
                          kv_last_page_len: torch.Tensor) -> None:
    """Scatter the step's new K/V rows into the last n_i token slots of each
    request's page list (the descriptors already include the new tokens)."""
    _lib.require_cuda(append_key, append_value, paged_kv_cache)
    ps, hkv, d, page_stride = _pages_view(paged_kv_cache)
    if append_key.dtype != paged_kv_cache.dtype or append_value.dtype != paged_kv_cache.dtype:
        raise ValueError("append: K/V dtype differs from the page dtype")
    ks = _row_stride(append_key, hkv, d, "append_key")
    vs = _row_stride(append_value, hkv, d, "append_value")
    nnz, batch = append_key.shape[0], kv_last_page_len.shape[0]
    _lib.check(_lib.lib.dsv_append_paged_kv(
        append_key.data_ptr(), append_value.data_ptr(), ks, vs, _i32_dev(append_indptr, "append_indptr").data_ptr(),
        paged_kv_cache.data_ptr(), page_stride, paged_kv_cache.shape[0], _i32_dev(kv_indices, "kv_indices").data_ptr(),
        _i32_dev(kv_indptr, "kv_indptr").data_ptr(), _i32_dev(kv_last_page_len, "kv_last_page_len").data_ptr(),
        batch, nnz, hkv, d, ps, _lib.dtype_code(paged_kv_cache.dtype), _lib.current_stream_ptr(append_key.device)))
    _lib.LAUNCHES[0] += 1


_INV_FREQ: dict[tuple[int, float], torch.Tensor] = {}


def rope_inv_freq(head_dim: int, rope_theta: float) -> torch.Tensor:
    """theta^(-2i/D) evaluated the way the reference's table is
    (deserve_worker/execution/exec.py:44): fp32 torch arithmetic on the host."""
    key = (head_dim, float(rope_theta))
    if key not in _INV_FREQ:
        _INV_FREQ[key] = (1.0 / (float(rope_theta) ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float()
                                                      / head_dim))).contiguous()
    return _INV_FREQ[key]


def apply_rope_inplace(q: torch.Tensor, k: torch.Tensor, indptr: torch.Tensor, offsets: torch.Tensor,
                       interleave: bool = True, rope_theta: float = 500000.0) -> None:
    _lib.require_cuda(q, k)
    if not interleave:
        raise ValueError("only the interleaved (adjacent-pair) rotary layout of the reference is implemented")
    if q.dtype != k.dtype:
        raise ValueError("rope: q and k dtypes differ")
    hq, d = q.shape[1], q.shape[2]
    hkv = k.shape[1]
    qs, ks = _row_stride(q, hq, d, "q"), _row_stride(k, hkv, d, "k")
    _lib.check(_lib.lib.dsv_apply_rope_inplace(
        q.data_ptr(), k.data_ptr(), qs, ks, _i32_dev(indptr, "indptr").data_ptr(),
        _i32_dev(offsets, "offsets").data_ptr(), offsets.shape[0], q.shape[0], hq, hkv, d, float(rope_theta),
        rope_inv_freq(d, rope_theta).data_ptr(), _lib.dtype_code(q.dtype), _lib.current_stream_ptr(q.device)))
    _lib.LAUNCHES[0] += 1


def apply_rope(q: torch.Tensor, k: torch.Tensor, indptr: torch.Tensor, offsets: torch.Tensor,
               interleave: bool = True, rope_theta: float = 500000.0):
    """Rotated copies of ragged q and k; token j of request i sits at position
    offsets[i] + j."""
    q2, k2 = q.clone(), k.clone()
    apply_rope_inplace(q2, k2, indptr, offsets, interleave, rope_theta)
    return q2, k2


def plan_capacity(batch: int, sm_count: int = 148) -> int:
    """int32 entries that a decode plan for `batch` requests can need."""
    items = max(4 * sm_count, batch) + batch
    return _PLAN_HEADER + 4 * items + 2 * batch


def make_decode_plan(kv_indptr_host: np.ndarray, n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int,
                     dtype: torch.dtype, sm_count: int, plan_out: np.ndarray) -> tuple[int, int]:
    """Fill plan_out (int32) with the split-KV schedule; returns (int32 entries
    used, device workspace bytes needed)."""
    kv_indptr_host = np.ascontiguousarray(kv_indptr_host, dtype=np.int32)
    used, ws = ctypes.c_int64(), ctypes.c_int64()
    _lib.check(_lib.lib.dsv_decode_plan(
        kv_indptr_host.ctypes.data, len(kv_indptr_host) - 1, n_q_heads, n_kv_heads, head_dim, page_size,
        _lib.dtype_code(dtype), sm_count, plan_out.ctypes.data, plan_out.size, ctypes.byref(used), ctypes.byref(ws)))
    return used.value, ws.value


def paged_decode(q: torch.Tensor, paged_kv_cache: torch.Tensor, kv_indices: torch.Tensor, kv_indptr: torch.Tensor,
                 kv_last_page_len: torch.Tensor, plan_host: np.ndarray, plan_dev: torch.Tensor,
                 workspace: torch.Tensor | None, out: torch.Tensor | None = None, sm_scale: float | None = None,
                 lse: torch.Tensor | None = None) -> torch.Tensor:
    """Functional form of the decode attention call: every buffer explicit."""
    _lib.require_cuda(q, paged_kv_cache, plan_dev)
    ps, hkv, d, page_stride = _pages_view(paged_kv_cache)
    if q.dtype != paged_kv_cache.dtype:
        raise ValueError("decode: q dtype differs from the page dtype")
    batch, hq = q.shape[0], q.shape[1]
    qs = _row_stride(q, hq, d, "q")
    if out is None:
        out = torch.empty((batch, hq, d), dtype=q.dtype, device=q.device)
    os_ = _row_stride(out, hq, d, "out")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    _lib.check(_lib.lib.dsv_paged_decode(
        q.data_ptr(), qs, paged_kv_cache.data_ptr(), page_stride, paged_kv_cache.shape[0], kv_indices.data_ptr(),
        kv_indptr.data_ptr(),
        kv_last_page_len.data_ptr(), out.data_ptr(), os_, _lib.ptr(lse), plan_host.ctypes.data, plan_dev.data_ptr(),
        _lib.ptr(workspace), 0 if workspace is None else workspace.numel() * workspace.element_size(), batch, hq, hkv,
        d, ps, _lib.dtype_code(q.dtype), float(sm_scale), _lib.current_stream_ptr(q.device)))
    _lib.LAUNCHES[0] += 2 if plan_host[2] > 0 else 1  # the attention kernel, and the merge when requests were split
    return out


class BatchDecodeWithPagedKVCacheWrapper:
    """begin_forward / forward / end_forward object of the reference's decode
    path (exec.py:21, 184-198; attention.py:185). `workspace_buffer` is a uint8
    device tensor owned by the caller: its head holds the device copy of the
    plan, the rest the split-KV partial states."""

    _PLAN_BYTES = 1 << 20

    def __init__(self, workspace_buffer: torch.Tensor, kv_layout: str = "NHD"):
        _lib.require_cuda(workspace_buffer)
        if kv_layout != "NHD":
            raise ValueError("only the NHD page layout of the reference is implemented")
        if workspace_buffer.dtype != torch.uint8 or workspace_buffer.numel() < 2 * self._PLAN_BYTES:
            raise ValueError("workspace_buffer must be a uint8 tensor of at least 2 MiB")
        self._ws = workspace_buffer
        self._sm_count = _lib.device_info()[0]
        self._plan_host: np.ndarray | None = None
        self._plan_pinned: torch.Tensor | None = None
        self._desc = None

    def begin_forward(self, indptr: torch.Tensor, indices: torch.Tensor, last_page_len: torch.Tensor,
                      num_qo_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                      pos_encoding_mode: str = "NONE", data_type=torch.float16, *,
                      indptr_host: np.ndarray | None = None) -> None:
        """Plan the split-KV schedule for this batch. `indptr_host` (the same
        values as `indptr`, in host memory) avoids a device->host copy."""
        if pos_encoding_mode != "NONE":
            raise ValueError("positional encoding inside attention is not part of this path")
        if indptr_host is None:
            indptr_host = indptr.cpu().numpy()
        batch = len(indptr_host) - 1
        cap = plan_capacity(batch, self._sm_count)
        if cap * 4 > self._PLAN_BYTES:
            raise _lib.DeserveKVError(f"decode plan for {batch} requests does not fit the workspace head")
        pinned, slot = _pinned_ring("decode_plan").take(cap)
        plan = pinned.numpy()
        used, ws_bytes = make_decode_plan(indptr_host, num_qo_heads, num_kv_heads, head_dim, page_size,
                                          data_type if isinstance(data_type, torch.dtype) else torch.float16,
                                          self._sm_count, plan)
        if ws_bytes > self._ws.numel() - self._PLAN_BYTES:
            raise _lib.DeserveKVError(f"workspace_buffer too small: split-KV partials need {ws_bytes} bytes")
        self._ws[: used * 4].view(torch.int32).copy_(pinned[:used], non_blocking=True)
        _pinned_ring("decode_plan").done(slot)
        _COUNTERS["h2d_bytes"] += used * 4
        self._plan_pinned, self._plan_host = pinned, plan
        self._desc = (indptr, indices, last_page_len, num_qo_heads, num_kv_heads, head_dim, page_size)

    def forward(self, q: torch.Tensor, paged_kv_cache: torch.Tensor, sm_scale: float | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
        if self._desc is None:
            raise RuntimeError("forward() called outside begin_forward()/end_forward()")
        indptr, indices, last_page_len, hq, hkv, d, ps = self._desc
        if q.dim() == 2:
            q = q.view(-1, hq, d)
        return paged_decode(q, paged_kv_cache, indices, indptr, last_page_len, self._plan_host,
                            self._ws[: self._PLAN_BYTES].view(torch.int32), self._ws[self._PLAN_BYTES :], out,
                            sm_scale)

    def end_forward(self) -> None:
        self._desc = None


_PREFILL_PLAN_HEADER = 12


def prefill_plan_capacity(nnz: int, batch: int, group: int) -> int:
    tq = max(1, 128 // group)
    return _PREFILL_PLAN_HEADER + 4 * (nnz // tq + batch + 1)


def make_prefill_plan(qo_indptr_host: np.ndarray, kv_len_host: np.ndarray, n_q_heads: int, n_kv_heads: int,
                      head_dim: int, page_size: int, dtype: torch.dtype, causal: bool, plan_out: np.ndarray,
                      min_new_tokens: int = 0) -> int:
    """Fill plan_out (int32) with the (request, q tile) work items; returns the int32 entries
    used. Requests with fewer than min_new_tokens new tokens get no item."""
    qo = np.ascontiguousarray(qo_indptr_host, dtype=np.int32)
    kl = np.ascontiguousarray(kv_len_host, dtype=np.int32)
    used = ctypes.c_int64()
    _lib.check(_lib.lib.dsv_prefill_plan(qo.ctypes.data, kl.ctypes.data, len(kl), n_q_heads, n_kv_heads, head_dim,
                                         page_size, _lib.dtype_code(dtype), 1 if causal else 0, int(min_new_tokens),
                                         plan_out.ctypes.data, plan_out.size, ctypes.byref(used)))
    return used.value


def paged_prefill(q: torch.Tensor, qo_indptr: torch.Tensor, paged_kv_cache: torch.Tensor, kv_indices: torch.Tensor,
                  kv_indptr: torch.Tensor, kv_last_page_len: torch.Tensor, plan_host: np.ndarray,
                  plan_dev: torch.Tensor, out: torch.Tensor | None = None, sm_scale: float | None = None,
                  causal: bool = True) -> torch.Tensor:
    """Functional form of the ragged causal prefill attention call: every buffer explicit."""
    _lib.require_cuda(q, paged_kv_cache, plan_dev)
    ps, hkv, d, page_stride = _pages_view(paged_kv_cache)
    if q.dtype != paged_kv_cache.dtype:
        raise ValueError("prefill: q dtype differs from the page dtype")
    nnz, hq = q.shape[0], q.shape[1]
    qs = _row_stride(q, hq, d, "q")
    if out is None:
        out = torch.empty((nnz, hq, d), dtype=q.dtype, device=q.device)
    os_ = _row_stride(out, hq, d, "out")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    _lib.check(_lib.lib.dsv_paged_prefill(
        q.data_ptr(), qs, qo_indptr.data_ptr(), paged_kv_cache.data_ptr(), page_stride, paged_kv_cache.shape[0],
        kv_indices.data_ptr(), kv_indptr.data_ptr(), kv_last_page_len.data_ptr(), out.data_ptr(), os_,
        plan_host.ctypes.data, plan_dev.data_ptr(), kv_last_page_len.shape[0], nnz, hq, hkv, d, ps,
        _lib.dtype_code(q.dtype), float(sm_scale), 1 if causal else 0, _lib.current_stream_ptr(q.device)))
    # one launch for the pair items (clusters of two CTAs), one for the single-CTA items
    _lib.LAUNCHES[0] += int(plan_host[1] > 0) + int(plan_host[8] > 0)
    return out


class BatchPrefillWithPagedKVCacheWrapper:
    """begin_forward / forward / end_forward object of the reference's prefill path
    (exec.py:22, 227-242; attention.py:188-192): ragged causal attention of the
    step's new q rows against the paged K/V, also used for mixed prefill+decode
    batches. In a mixed batch the rows of requests with ONE new token (plain decode
    rows; causal attention of a single last row is unmasked attention) are sent to
    the decode kernel, which streams their K/V at HBM speed, and only the prompt
    chunks go to the tensor-core prefill kernel; both write into the same output.
    The head of `workspace_buffer` holds the device copies of the plans and of the
    decode rows' sub-descriptors, the rest the split-KV partial states."""

    _PLAN_BYTES = 1 << 20
    SPLIT_MIN_KV = 64  # a decode row with at least this many kv tokens makes the second launch worth it

    def __init__(self, workspace_buffer: torch.Tensor, kv_layout: str = "NHD"):
        _lib.require_cuda(workspace_buffer)
        if kv_layout != "NHD":
            raise ValueError("only the NHD page layout of the reference is implemented")
        if workspace_buffer.dtype != torch.uint8 or workspace_buffer.numel() < self._PLAN_BYTES:
            raise ValueError("workspace_buffer must be a uint8 tensor of at least 1 MiB")
        self._ws = workspace_buffer
        # head of the workspace that holds the plans and the decode rows' page lists: an eighth of
        # the buffer, between 1 and 4 MiB (512 decode rows with 8k-token contexts list 266k pages)
        self._PLAN_BYTES = int(min(4 << 20, max(1 << 20, (workspace_buffer.numel() // 8) & ~0xFFFFF)))
        self._sm_count = _lib.device_info()[0]
        self._plan_host: np.ndarray | None = None
        self._pinned = None
        self._desc = None
        self._dec = None

    def begin_forward(self, qo_indptr: torch.Tensor, paged_kv_indptr: torch.Tensor, paged_kv_indices: torch.Tensor,
                      paged_kv_last_page_len: torch.Tensor, num_qo_heads: int, num_kv_heads: int, head_dim: int,
                      page_size: int, data_type=torch.float16, causal: bool = True, *,
                      qo_indptr_host: np.ndarray | None = None, kv_indptr_host: np.ndarray | None = None,
                      last_page_len_host: np.ndarray | None = None, kv_indices_host: np.ndarray | None = None) -> None:
        """Plan the q tiles of this batch. The *_host arrays (same values as the
        device tensors) avoid device->host copies."""
        if qo_indptr_host is None:
            qo_indptr_host = qo_indptr.cpu().numpy()
        if kv_indptr_host is None:
            kv_indptr_host = paged_kv_indptr.cpu().numpy()
        if last_page_len_host is None:
            last_page_len_host = paged_kv_last_page_len.cpu().numpy()
        n_pages = np.diff(kv_indptr_host)
        kv_len = np.where(n_pages > 0, (n_pages - 1) * page_size + last_page_len_host, 0).astype(np.int32)
        n_new = np.diff(qo_indptr_host)
        batch, nnz = len(kv_len), int(qo_indptr_host[-1])
        dtype = data_type if isinstance(data_type, torch.dtype) else torch.float16
        # decode rows of a mixed batch go to the decode kernel
        # (all of them or none: the prefill plan then skips every request with a single new token)
        dec = np.flatnonzero(n_new == 1) if causal else np.zeros(0, dtype=np.int64)
        split = (len(dec) > 0 and int(kv_len[dec].max()) >= self.SPLIT_MIN_KV
                 and self._ws.numel() >= 4 * self._PLAN_BYTES)
        cap = prefill_plan_capacity(nnz, batch, num_qo_heads // num_kv_heads)
        dec_cap = 0
        if split:
            if kv_indices_host is None:
                kv_indices_host = paged_kv_indices.cpu().numpy()
            sub_pages = n_pages[dec]
            sub_indptr = np.zeros(len(dec) + 1, dtype=np.int32)
            np.cumsum(sub_pages, out=sub_indptr[1:])
            # sections: prefill plan | decode plan | sub indptr | sub last | q rows | sub indices
            dec_cap = plan_capacity(len(dec), self._sm_count)
            total = cap + dec_cap + 3 * (len(dec) + 4) + int(sub_indptr[-1]) + 16
        else:
            total = cap
        if total * 4 > self._PLAN_BYTES:
            if split:  # too many decode rows for the workspace head: keep them in the prefill kernel
                split, total = False, cap
            if cap * 4 > self._PLAN_BYTES:
                raise _lib.DeserveKVError(f"prefill plan for {nnz} tokens does not fit the workspace head")
        pinned, slot = _pinned_ring("prefill_plan").take(total)
        buf = pinned.numpy()
        used = make_prefill_plan(qo_indptr_host, kv_len, num_qo_heads, num_kv_heads, head_dim, page_size, dtype, causal,
                                 buf[:cap], min_new_tokens=2 if split else 0)
        self._dec = None
        end = used
        if split:
            a4 = lambda n: (n + 3) & ~3
            o_plan = a4(used)
            d_used, ws_bytes = make_decode_plan(sub_indptr, num_qo_heads, num_kv_heads, head_dim, page_size, dtype,
                                                self._sm_count, buf[o_plan : o_plan + dec_cap])
            if ws_bytes > self._ws.numel() - self._PLAN_BYTES:
                raise _lib.DeserveKVError(f"workspace_buffer too small: split-KV partials need {ws_bytes} bytes")
            o_ip = a4(o_plan + d_used)
            o_last = a4(o_ip + len(dec) + 1)
            o_rows = a4(o_last + len(dec))
            o_idx = a4(o_rows + len(dec))
            end = o_idx + int(sub_indptr[-1])
            buf[o_ip : o_ip + len(dec) + 1] = sub_indptr
            buf[o_last : o_last + len(dec)] = last_page_len_host[dec]
            buf[o_rows : o_rows + len(dec)] = qo_indptr_host[dec]        # the single new row of each decode request
            starts = kv_indptr_host[dec]
            pos = 0
            for s0, n in zip(starts.tolist(), sub_pages.tolist()):
                buf[o_idx + pos : o_idx + pos + n] = kv_indices_host[s0 : s0 + n]
                pos += n
            self._dec = (o_plan, d_used, o_ip, o_last, o_rows, o_idx, len(dec), int(sub_indptr[-1]), buf[o_plan : o_plan + d_used])
        self._ws[: end * 4].view(torch.int32).copy_(pinned[:end], non_blocking=True)
        _pinned_ring("prefill_plan").done(slot)
        _COUNTERS["h2d_bytes"] += end * 4
        self._pinned, self._plan_host = pinned, buf
        self._desc = (qo_indptr, paged_kv_indptr, paged_kv_indices, paged_kv_last_page_len, num_qo_heads, head_dim, causal)

    def forward(self, q: torch.Tensor, paged_kv_cache: torch.Tensor, causal: bool = True, sm_scale: float | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
        if self._desc is None:
            raise RuntimeError("forward() called outside begin_forward()/end_forward()")
        qo, kv_indptr, kv_indices, last, hq, d, planned_causal = self._desc
        if causal != planned_causal:
            raise ValueError("forward(causal=...) differs from the value given to begin_forward")
        if q.dim() == 2:
            q = q.view(-1, hq, d)
        head = self._ws[: self._PLAN_BYTES].view(torch.int32)
        if out is None:
            out = torch.empty((q.shape[0], hq, d), dtype=q.dtype, device=q.device)
        if self._plan_host[1] > 0 or self._plan_host[8] > 0:  # single-CTA items, pair items
            paged_prefill(q, qo, paged_kv_cache, kv_indices, kv_indptr, last, self._plan_host, head, out, sm_scale, causal)
        if self._dec is not None:
            o_plan, d_used, o_ip, o_last, o_rows, o_idx, n_dec, n_idx, plan_host = self._dec
            rows = head[o_rows : o_rows + n_dec].long()
            out_dec = paged_decode(q.index_select(0, rows), paged_kv_cache, head[o_idx : o_idx + n_idx],
                                   head[o_ip : o_ip + n_dec + 1], head[o_last : o_last + n_dec], plan_host,
                                   head[o_plan : o_plan + d_used], self._ws[self._PLAN_BYTES :], sm_scale=sm_scale)
            out.index_copy_(0, rows, out_dec)
        return out

    def end_forward(self) -> None:
        self._desc = None
        self._dec = None


def rope_append_paged_kv_cache(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, indptr: torch.Tensor,
                               offsets: torch.Tensor, paged_kv_cache: torch.Tensor, kv_indices: torch.Tensor,
                               kv_indptr: torch.Tensor, kv_last_page_len: torch.Tensor,
                               rope_theta: float = 500000.0) -> None:
    """apply_rope + append_paged_kv_cache in one launch: q rotated in place, rotated
    k and plain v written into their page slots."""
    _lib.require_cuda(q, k, v, paged_kv_cache)
    ps, hkv, d, page_stride = _pages_view(paged_kv_cache)
    if not (q.dtype == k.dtype == v.dtype == paged_kv_cache.dtype):
        raise ValueError("rope_append: dtypes of q, k, v and the pages differ")
    hq = q.shape[1]
    qs, ks, vs = _row_stride(q, hq, d, "q"), _row_stride(k, hkv, d, "k"), _row_stride(v, hkv, d, "v")
    _lib.check(_lib.lib.dsv_rope_append_paged_kv(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), qs, ks, vs, _i32_dev(indptr, "indptr").data_ptr(),
        _i32_dev(offsets, "offsets").data_ptr(), paged_kv_cache.data_ptr(), page_stride, paged_kv_cache.shape[0],
        _i32_dev(kv_indices, "kv_indices").data_ptr(), _i32_dev(kv_indptr, "kv_indptr").data_ptr(),
        _i32_dev(kv_last_page_len, "kv_last_page_len").data_ptr(), kv_last_page_len.shape[0], q.shape[0], hq, hkv, d, ps,
        float(rope_theta), rope_inv_freq(d, rope_theta).data_ptr(), _lib.dtype_code(q.dtype),
        _lib.current_stream_ptr(q.device)))
    _lib.LAUNCHES[0] += 1


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * weight over the last dimension of a [rows, dim] tensor."""
    _lib.require_cuda(x, weight)
    if x.dim() != 2 or x.stride(1) != 1 or weight.shape != (x.shape[1],) or weight.dtype != x.dtype:
        raise ValueError("rmsnorm: x must be [rows, dim] with dense rows and weight [dim] of the same dtype")
    if out is None:
        out = torch.empty_like(x, memory_format=torch.contiguous_format)
    _lib.check(_lib.lib.dsv_rmsnorm(x.data_ptr(), weight.contiguous().data_ptr(), out.data_ptr(), x.stride(0),
                                    out.stride(0), x.shape[0], x.shape[1], float(eps), _lib.dtype_code(x.dtype),
                                    _lib.current_stream_ptr(x.device)))
    _lib.LAUNCHES[0] += 1
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """silu(gate_up[:, :F]) * gate_up[:, F:] for a [rows, 2F] tensor (gate columns, then up columns)."""
    _lib.require_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.stride(1) != 1 or gate_up.shape[1] % 2:
        raise ValueError("silu_mul: gate_up must be [rows, 2 * ffn_dim] with dense rows")
    ffn = gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((gate_up.shape[0], ffn), dtype=gate_up.dtype, device=gate_up.device)
    _lib.check(_lib.lib.dsv_silu_mul(gate_up.data_ptr(), out.data_ptr(), gate_up.stride(0), out.stride(0),
                                     gate_up.shape[0], ffn, _lib.dtype_code(gate_up.dtype),
                                     _lib.current_stream_ptr(gate_up.device)))
    _lib.LAUNCHES[0] += 1
    return out


def greedy_sample(logits: torch.Tensor) -> torch.Tensor:
    """int32 argmax of every row of [rows, vocab] logits (lowest index among ties)."""
    _lib.require_cuda(logits)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("greedy_sample: logits must be [rows, vocab] with dense rows")
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _lib.check(_lib.lib.dsv_greedy_sample(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1],
                                          out.data_ptr(), _lib.dtype_code(logits.dtype),
                                          _lib.current_stream_ptr(logits.device)))
    _lib.LAUNCHES[0] += 1
    return out
