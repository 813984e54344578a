"""ctypes binding of libdeserve_kv.so (the C ABI declared in include/deserve_kv.h).

There is no fallback: if the shared library is missing and cannot be built,
importing this module raises, and every wrapper refuses tensors that are not on
a CUDA device.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

import torch

from . import build as _build

LIB_PATH = Path(__file__).resolve().parent / "libdeserve_kv.so"

DSV_F32, DSV_F16, DSV_BF16 = 0, 1, 2
STATIC_SCRATCH_BYTES = 16 << 20
E_INVALID, E_CUDA, E_WORKSPACE, E_UNSUPPORTED, E_DEVICE = -1, -2, -3, -4, -5

_DTYPES = {torch.float32: DSV_F32, torch.float16: DSV_F16, torch.bfloat16: DSV_BF16}


class DeserveKVError(RuntimeError):
    """A C-ABI call failed (CUDA error, workspace too small, device self-check)."""


def _load() -> ctypes.CDLL:
    if _build.is_stale():
        try:
            _build.build()
        except Exception as exc:  # no nvcc on this machine: use the shipped binary if there is one
            if not LIB_PATH.exists():
                raise ImportError(
                    f"libdeserve_kv.so is missing at {LIB_PATH} and could not be built ({exc}); "
                    "run `python -m deserve_b200.build` on a machine with nvcc"
                ) from exc
    return ctypes.CDLL(str(LIB_PATH))


lib = _load()

_p32 = POINTER(c_int32)
_p64 = POINTER(c_int64)

_SIGNATURES = {
    "dsv_version": (c_int, []),
    "dsv_last_error": (c_char_p, []),
    "dsv_device_info": (c_int, [POINTER(c_int)] * 3),
    "dsv_read_device_status": (c_int, [POINTER(c_int)]),
    "dsv_selftest_wait_timeout": (c_int, [c_int, c_void_p]),
    "dsv_peer_push": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int32, c_void_p, c_int, c_void_p]),
    "dsv_peer_signal": (c_int, [c_void_p, c_int32, c_void_p]),
    "dsv_peer_wait": (c_int, [c_void_p, c_int32, c_int64, c_void_p]),
    "dsv_host_build_step": (c_int, [c_void_p, c_int32, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32,
                                    c_int32, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "dsv_device_build_step": (c_int, [c_void_p, c_int32, c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_int64, c_void_p,
                                      c_int32, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "dsv_device_free_rows": (c_int, [c_void_p, c_int32, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p]),
    "dsv_append_paged_kv": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64,
                                    c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "dsv_apply_rope_inplace": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int, c_int,
                                       c_int, c_int, c_float, c_void_p, c_int, c_void_p]),
    "dsv_rope_append_paged_kv": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                         c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                         c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p]),
    "dsv_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_float, c_int, c_void_p]),
    "dsv_silu_mul": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_void_p]),
    "dsv_greedy_sample": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p]),
    "dsv_decode_plan": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int64, _p64,
                                _p64]),
    "dsv_paged_decode": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                                 c_int, c_int, c_float, c_void_p]),
    "dsv_paged_decode_static": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_float, c_void_p]),
    "dsv_prefill_plan": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                 c_int64, _p64]),
    "dsv_paged_prefill": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_float, c_int, c_void_p]),
    "dsv_pack_pages": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int64, c_int, c_int,
                               c_void_p, c_void_p]),
    "dsv_unpack_pages": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int64,
                                 c_int, c_int, c_void_p]),
    "dsv_swap_out_pages": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "dsv_swap_in_pages": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "dsv_region_swap": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int32]),
}

for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


# kernels of this library launched through the Python operators since the counter was last reset
LAUNCHES = [0]


def last_error() -> str:
    return lib.dsv_last_error().decode()


def check(rc: int) -> None:
    """Turn a negative return code into the exception type the reference raises
    for the same condition: bad arguments -> ValueError, the rest -> RuntimeError."""
    if rc == 0:
        return
    msg = last_error()
    if rc == E_INVALID:
        raise ValueError(msg)
    raise DeserveKVError(f"[dsv {rc}] {msg}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"unsupported KV dtype {dtype}; expected float32, float16 or bfloat16") from None


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "deserve_b200 kernels run on CUDA tensors only; got a tensor on "
                f"{t.device}. There is no CPU path in this package."
            )


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def current_stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def device_info() -> tuple[int, int, int]:
    a, b, c = c_int(), c_int(), c_int()
    check(lib.dsv_device_info(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)))
    return a.value, b.value, c.value


def read_device_status() -> int:
    s = c_int()
    check(lib.dsv_read_device_status(ctypes.byref(s)))
    return s.value
