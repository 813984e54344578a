"""Byte framing of a step request between pipeline stages.

Two framings exist in the reference, both made of the same two parts — the
tensors as one safetensors blob and the metadata dict pickled:

  * deserve_worker/model/utils.py:12-47 (what PipelineProcessor.send_request posts,
    engine/pipeline/processor.py:224):  u32be(len(meta)) | meta | tensors.
    A tensor without elements is replaced by a one-element stand-in named '#name'.
  * deserve_network/src/server.rs:97-114,197-201 (the Rust transport):
    u32be(len(tensors)) | tensors | meta.

The safetensors container is written and read here directly (8-byte little-endian
header length, a compact JSON header padded with spaces to a multiple of 8, raw
little-endian data): tensors are ordered by descending dtype rank, then by name,
as the published serializer orders them, so frames are byte-identical to the
reference's for the same inputs.
"""
from __future__ import annotations

import io
import json
import pickle
import struct
from typing import Any

import numpy as np
import torch

# dtype names in the serializer's rank order (low to high)
_RANK = ["BOOL", "U8", "I8", "F8_E5M2", "F8_E4M3", "I16", "U16", "F16", "BF16", "I32", "U32", "F32", "F64", "I64", "U64"]
_NAME = {torch.bool: "BOOL", torch.uint8: "U8", torch.int8: "I8", torch.int16: "I16", torch.float16: "F16",
         torch.bfloat16: "BF16", torch.int32: "I32", torch.float32: "F32", torch.float64: "F64", torch.int64: "I64"}
_DTYPE = {v: k for k, v in _NAME.items()}


def _raw(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


def st_save(tensors: dict[str, torch.Tensor]) -> bytes:
    """The safetensors container of a dict of dense tensors."""
    for name, t in tensors.items():
        if t.dtype not in _NAME:
            raise ValueError(f"tensor {name!r}: dtype {t.dtype} has no safetensors name here")
    order = sorted(tensors, key=lambda n: (-_RANK.index(_NAME[tensors[n].dtype]), n))
    header, blobs, at = {}, [], 0
    for name in order:
        t = tensors[name]
        data = _raw(t)
        header[name] = {"dtype": _NAME[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(data)]}
        at += len(data)
        blobs.append(data)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    return struct.pack("<Q", len(text)) + text + b"".join(blobs)


def st_load(blob: bytes) -> dict[str, torch.Tensor]:
    if len(blob) < 8:
        raise ValueError("safetensors: shorter than its length field")
    (n,) = struct.unpack("<Q", blob[:8])
    if 8 + n > len(blob):
        raise ValueError("safetensors: header runs past the end")
    header = json.loads(blob[8 : 8 + n])
    body = memoryview(blob)[8 + n :]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        dtype = _DTYPE[info["dtype"]]
        if b > len(body) or a > b:
            raise ValueError(f"safetensors: tensor {name!r} lies outside the data")
        if b == a:
            out[name] = torch.empty(info["shape"], dtype=dtype)
        else:
            raw = torch.from_numpy(np.frombuffer(body[a:b], dtype=np.uint8).copy())
            out[name] = raw.view(dtype).reshape(info["shape"])
    return out


class _MetadataUnpickler(pickle.Unpickler):
    """Metadata is lists, dicts, strings and numbers, plus the sampling parameters of
    prompts that start in the step. Nothing else is constructed: a frame naming any
    other global is refused instead of imported."""

    def __init__(self, data: bytes, allowed: dict):
        super().__init__(io.BytesIO(data))
        self._allowed = allowed

    def find_class(self, module: str, name: str):
        try:
            return self._allowed[(module, name)]
        except KeyError:
            raise pickle.UnpicklingError(f"frame metadata names {module}.{name}, which is not a metadata type") from None


def _load_metadata(data: bytes, extra_classes=()) -> dict[str, Any]:
    from .task import SamplingParams

    allowed = {(c.__module__, c.__qualname__): c for c in (SamplingParams, *extra_classes)}
    return _MetadataUnpickler(data, allowed).load()


def _with_standins(tensors: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    return {(f"#{k}" if v.numel() == 0 else k): (torch.ones((1,), dtype=v.dtype) if v.numel() == 0 else v)
            for k, v in tensors.items()}


def _without_standins(tensors: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    return {(k[1:] if k.startswith("#") else k): (torch.empty((0,), dtype=v.dtype) if k.startswith("#") else v)
            for k, v in tensors.items()}


def dumps(tensors: dict[str, torch.Tensor], metadata: dict[str, Any]) -> bytes:
    """u32be(len(meta)) | pickle(meta) | safetensors  (model/utils.py:12-30)."""
    meta = pickle.dumps(metadata)
    return len(meta).to_bytes(4, "big") + meta + st_save(_with_standins(tensors))


def loads(frame: bytes, extra_classes=()) -> tuple[dict[str, torch.Tensor], dict[str, Any]]:
    """Inverse of dumps (model/utils.py:33-47). The metadata is unpickled with an
    allow-list: plain containers and this package's SamplingParams, plus the classes
    in `extra_classes` (inside deserve_worker: its own SamplingParams)."""
    n = int.from_bytes(frame[:4], "big")
    if 4 + n > len(frame):
        raise ValueError("frame: metadata length runs past the end")
    return _without_standins(st_load(frame[4 + n :])), _load_metadata(frame[4 : 4 + n], extra_classes)


def dumps_network(tensors: dict[str, torch.Tensor], metadata: dict[str, Any]) -> bytes:
    """u32be(len(safetensors)) | safetensors | pickle(meta)  (server.rs:197-201;
    the Python side pickles the metadata, deserve_network/__init__.py:27-30)."""
    blob = st_save(tensors)
    return len(blob).to_bytes(4, "big") + blob + pickle.dumps(metadata)


def loads_network(frame: bytes, extra_classes=()) -> tuple[dict[str, torch.Tensor], dict[str, Any]]:
    """Inverse of dumps_network (server.rs:97-114, __init__.py:32-34); metadata
    allow-list as in loads."""
    n = int.from_bytes(frame[:4], "big")
    if 4 + n > len(frame):
        raise ValueError("frame: tensor length runs past the end")
    return st_load(frame[4 : 4 + n]), _load_metadata(frame[4 + n :], extra_classes)
