"""On-disk format for ``QuantizedTensor`` (and whole quantized models).

The reference has none: ``QuantizedLinear`` keeps its streams as plain
attributes that are absent from ``state_dict()``
(integration/atlas_wrappers.py:23-27), so a model must be re-quantized on every
start.  This module writes the six fields of any number of named
``QuantizedTensor`` records (plus an optional bias each) into one flat file:

    bytes 0..7     magic  b"ATLASQT1"
    bytes 8..15    little-endian uint64: length H of the JSON header
    bytes 16..16+H JSON: {"records": {name: {"shape": [...], "block_size": n,
                   "arrays": {field: {"dtype": "int8", "count": n, "offset": o}}}}}
    then the raw little-endian arrays, each starting on a 64-byte boundary
    (offsets are relative to the start of the file)

Every array can therefore be mapped with ``numpy.memmap(path, dtype, "r",
offset, shape)`` without reading the rest.  fp16 arrays are stored as their raw
16-bit patterns under dtype "float16".
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Tuple, Union

import numpy as np
import torch

from .adaptive_quantizer import QuantizedTensor

MAGIC = b"ATLASQT1"
_ALIGN = 64
_FIELDS = (("fp8_data", "int8"), ("fp16_outliers", "float16"), ("outlier_indices", "int64"),
           ("scale_factors", "float16"))
_TORCH = {"int8": torch.int8, "float16": torch.float16, "int64": torch.int64}

Record = Union[QuantizedTensor, Tuple[QuantizedTensor, Optional[torch.Tensor]]]


def _np(t: torch.Tensor, dtype: str) -> np.ndarray:
    t = t.detach().to("cpu").contiguous()
    if dtype == "float16":
        return t.view(torch.int16).numpy().view(np.float16)
    return t.numpy()


def save_quantized_state(path: str, records: Dict[str, Record]) -> None:
    """Write named ``QuantizedTensor`` records (optionally ``(q, bias)`` pairs) to ``path``."""
    header = {"records": {}}
    arrays = []
    for name, rec in records.items():
        q, bias = rec if isinstance(rec, tuple) and not hasattr(rec, "fp8_data") else (rec, None)
        entry = {"shape": [int(v) for v in q.original_shape], "block_size": int(q.block_size), "arrays": {}}
        for field, dtype in _FIELDS:
            a = _np(getattr(q, field), dtype)
            entry["arrays"][field] = {"dtype": dtype, "count": int(a.size)}
            arrays.append((entry["arrays"][field], a))
        if bias is not None:
            a = _np(bias.to(torch.float16), "float16")
            entry["arrays"]["bias"] = {"dtype": "float16", "count": int(a.size)}
            arrays.append((entry["arrays"]["bias"], a))
        header["records"][name] = entry
    # offsets depend on the header's own length: lay the arrays out after a header padded to a fixed size
    for meta, _ in arrays:
        meta["offset"] = 0
    probe = json.dumps(header).encode()
    header_room = (16 + len(probe) + 24 * len(arrays) + _ALIGN - 1) // _ALIGN * _ALIGN   # room for the real offsets
    pos = header_room
    for meta, a in arrays:
        meta["offset"] = pos
        pos = (pos + a.nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
    blob = json.dumps(header).encode()
    if 16 + len(blob) > header_room:
        raise RuntimeError("header grew past its reserved room")
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(MAGIC)
        f.write(np.uint64(len(blob)).tobytes())
        f.write(blob)
        for meta, a in arrays:
            f.seek(meta["offset"])
            f.write(a.tobytes())
        f.truncate(pos)
    os.replace(tmp, path)


def read_header(path: str) -> dict:
    with open(path, "rb") as f:
        if f.read(8) != MAGIC:
            raise ValueError(f"{path}: not an AtlasInfer quantized-tensor file")
        n = int(np.frombuffer(f.read(8), dtype=np.uint64)[0])
        return json.loads(f.read(n).decode())


def _load_array(path: str, meta: dict, device) -> torch.Tensor:
    dtype = meta["dtype"]
    count = int(meta["count"])
    if count == 0:
        return torch.empty(0, dtype=_TORCH[dtype], device=device)
    raw = np.memmap(path, dtype=np.int16 if dtype == "float16" else np.dtype(dtype), mode="r",
                    offset=int(meta["offset"]), shape=(count,))
    t = torch.from_numpy(np.array(raw))   # a private, writable copy of the mapped bytes
    if dtype == "float16":
        t = t.view(torch.float16)
    return t.to(device)


def load_quantized_state(path: str, device="cpu", names=None) -> Dict[str, Tuple[QuantizedTensor, Optional[torch.Tensor]]]:
    """Read records written by ``save_quantized_state``: name -> (QuantizedTensor, bias or None) on ``device``."""
    header = read_header(path)
    out = {}
    for name, entry in header["records"].items():
        if names is not None and name not in names:
            continue
        arr = entry["arrays"]
        q = QuantizedTensor(*(_load_array(path, arr[f], device) for f, _ in _FIELDS),
                            torch.Size(entry["shape"]), int(entry["block_size"]))
        bias = _load_array(path, arr["bias"], device) if "bias" in arr else None
        out[name] = (q, bias)
    return out


def save_quantized(path: str, q: QuantizedTensor, bias: Optional[torch.Tensor] = None) -> None:
    """One ``QuantizedTensor`` (and optional bias) to ``path``."""
    save_quantized_state(path, {"tensor": (q, bias)})


def load_quantized(path: str, device="cpu") -> QuantizedTensor:
    """The ``QuantizedTensor`` written by ``save_quantized``."""
    return load_quantized_state(path, device)["tensor"][0]


def save_quantized_model(model: torch.nn.Module, path: str) -> int:
    """Every ``QuantizedLinear`` of ``model`` (by qualified name) into one file; returns how many."""
    records = {}
    for name, mod in model.named_modules():
        if type(mod).__name__ == "QuantizedLinear":
            records[name] = (mod.quantized_weights, mod.bias)
    save_quantized_state(path, records)
    return len(records)


def load_quantized_model(model: torch.nn.Module, path: str, device="cpu") -> int:
    """Replace the ``nn.Linear`` / ``QuantizedLinear`` modules named in the file by ``QuantizedLinear``
    built from the stored streams (no re-quantization); returns how many were installed."""
    from ..integration.atlas_wrappers import QuantizedLinear
    from ..integration.model_modifier import _replace_module, _split
    state = load_quantized_state(path, device)
    for name, (q, bias) in state.items():
        parent_name, child = _split(name)
        parent = model.get_submodule(parent_name) if parent_name else model
        _replace_module(parent, child, QuantizedLinear(q, bias))
    return len(state)
