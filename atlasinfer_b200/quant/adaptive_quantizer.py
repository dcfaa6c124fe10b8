"""Adaptive hybrid quantizer with the reference's Python surface, computed on a B200.

Mirrors ``atlasinfer_core/quant/adaptive_quantizer.py`` of AtlasInfer: the same
``QuantizedTensor`` NamedTuple (:8-42), ``quantize_tensor`` (:51-148),
``dequantize_tensor`` (:156-251) and ``clear_dequantized_cache`` (:253-263) with
the same argument names, defaults, result devices and error behaviour.  The
arithmetic runs in ``libatlas_b200.so`` (hand-written sm_100a kernels); outputs
are bit-identical to the reference's.  Tensors that live on the CPU are staged
through the GPU and the results returned to the CPU, as the reference's callers
expect (``integration/model_modifier.py:128-131`` always passes CPU weights).
"""
from __future__ import annotations

import threading
from typing import NamedTuple, Optional

import torch

from .. import _capi


class QuantizedTensor(NamedTuple):
    """Hybrid INT8-code / fp16-outlier image of a tensor (reference :8-18).

    ``fp8_data`` holds the non-outlier codes of every block back to back,
    ``fp16_outliers`` / ``outlier_indices`` the raw outlier values and their
    ascending flat positions in the zero-padded tensor, ``scale_factors`` one
    fp16 scale per block.
    """

    fp8_data: torch.Tensor
    fp16_outliers: torch.Tensor
    outlier_indices: torch.Tensor
    scale_factors: torch.Tensor
    original_shape: torch.Size
    block_size: int

    def to(self, device):
        """Rebuild the tuple on ``device``; returns ``self`` if already there (:20-32)."""
        if self.fp8_data.device == device:
            return self
        return QuantizedTensor(
            fp8_data=self.fp8_data.to(device),
            fp16_outliers=self.fp16_outliers.to(device),
            outlier_indices=self.outlier_indices.to(device),
            scale_factors=self.scale_factors.to(device),
            original_shape=self.original_shape,
            block_size=self.block_size,
        )

    def memory_footprint(self, include_overhead=True) -> int:
        """Bytes held by the four streams, plus 128 if ``include_overhead`` (:34-42)."""
        total = 0
        for t in (self.fp8_data, self.fp16_outliers, self.outlier_indices, self.scale_factors):
            total += t.element_size() * t.nelement()
        return total + (128 if include_overhead else 0)


def _launch_quantize(flat: torch.Tensor, block_size: int, z_threshold: float, counts: torch.Tensor, capacity: int):
    """Enqueue the quantize kernel for a flat fp16 CUDA tensor; nothing is read back here."""
    L = _capi.load()
    dev = flat.device
    numel = flat.numel()
    n_blocks = (numel + block_size - 1) // block_size
    padded = n_blocks * block_size
    ws_bytes = int(L.atlas_quantize_workspace_bytes(numel, block_size))
    with torch.cuda.device(dev):
        codes = torch.empty(padded, dtype=torch.int8, device=dev)
        scales = torch.empty(n_blocks, dtype=torch.float16, device=dev)
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        ovals = torch.empty(capacity, dtype=torch.float16, device=dev)
        oidx = torch.empty(capacity, dtype=torch.int64, device=dev)
        status = L.atlas_quantize(
            flat.data_ptr(), numel, block_size, float(z_threshold), codes.data_ptr(),
            _capi.ptr(ovals), _capi.ptr(oidx), capacity, scales.data_ptr(), counts.data_ptr(),
            workspace.data_ptr(), ws_bytes, _capi.stream_ptr(dev))
    _capi.check(status, "atlas_quantize")
    return dict(flat=flat, codes=codes, scales=scales, ovals=ovals, oidx=oidx, workspace=workspace,
                capacity=capacity, padded=padded)


def _first_capacity(padded: int) -> int:
    # |z| > t bounds the outliers of a block by (block_size - 1) / t^2, but weight-like data has well under
    # 1 %: start with 1/32 of the tensor and retry with full capacity in the rare case that is short
    return min(padded, padded // 32 + 1024)


def _quantize_many_on_device(flats, block_size: int, z_threshold: float):
    """Quantize several flat fp16 CUDA tensors (one device): all kernels are enqueued first, the stream
    lengths of all of them come back in one device-to-host copy.  Returns the four streams per tensor."""
    dev = flats[0].device
    with torch.cuda.device(dev):
        counts = torch.empty((len(flats), 4), dtype=torch.int64, device=dev)
    jobs = []
    for i, flat in enumerate(flats):
        padded = (flat.numel() + block_size - 1) // block_size * block_size
        jobs.append(_launch_quantize(flat, block_size, z_threshold, counts[i], _first_capacity(padded)))
    host = counts.cpu()   # the one synchronisation
    out = []
    for i, job in enumerate(jobs):
        n_codes, n_out, timed_out, _ = (int(v) for v in host[i])
        if timed_out:
            raise _capi.AtlasError(_capi.ERR_TIMEOUT, "atlas_quantize: device-side wait timed out")
        if n_out > job["capacity"]:   # rare: more outliers than the first buffer holds
            job = _launch_quantize(job["flat"], block_size, z_threshold, counts[i], job["padded"])
            n_codes, n_out, timed_out, _ = (int(v) for v in counts[i].cpu())
            if timed_out:
                raise _capi.AtlasError(_capi.ERR_TIMEOUT, "atlas_quantize: device-side wait timed out")
        # codes: a view (the buffer is 0.3 % longer than the stream); outliers: copied out of their roomy buffers
        out.append((job["codes"][:n_codes], job["ovals"][:n_out].clone(), job["oidx"][:n_out].clone(), job["scales"]))
    return out


def _quantize_on_device(flat: torch.Tensor, block_size: int, z_threshold: float):
    """Run the quantize kernel on a flat fp16 CUDA tensor; returns the four streams."""
    return _quantize_many_on_device([flat], block_size, z_threshold)[0]


def quantize_tensor(
    fp16_tensor: torch.Tensor,
    block_size: int = 128,
    z_threshold: float = 3.0,
) -> QuantizedTensor:
    """Quantize an fp16 tensor into the hybrid format (reference :51-148).

    Results live on the input's device.  ``block_size`` must be a multiple of
    32 in [32, 512] (``NotImplementedError`` otherwise).
    """
    if not isinstance(fp16_tensor, torch.Tensor):
        raise TypeError(f"Input must be a PyTorch Tensor, got {type(fp16_tensor)}")
    if fp16_tensor.dtype != torch.float16:
        print(f"Warning: Input tensor was {fp16_tensor.dtype}, converting to FP16 for quantization.")
        fp16_tensor = fp16_tensor.to(torch.float16)

    input_device = fp16_tensor.device
    original_shape = fp16_tensor.shape
    if fp16_tensor.numel() == 0:
        def empty(dt):
            return torch.empty((0,), dtype=dt, device=input_device)
        return QuantizedTensor(empty(torch.int8), empty(torch.float16), empty(torch.long),
                               empty(torch.float16), original_shape, block_size)

    dev = _capi.require_cuda(input_device)
    flat = fp16_tensor.detach().reshape(-1).contiguous()
    if flat.device != dev:
        flat = flat.to(dev, non_blocking=True)
    codes, ovals, oidx, scales = _quantize_on_device(flat, int(block_size), float(z_threshold))
    if input_device != dev:
        codes, ovals, oidx, scales = (t.to(input_device) for t in (codes, ovals, oidx, scales))
    return QuantizedTensor(codes, ovals, oidx, scales, original_shape, block_size)


def quantize_tensors(tensors, block_size: int = 128, z_threshold: float = 3.0):
    """``[quantize_tensor(t, block_size, z_threshold) for t in tensors]`` with one host synchronisation.

    The reference quantizes layer by layer (integration/model_modifier.py:117-131).  Here the kernels of all
    tensors are enqueued back to back and the data-dependent stream lengths are read once for the whole
    batch, so the GPU never idles between tensors.  Results are identical to the one-by-one calls and live
    on each input's device."""
    tensors = list(tensors)
    results = [None] * len(tensors)
    per_device = {}
    for i, t in enumerate(tensors):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"Input must be a PyTorch Tensor, got {type(t)}")
        if t.dtype != torch.float16:
            print(f"Warning: Input tensor was {t.dtype}, converting to FP16 for quantization.")
            t = t.to(torch.float16)
        if t.numel() == 0:
            results[i] = quantize_tensor(t, block_size, z_threshold)
            continue
        dev = _capi.require_cuda(t.device)
        flat = t.detach().reshape(-1).contiguous()
        if flat.device != dev:
            flat = flat.to(dev, non_blocking=True)
        per_device.setdefault(dev, []).append((i, flat, t.device, t.shape))
    for dev, items in per_device.items():
        streams = _quantize_many_on_device([f for _, f, _, _ in items], int(block_size), float(z_threshold))
        for (i, _, in_dev, shape), (codes, ovals, oidx, scales) in zip(items, streams):
            if in_dev != dev:
                codes, ovals, oidx, scales = (x.to(in_dev) for x in (codes, ovals, oidx, scales))
            results[i] = QuantizedTensor(codes, ovals, oidx, scales, shape, block_size)
    return results


# --- dequantization cache (reference :153-154): id(quant_data) -> fp16 tensor.  Each entry also
# holds the QuantizedTensor itself, so an id cannot be recycled while its entry is alive.
_dequantized_weights_cache = {}
_cache_lock = threading.Lock()


def _dequantize_on_device(q: QuantizedTensor, dev: torch.device) -> torch.Tensor:
    L = _capi.load()
    shape = torch.Size(q.original_shape)
    numel = shape.numel()
    out = torch.empty(numel, dtype=torch.float16, device=dev)
    if numel:
        codes, ovals = q.fp8_data.contiguous(), q.fp16_outliers.contiguous()
        oidx, scales = q.outlier_indices.contiguous(), q.scale_factors.contiguous()
        with torch.cuda.device(dev):
            status = L.atlas_dequantize(
                _capi.ptr(codes), codes.numel(), _capi.ptr(ovals), _capi.ptr(oidx), oidx.numel(),
                scales.data_ptr(), numel, int(q.block_size), out.data_ptr(), _capi.stream_ptr(dev))
        _capi.check(status, "atlas_dequantize")
    return out.view(shape)


def dequantize_tensor(quant_data: QuantizedTensor, target_device: torch.device) -> torch.Tensor:
    """fp16 reconstruction of ``quant_data`` on ``target_device`` (reference :156-251).

    Like the reference, the result is cached per ``quant_data`` object until
    ``clear_dequantized_cache`` is called.  The quantized linear layer of this
    package never calls this function; it multiplies by the codes directly.
    """
    target_device = torch.device(target_device)
    key = id(quant_data)
    with _cache_lock:
        entry = _dequantized_weights_cache.get(key)
        if entry is not None:
            cached = entry[1]
            if cached.device != target_device:
                cached = cached.to(target_device)
                _dequantized_weights_cache[key] = (quant_data, cached)
            return cached

    dev = _capi.require_cuda(target_device)
    result = _dequantize_on_device(quant_data.to(dev), dev)
    if target_device != dev:
        result = result.to(target_device)
    with _cache_lock:
        _dequantized_weights_cache[key] = (quant_data, result)
    return result


def clear_dequantized_cache(quant_data_id=None):
    """Drop one cached reconstruction, or all of them (reference :253-263)."""
    global _dequantized_weights_cache
    with _cache_lock:
        if quant_data_id is not None and quant_data_id in _dequantized_weights_cache:
            del _dequantized_weights_cache[quant_data_id]
        elif quant_data_id is None:
            _dequantized_weights_cache = {}
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
