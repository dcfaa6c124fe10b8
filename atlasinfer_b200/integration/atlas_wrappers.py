"""``QuantizedLinear`` with the reference's surface, computed by the B200 kernels.

Mirrors ``integration/atlas_wrappers.py:21-83`` of AtlasInfer: a module that
keeps a ``QuantizedTensor`` and an optional bias as plain attributes
(``quantized_weights``, ``bias``, ``original_shape`` -- readable and
re-assignable, absent from ``state_dict``), moves them lazily to the
activations' device, and returns ``x @ W^T + bias``.  Where the reference
dequantizes the whole weight to a cached fp16 copy and calls ``F.linear``
(:56, :67), this module keeps a tile-major uint8 image of the codes beside the
canonical streams and calls the fused dequant GEMV / GEMM of
``libatlas_b200.so``; no fp16 weight is ever materialised.
"""
from __future__ import annotations

import os
from typing import NamedTuple, Optional

import torch
import torch.nn as nn

from .. import _capi
from ..quant.adaptive_quantizer import QuantizedTensor

# rows of x up to which the CUDA-core-issued streaming kernel is used; above it the tcgen05 kernel
GEMV_MAX_ROWS = 16

_VERBOSE = os.environ.get("ATLAS_VERBOSE", "0") not in ("", "0")


class KernelLayout(NamedTuple):
    """Device-resident kernel image of one quantized [N, K] weight (written by atlas_repack)."""

    source: object                 # the QuantizedTensor it was built from (identity-checked)
    tiles: torch.Tensor            # uint8, tile-major dense codes + 128
    scales_tiled: torch.Tensor     # fp16, [N/128][K/block][128]
    row_ptr: torch.Tensor          # int32 [N + 1], CSR over the canonical outlier streams
    chunk_ptr: torch.Tensor        # int32 [N_padded/16][K/64 + 1]
    entries: torch.Tensor          # int32 (row%16 << 24 | col), strip-major, column-sorted
    vals_sorted: torch.Tensor      # fp16 outlier values in the order of `entries`
    n_rows: int
    n_cols: int
    block_size: int


_status_words = {}


def status_word(dev: torch.device) -> torch.Tensor:
    """The device int32 kernels set non-zero when a bounded wait ran out (one per device)."""
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status_words[key] = t
    return t


def check_status(dev: torch.device) -> None:
    """Synchronise and raise if any kernel on ``dev`` reported a timed-out wait."""
    if int(status_word(dev).item()) != 0:
        status_word(dev).zero_()
        raise _capi.AtlasError(_capi.ERR_TIMEOUT, "a quantized-linear kernel gave up on a bounded wait")


def kernel_layout_supported(shape, block_size: int) -> Optional[str]:
    """``None`` if a weight of ``shape`` can use the fused kernels, else the reason."""
    if len(shape) != 2:
        return f"weight must be 2-D, got shape {tuple(shape)}"
    k = int(shape[1])
    if k % 64 != 0:
        return f"in_features {k} is not a multiple of 64"
    if block_size % 16 != 0 or k % block_size != 0:
        return f"block_size {block_size} must be a multiple of 16 that divides in_features {k}"
    return None


def build_kernel_layout(q: QuantizedTensor) -> KernelLayout:
    """Expand the compacted code stream of ``q`` (on a CUDA device) into the kernel layout."""
    reason = kernel_layout_supported(q.original_shape, int(q.block_size))
    if reason is not None:
        raise NotImplementedError("QuantizedLinear: " + reason)
    L = _capi.load()
    dev = q.fp8_data.device
    n, k = int(q.original_shape[0]), int(q.original_shape[1])
    n_out = q.outlier_indices.numel()
    bs = int(q.block_size)
    n_pad = (n + 127) // 128 * 128
    with torch.cuda.device(dev):
        tiles = torch.empty(int(L.atlas_tiles_bytes(n, k)), dtype=torch.uint8, device=dev)
        scales_tiled = torch.empty(n_pad * (k // bs), dtype=torch.float16, device=dev)
        row_ptr = torch.empty(n + 1, dtype=torch.int32, device=dev)
        chunk_ptr = torch.empty((n_pad // 16) * (k // 64 + 1), dtype=torch.int32, device=dev)
        entries = torch.empty(n_out, dtype=torch.int32, device=dev)
        vals_sorted = torch.empty(n_out, dtype=torch.float16, device=dev)
        codes, oidx = q.fp8_data.contiguous(), q.outlier_indices.contiguous()
        ovals, scales = q.fp16_outliers.contiguous(), q.scale_factors.contiguous()
        status = L.atlas_repack(_capi.ptr(codes), codes.numel(), _capi.ptr(ovals), _capi.ptr(oidx), n_out,
                                scales.data_ptr(), n, k, bs, tiles.data_ptr(), scales_tiled.data_ptr(),
                                row_ptr.data_ptr(), chunk_ptr.data_ptr(), _capi.ptr(entries),
                                _capi.ptr(vals_sorted), _capi.stream_ptr(dev))
    _capi.check(status, "atlas_repack")
    return KernelLayout(q, tiles, scales_tiled, row_ptr, chunk_ptr, entries, vals_sorted, n, k, bs)


def quantized_linear_forward(x: torch.Tensor, layout: KernelLayout, bias: Optional[torch.Tensor],
                             force: Optional[str] = None) -> torch.Tensor:
    """``x @ W^T + bias`` on CUDA tensors through the C ABI.  ``force``: "gemv" / "gemm"."""
    L = _capi.load()
    dev = x.device
    if x.dtype == torch.float16:
        dtype = _capi.DTYPE_F16
    elif x.dtype == torch.bfloat16:
        dtype = _capi.DTYPE_BF16
    else:
        raise RuntimeError(f"QuantizedLinear expects fp16 (or bf16) activations, got {x.dtype}")
    n, k = layout.n_rows, layout.n_cols
    if x.shape[-1] != k:
        raise RuntimeError(f"QuantizedLinear: input has {x.shape[-1]} features, weight expects {k}")
    x2 = x.reshape(-1, k)
    if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) < k):
        x2 = x2.contiguous()
    m = x2.shape[0]
    ldx = x2.stride(0) if m > 1 else k
    y = torch.empty((m, n), dtype=x.dtype, device=dev)
    if m == 0:
        return y.view(*x.shape[:-1], n)
    b = None
    if bias is not None:
        b = bias if bias.dtype == torch.float16 else bias.to(torch.float16)
        b = b.contiguous()
    use_gemv = (m <= GEMV_MAX_ROWS) if force is None else (force == "gemv")
    args = [x2.data_ptr(), dtype, m, ldx, layout.tiles.data_ptr(), layout.scales_tiled.data_ptr(),
            layout.chunk_ptr.data_ptr(), _capi.ptr(layout.entries), _capi.ptr(layout.vals_sorted), n, k,
            layout.block_size, _capi.ptr(b), y.data_ptr(), n]
    flag = status_word(dev).data_ptr()
    with torch.cuda.device(dev):
        if use_gemv:
            status = L.atlas_qlinear_gemv(*args, flag, _capi.stream_ptr(dev))
            _capi.check(status, "atlas_qlinear_gemv")
        else:
            ws_bytes = int(L.atlas_qlinear_gemm_workspace_bytes(m, n, k))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            status = L.atlas_qlinear_gemm(*args, ws.data_ptr(), ws_bytes, flag, _capi.stream_ptr(dev))
            _capi.check(status, "atlas_qlinear_gemm")
    return y.view(*x.shape[:-1], n)


class QuantizedLinear(nn.Module):
    """A linear layer whose weight is a ``QuantizedTensor`` (reference :21-83)."""

    def __init__(self, quantized_weights: "QuantizedTensor", bias: Optional[torch.Tensor]):
        super().__init__()
        self.quantized_weights = quantized_weights
        self.bias = bias
        self.original_shape = getattr(quantized_weights, "original_shape", None)
        self._kernel_layout: Optional[KernelLayout] = None

    def _layout_for(self, q: QuantizedTensor) -> KernelLayout:
        lay = self._kernel_layout
        if lay is None or lay.source is not q or lay.tiles.device != q.fp8_data.device:
            lay = build_kernel_layout(q)
            self._kernel_layout = lay
        return lay

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q_tensor = self.quantized_weights
        if not hasattr(q_tensor, "fp8_data"):
            raise TypeError(
                f"Weight in QuantizedLinear ({id(self)}) is not a valid QuantizedTensor: {type(q_tensor)}")
        # the kernels need a GPU; CPU activations are staged through it and the result returned
        compute_device = x.device if x.device.type == "cuda" else _capi.require_cuda()
        if q_tensor.fp8_data.device != compute_device:
            if _VERBOSE:
                print(f"QuantizedLinear {id(self)}: weights {q_tensor.fp8_data.device} -> {compute_device}")
            self.quantized_weights = q_tensor.to(compute_device)
            q_tensor = self.quantized_weights
        bias = self.bias
        if bias is not None and bias.device != compute_device:
            self.bias = bias.to(compute_device)
            bias = self.bias
        layout = self._layout_for(q_tensor)
        xin = x if x.device == compute_device else x.to(compute_device)
        y = quantized_linear_forward(xin, layout, bias)
        return y if x.device == compute_device else y.to(x.device)

    def extra_repr(self) -> str:
        q_shape, q_device = None, "N/A"
        if getattr(self, "quantized_weights", None):
            q_shape = self.original_shape
            try:
                q_device = self.quantized_weights.fp8_data.device
            except AttributeError:
                pass
        return f"quantized_shape={q_shape}, bias={self.bias is not None}, device={q_device}"
