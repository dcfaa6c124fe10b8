"""ctypes wrapper around ``atlas_oracle.c`` -- TEST INFRASTRUCTURE ONLY.

The oracle is the checker for the CUDA path: tests, the smoke check and the
benchmark's CPU-baseline leg call it; the product never does.  Parity status:
pinned against outputs of the unmodified reference quantizer
(``tests/golden/*.npz``, made by ``tests/golden/make_golden.py``).

All functions take and return CPU ``torch`` tensors.  fp16 tensors are passed
to C as their raw 16-bit patterns.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import NamedTuple, Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libatlas_oracle.so")
_lib = None

# torch's vectorised fp32 row sum used 8 lanes on the build that generated the
# golden fixtures (adaptive_quantizer.py:46 reaches it through torch.mean).
TORCH_SUM_LANES = 8


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile beside it and return the .so path."""
    src = os.path.join(_HERE, "atlas_oracle.c")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        vp, i64, i32, f64 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_double
        L.atlas_oracle_quantize.argtypes = [vp, i64, i32, f64, i32, vp, vp, vp, vp, vp, vp]
        L.atlas_oracle_quantize.restype = i32
        L.atlas_oracle_dequantize.argtypes = [vp, i64, vp, vp, i64, vp, i64, i32, vp]
        L.atlas_oracle_dequantize.restype = i32
        L.atlas_oracle_linear.argtypes = [vp, i64, i64, vp, i64, vp, vp]
        L.atlas_oracle_linear.restype = None
        L.atlas_oracle_row_sum_f32.argtypes = [vp, i64, i32]
        L.atlas_oracle_row_sum_f32.restype = ctypes.c_float
        L.atlas_oracle_threads.restype = i32
        _lib = L
    return _lib


class OracleQuantized(NamedTuple):
    """Field-for-field image of the reference ``QuantizedTensor`` (adaptive_quantizer.py:8-18)."""

    fp8_data: torch.Tensor          # int8, compacted non-outlier codes
    fp16_outliers: torch.Tensor     # fp16 raw outlier values
    outlier_indices: torch.Tensor   # int64 flat indices into the padded tensor
    scale_factors: torch.Tensor     # fp16, one per block
    original_shape: torch.Size
    block_size: int


def threads() -> int:
    return int(lib().atlas_oracle_threads())


def quantize(w: torch.Tensor, block_size: int = 128, z_threshold: float = 3.0,
             lanes: int = TORCH_SUM_LANES) -> OracleQuantized:
    """``quantize_tensor`` (adaptive_quantizer.py:51-148) on a CPU tensor."""
    if w.dtype != torch.float16:
        w = w.to(torch.float16)
    w = w.detach().cpu().contiguous()
    numel = w.numel()
    nb = (numel + block_size - 1) // block_size
    padded = nb * block_size
    codes = torch.empty(padded, dtype=torch.int8)
    ovals = torch.empty(padded, dtype=torch.float16)
    oidx = torch.empty(padded, dtype=torch.int64)
    scales = torch.empty(nb, dtype=torch.float16)
    nc = ctypes.c_int64(0)
    no = ctypes.c_int64(0)
    rc = lib().atlas_oracle_quantize(
        w.data_ptr(), numel, block_size, float(z_threshold), lanes,
        codes.data_ptr(), ovals.data_ptr(), oidx.data_ptr(), scales.data_ptr(),
        ctypes.byref(nc), ctypes.byref(no))
    if rc != 0:
        raise RuntimeError(f"atlas_oracle_quantize failed with {rc}")
    return OracleQuantized(codes[: nc.value].clone(), ovals[: no.value].clone(),
                           oidx[: no.value].clone(), scales, w.shape, block_size)


def dequantize(q) -> torch.Tensor:
    """``dequantize_tensor`` (adaptive_quantizer.py:156-251), cache left out."""
    shape = torch.Size(q.original_shape)
    numel = shape.numel()
    out = torch.zeros(numel, dtype=torch.float16)
    codes = q.fp8_data.cpu().contiguous()
    ovals = q.fp16_outliers.cpu().contiguous()
    oidx = q.outlier_indices.cpu().contiguous()
    scales = q.scale_factors.cpu().contiguous()
    rc = lib().atlas_oracle_dequantize(
        codes.data_ptr(), codes.numel(), ovals.data_ptr(), oidx.data_ptr(), oidx.numel(),
        scales.data_ptr(), numel, int(q.block_size), out.data_ptr())
    if rc != 0:
        raise RuntimeError("atlas_oracle_dequantize: inconsistent streams")
    return out.view(shape)


def linear(x: torch.Tensor, w_fp16: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 image of ``F.linear(x, dequantized_weight, bias)`` (atlas_wrappers.py:67).

    ``x`` is widened exactly to fp32, products are accumulated in fp64; the
    result (fp32, shape x.shape[:-1] + (N,)) is what linear outputs are held to
    within max|err| <= 1e-2 * rms.
    """
    w = w_fp16.detach().cpu().contiguous()
    assert w.dtype == torch.float16 and w.dim() == 2
    n, k = w.shape
    xf = x.detach().cpu().to(torch.float32).contiguous().view(-1, k)
    m = xf.shape[0]
    y = torch.empty(m, n, dtype=torch.float32)
    b = None
    if bias is not None:
        b = bias.detach().cpu().to(torch.float16).contiguous()
    lib().atlas_oracle_linear(xf.data_ptr(), m, k, w.data_ptr(), n,
                              b.data_ptr() if b is not None else None, y.data_ptr())
    return y.view(*x.shape[:-1], n)


def row_sum_f32(row: torch.Tensor, lanes: int = TORCH_SUM_LANES) -> float:
    r = row.detach().cpu().to(torch.float32).contiguous()
    return float(lib().atlas_oracle_row_sum_f32(r.data_ptr(), r.numel(), lanes))
