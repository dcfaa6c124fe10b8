"""ctypes binding of ``libatlas_b200.so`` (declared in ``include/atlas_b200.h``).

The library is the only compute path of this package: if it is missing, or no
sm_100a GPU is usable, calls raise -- there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libatlas_b200.so")

OK, ERR_BAD_ARGUMENT, ERR_UNSUPPORTED, ERR_CAPACITY, ERR_LAUNCH, ERR_TIMEOUT, ERR_NO_DEVICE = range(7)
DTYPE_F16, DTYPE_BF16 = 0, 1

# every symbol include/atlas_b200.h declares
EXPORTS = (
    "atlas_version", "atlas_last_error", "atlas_status_string",
    "atlas_quantize_workspace_bytes", "atlas_quantize", "atlas_quantize_noalloc", "atlas_dequantize",
    "atlas_tiles_bytes", "atlas_repack", "atlas_qlinear_gemv",
    "atlas_qlinear_stream_workspace_bytes", "atlas_qlinear_stream", "atlas_qlinear_stream_gather",
    "atlas_peer_wait", "atlas_peer_push", "atlas_peer_alloc", "atlas_peer_free", "atlas_peer_export", "atlas_peer_import",
    "atlas_peer_release",
    "atlas_qlinear_gemm_workspace_bytes", "atlas_qlinear_gemm", "atlas_qlinear_gemm_gather",
)

MAX_PEERS = 8
PEER_HANDLE_BYTES = 64


class PeerGather(ctypes.Structure):
    """``AtlasPeerGather`` of include/atlas_b200.h."""

    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("y_dst", ctypes.c_void_p * MAX_PEERS), ("flags_dst", ctypes.c_void_p * MAX_PEERS),
                ("state", ctypes.c_void_p), ("wait_flags", ctypes.c_void_p), ("poll_limit", ctypes.c_int64)]


_lib: Optional[ctypes.CDLL] = None


class AtlasError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def load() -> ctypes.CDLL:
    """Load the C-ABI library, or raise with build instructions."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"atlasinfer_b200: {LIB_PATH} is missing. Build it with "
            "`python -m atlasinfer_b200.build` (needs nvcc); there is no fallback path.")
    L = ctypes.CDLL(LIB_PATH)
    vp, i64, i32, f64, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_double, ctypes.c_size_t
    L.atlas_version.restype = i32
    L.atlas_last_error.restype = ctypes.c_char_p
    L.atlas_status_string.restype = ctypes.c_char_p
    L.atlas_status_string.argtypes = [i32]
    L.atlas_quantize_workspace_bytes.restype = sz
    L.atlas_quantize_workspace_bytes.argtypes = [i64, i32]
    L.atlas_quantize.restype = i32
    L.atlas_quantize.argtypes = [vp, i64, i32, f64, vp, vp, vp, i64, vp, vp, vp, sz, vp]
    L.atlas_quantize_noalloc.restype = i32
    L.atlas_quantize_noalloc.argtypes = [vp, i64, i32, f64, vp, vp, vp, i64, vp, vp, vp]
    L.atlas_dequantize.restype = i32
    L.atlas_dequantize.argtypes = [vp, i64, vp, vp, i64, vp, i64, i32, vp, vp]
    L.atlas_tiles_bytes.restype = sz
    L.atlas_tiles_bytes.argtypes = [i64, i64]
    L.atlas_repack.restype = i32
    L.atlas_repack.argtypes = [vp, i64, vp, vp, i64, vp, i64, i64, i32, vp, vp, vp, vp, vp, vp, vp]
    lin = [vp, i32, i64, i64, vp, vp, vp, vp, vp, i64, i64, i32, vp, vp, i64]
    L.atlas_qlinear_gemv.restype = i32
    L.atlas_qlinear_gemv.argtypes = lin + [vp, vp]
    L.atlas_qlinear_stream_workspace_bytes.restype = sz
    L.atlas_qlinear_stream_workspace_bytes.argtypes = [i64]
    L.atlas_qlinear_stream.restype = i32
    L.atlas_qlinear_stream.argtypes = lin + [vp, sz, vp, vp]
    L.atlas_qlinear_stream_gather.restype = i32
    L.atlas_qlinear_stream_gather.argtypes = lin[:13] + [i64, vp, sz, vp, vp, ctypes.POINTER(PeerGather)]
    L.atlas_qlinear_gemm_gather.restype = i32
    L.atlas_qlinear_gemm_gather.argtypes = lin[:13] + [i64, vp, sz, vp, vp, ctypes.POINTER(PeerGather)]
    L.atlas_peer_wait.restype = i32
    L.atlas_peer_wait.argtypes = [vp, i32, vp, i64, vp, vp]
    L.atlas_peer_push.restype = i32
    L.atlas_peer_push.argtypes = [vp, i64, i64, i64, i64, ctypes.POINTER(PeerGather), vp]
    L.atlas_peer_alloc.restype = i32
    L.atlas_peer_alloc.argtypes = [sz, ctypes.POINTER(vp)]
    L.atlas_peer_free.restype = i32
    L.atlas_peer_free.argtypes = [vp]
    L.atlas_peer_export.restype = i32
    L.atlas_peer_export.argtypes = [vp, ctypes.c_char_p]
    L.atlas_peer_import.restype = i32
    L.atlas_peer_import.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    L.atlas_peer_release.restype = i32
    L.atlas_peer_release.argtypes = [vp]
    L.atlas_qlinear_gemm_workspace_bytes.restype = sz
    L.atlas_qlinear_gemm_workspace_bytes.argtypes = [i64, i64, i64]
    L.atlas_qlinear_gemm.restype = i32
    L.atlas_qlinear_gemm.argtypes = lin + [vp, sz, vp, vp]
    _lib = L
    return L


def check(status: int, what: str) -> None:
    if status == OK:
        return
    L = load()
    detail = (L.atlas_last_error() or b"").decode()
    kind = (L.atlas_status_string(status) or b"").decode()
    msg = f"{what}: {kind}" + (f" ({detail})" if detail else "")
    if status == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise AtlasError(status, msg)


def require_cuda(device: Optional[torch.device] = None) -> torch.device:
    """The CUDA device work is staged on; raises when there is none."""
    if device is not None and device.type == "cuda":
        return device
    if not torch.cuda.is_available():
        raise RuntimeError(
            "atlasinfer_b200 computes on a B200 GPU only and none is visible; "
            "there is no CPU implementation to fall back to")
    return torch.device("cuda", torch.cuda.current_device())


def stream_ptr(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None or t.numel() == 0:
        return None
    return int(t.data_ptr())
