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

# rows of x up to which the per-strip streaming kernel is used (8 rows per pass over the weight); above it the
# tcgen05 kernel.  The persistent streaming kernel takes up to STREAM_MAX_ROWS rows in one pass; it is what the
# column-parallel linear with the fused gather runs on and can be asked for with force="stream".
GEMV_MAX_ROWS = 16
STREAM_MAX_ROWS = 32

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
    """Synchronise and raise if any kernel on ``dev`` reported a timed-out wait.

    The linear kernels never stall the host: a bounded wait that runs out inside a kernel (a copy that never
    lands, a peer that never arrives) sets a per-device status word and the kernel finishes on what it has.
    ``QuantizedLinear.forward`` does not read the word (that would synchronise every call); a caller that wants
    the check calls this where a synchronisation is acceptable, e.g. once per generated token or per batch.
    The word is cleared when the error is raised."""
    if int(status_word(dev).item()) != 0:
        status_word(dev).zero_()
        raise _capi.AtlasError(_capi.ERR_TIMEOUT, "a quantized-linear kernel gave up on a bounded wait")


_stream_workspaces = {}


def stream_workspace(dev: torch.device) -> torch.Tensor:
    """Scratch of the persistent streaming kernel on ``dev``: tickets and fp32 partial tiles.

    Zero-filled once; every launch leaves it zero-filled where it must be.  One per device: launches that use it
    must be ordered with respect to each other."""
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _stream_workspaces.get(index)
    if t is None:
        L = _capi.load()
        t = torch.zeros(int(L.atlas_qlinear_stream_workspace_bytes(STREAM_MAX_ROWS)), dtype=torch.uint8, device=dev)
        _stream_workspaces[index] = t
    return t


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
    # the linear kernels read the weight-side buffers before the stream's earlier work has completed
    # (programmatic dependent launch), so the layout must be final before any of them is launched
    torch.cuda.current_stream(dev).synchronize()
    return KernelLayout(q, tiles, scales_tiled, row_ptr, chunk_ptr, entries, vals_sorted, n, k, bs)


def quantized_linear_forward(x: torch.Tensor, layout: KernelLayout, bias: Optional[torch.Tensor],
                             force: Optional[str] = None) -> torch.Tensor:
    """``x @ W^T + bias`` on CUDA tensors through the C ABI.

    ``force``: "gemv" (per-strip streaming kernel), "gemm" (tcgen05 kernel) or "stream" (persistent streaming
    kernel, one pass for up to 32 rows); default: "gemv" up to 16 rows of x, "gemm" above."""
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
    if force is None:
        force = "gemv" if m <= GEMV_MAX_ROWS else "gemm"
    if force not in ("stream", "gemv", "gemm"):
        raise ValueError(f"force={force!r}")
    args = [x2.data_ptr(), dtype, m, ldx, layout.tiles.data_ptr(), layout.scales_tiled.data_ptr(),
            layout.chunk_ptr.data_ptr(), _capi.ptr(layout.entries), _capi.ptr(layout.vals_sorted), n, k,
            layout.block_size, _capi.ptr(b), y.data_ptr(), n]
    flag = status_word(dev).data_ptr()
    with torch.cuda.device(dev):
        if force == "stream":
            ws = stream_workspace(dev)
            status = L.atlas_qlinear_stream(*args, ws.data_ptr(), ws.numel(), flag, _capi.stream_ptr(dev))
            _capi.check(status, "atlas_qlinear_stream")
        elif force == "gemv":
            status = L.atlas_qlinear_gemv(*args, flag, _capi.stream_ptr(dev))
            _capi.check(status, "atlas_qlinear_gemv")
        else:
            ws_bytes = int(L.atlas_qlinear_gemm_workspace_bytes(m, n, k))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            status = L.atlas_qlinear_gemm(*args, ws.data_ptr(), ws_bytes, flag, _capi.stream_ptr(dev))
            _capi.check(status, "atlas_qlinear_gemm")
    return y.view(*x.shape[:-1], n)


def concat_layouts(layouts) -> KernelLayout:
    """One kernel layout whose rows are those of ``layouts`` back to back (same in_features and block size).

    Every member but the last is padded to a whole number of 128-row tiles (its own layout already is), so a
    member is a contiguous run of tiles, scales and strips of the result, and one launch over the result
    computes all members.  Row ``i`` of member ``j`` is row ``offsets[j] + i`` of the result."""
    first = layouts[0]
    if any(l.n_cols != first.n_cols or l.block_size != first.block_size for l in layouts):
        raise ValueError("fused linears must share in_features and block size")
    k_tiles = first.n_cols // 64
    chunk_ptrs, base = [], 0
    for l in layouts:
        chunk_ptrs.append(l.chunk_ptr + base)          # entry indices become positions in the joined list
        base += l.entries.numel()
    padded = [(l.n_rows + 127) // 128 * 128 for l in layouts]
    n_rows = sum(padded[:-1]) + layouts[-1].n_rows
    dev = first.tiles.device
    row_ptr = torch.empty(0, dtype=torch.int32, device=dev)   # CSR view of the canonical streams: not joined
    assert all(l.chunk_ptr.numel() == (p_ // 16) * (k_tiles + 1) for l, p_ in zip(layouts, padded))
    return KernelLayout(tuple(l.source for l in layouts), torch.cat([l.tiles for l in layouts]),
                        torch.cat([l.scales_tiled for l in layouts]), row_ptr, torch.cat(chunk_ptrs),
                        torch.cat([l.entries for l in layouts]), torch.cat([l.vals_sorted for l in layouts]),
                        n_rows, first.n_cols, first.block_size)


def slice_layout(fused: KernelLayout, row_offset: int, n_rows: int, source, entry_count: Optional[int] = None) -> KernelLayout:
    """The member of a fused layout that starts at ``row_offset`` (a multiple of 128), as views of its buffers."""
    if row_offset % 128:
        raise ValueError("members of a fused layout start on 128-row boundaries")
    k, bs = fused.n_cols, fused.block_size
    k_tiles = k // 64
    n_pad = (n_rows + 127) // 128 * 128
    t0, s0, c0 = row_offset * k, row_offset * (k // bs), (row_offset // 16) * (k_tiles + 1)
    return KernelLayout(source, fused.tiles[t0:t0 + n_pad * k], fused.scales_tiled[s0:s0 + n_pad * (k // bs)],
                        fused.row_ptr, fused.chunk_ptr[c0:c0 + (n_pad // 16) * (k_tiles + 1)],
                        fused.entries, fused.vals_sorted, n_rows, k, bs)


class FusedLinearGroup:
    """Several ``QuantizedLinear`` layers that read the same activations, computed by one launch.

    The reference issues q/k/v (and gate/up) as separate ``F.linear`` calls on the same input
    (integration/atlas_wrappers.py:67, once per module).  Here the members' kernel layouts are joined row-wise
    (``concat_layouts``); the first member that is called with an input computes the joined product and the
    other members, called with the very same tensor, return their slice of it (for prompt-sized inputs this
    also means one bf16 -> fp16 conversion of the activations instead of one per member).  A member called
    with any other input computes the joined product anew.  A member's slice equals its stand-alone output up to the rounding of
    the fp32 partial sums (the K range of a row tile is cut between CTAs at other places when the launch
    covers more rows), not bit for bit.
    """

    def __init__(self, members):
        self.members = list(members)
        self.layout: Optional[KernelLayout] = None
        self.bias: Optional[torch.Tensor] = None
        self.offsets = []
        self._cache = None      # (x, x._version, y_all, members served)
        self.launches = 0       # joined launches issued (for tests and launch counting)
        for i, mod in enumerate(self.members):
            mod._group = self
            mod._group_index = i

    def build(self, dev: torch.device) -> None:
        layouts = []
        for mod in self.members:
            q = mod.quantized_weights
            if q.fp8_data.device != dev:
                q = q.to(dev)
                mod.quantized_weights = q
            if mod.bias is not None and mod.bias.device != dev:
                mod.bias = mod.bias.to(dev)
            layouts.append(mod._layout_for(q))
        fused = concat_layouts(layouts)
        self.offsets, off = [], 0
        for lay in layouts:
            self.offsets.append(off)
            off += (lay.n_rows + 127) // 128 * 128
        if any(mod.bias is not None for mod in self.members):
            b = torch.zeros(fused.n_rows, dtype=torch.float16, device=dev)
            for mod, lay, o in zip(self.members, layouts, self.offsets):
                if mod.bias is not None:
                    b[o:o + lay.n_rows] = mod.bias.to(torch.float16)
            self.bias = b
        # the members now look at the joined buffers; their own copies are released
        for mod, lay, o in zip(self.members, layouts, self.offsets):
            mod._kernel_layout = slice_layout(fused, o, lay.n_rows, lay.source)
        self.layout = fused
        torch.cuda.current_stream(dev).synchronize()

    def member_forward(self, index: int, x: torch.Tensor) -> Optional[torch.Tensor]:
        """Member ``index``'s output for ``x``, or None if the group does not apply (the member computes alone)."""
        if x.device.type != "cuda" or x.dtype not in (torch.float16, torch.bfloat16):
            return None
        rows = x.numel() // x.shape[-1] if x.shape[-1] else 0
        if rows == 0:
            return None
        if self.layout is None or self.layout.tiles.device != x.device:
            self.build(x.device)
        c = self._cache
        if c is None or c[0] is not x or c[1] != x._version or index in c[3]:
            y_all = quantized_linear_forward(x, self.layout, self.bias)
            self.launches += 1
            c = (x, x._version, y_all, set())
            self._cache = c
        c[3].add(index)
        off = self.offsets[index]
        n = self.members[index].original_shape[0]
        out = c[2][..., off:off + n]
        if len(c[3]) == len(self.members):
            self._cache = None   # everyone has been served: do not keep x and y alive
        return out


def fuse_linears(members) -> FusedLinearGroup:
    """Join ``QuantizedLinear`` layers that share their input (e.g. q/k/v, gate/up) into one launch."""
    members = list(members)
    shapes = {(tuple(m.original_shape)[1], int(m.quantized_weights.block_size)) for m in members}
    if len(shapes) != 1:
        raise ValueError(f"fused linears must share in_features and block size, got {sorted(shapes)}")
    return FusedLinearGroup(members)


class QuantizedLinear(nn.Module):
    """A linear layer whose weight is a ``QuantizedTensor`` (reference :21-83)."""

    def __init__(self, quantized_weights: "QuantizedTensor", bias: Optional[torch.Tensor]):
        super().__init__()
        self.quantized_weights = quantized_weights
        self.bias = bias
        self.original_shape = getattr(quantized_weights, "original_shape", None)
        self._kernel_layout: Optional[KernelLayout] = None
        self._group: Optional[FusedLinearGroup] = None   # set by fuse_linears
        self._group_index = 0
        self._bias_f16 = None   # (bias it was made from, its fp16 contiguous image)

    def _bias_for(self, bias: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """The bias as the kernels want it (fp16, contiguous), converted once per bias tensor and made
        final before any kernel that reads it is launched."""
        if bias is None or (bias.dtype == torch.float16 and bias.is_contiguous()):
            return bias
        cached = self._bias_f16
        if cached is None or cached[0] is not bias:
            image = bias.to(torch.float16).contiguous()
            if image.device.type == "cuda":
                torch.cuda.current_stream(image.device).synchronize()
            cached = (bias, image)
            self._bias_f16 = cached
        return cached[1]

    def _layout_for(self, q: QuantizedTensor) -> KernelLayout:
        lay = self._kernel_layout
        if lay is None or lay.source is not q or lay.tiles.device != q.fp8_data.device:
            lay = build_kernel_layout(q)
            self._kernel_layout = lay
        return lay

    def offload_canonical(self, device="cpu") -> None:
        """Keep only the kernel layout on the GPU: the canonical streams move to ``device`` (host by default).

        The module then holds ~1.03 bytes per weight of GPU memory instead of ~2.07 (canonical streams +
        kernel layout).  ``quantized_weights`` stays a complete ``QuantizedTensor`` (for saving, dequantizing,
        ``memory_footprint``); the forward keeps using the layout that was built from it."""
        q = self.quantized_weights
        dev = q.fp8_data.device
        if dev.type != "cuda":
            return
        lay = self._layout_for(q)
        moved = q.to(torch.device(device))
        self.quantized_weights = moved
        if self._group is not None and self._group.layout is not None:
            srcs = tuple(moved if s_ is q else s_ for s_ in self._group.layout.source)
            self._group.layout = self._group.layout._replace(source=srcs)
        self._kernel_layout = lay._replace(source=moved)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q_tensor = self.quantized_weights
        if not hasattr(q_tensor, "fp8_data"):
            raise TypeError(
                f"Weight in QuantizedLinear ({id(self)}) is not a valid QuantizedTensor: {type(q_tensor)}")
        if self._group is not None:
            y = self._group.member_forward(self._group_index, x)
            if y is not None:
                return y
        # the kernels need a GPU; CPU activations are staged through it and the result returned
        compute_device = x.device if x.device.type == "cuda" else _capi.require_cuda()
        lay = self._kernel_layout
        if lay is not None and lay.source is q_tensor and lay.tiles.device == compute_device:
            # the kernel image of these very streams is already on the device (the streams themselves may have
            # been moved off it by offload_canonical)
            bias = self.bias
            if bias is not None and bias.device != compute_device:
                self.bias = bias.to(compute_device)
                bias = self.bias
            xin = x if x.device == compute_device else x.to(compute_device)
            y = quantized_linear_forward(xin, lay, self._bias_for(bias))
            return y if x.device == compute_device else y.to(x.device)
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
        y = quantized_linear_forward(xin, layout, self._bias_for(bias))
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
