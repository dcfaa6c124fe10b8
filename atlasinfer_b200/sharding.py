"""Multi-GPU plumbing of the quantization path: one process per GPU.

The reference is single-process (it has no ``torch.distributed`` import); this
module adds the two partitionings its path admits:

* whole-model quantization shards by layer -- every tensor is independent, so
  ranks quantize disjoint layers and no collective is involved;
* the quantized linear shards column-parallel by output features: rank r owns
  rows [r*N/g, (r+1)*N/g) of every W[N, K] and the shards of y are
  all-gathered (NCCL over NVLink).  Because in_features is a multiple of the
  block size, a row range is a contiguous slice of codes and scales and a
  re-based slice of the outlier streams, and quantizing the shard gives the
  same streams as slicing the quantized whole.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .quant.adaptive_quantizer import QuantizedTensor


def split_range(n: int, parts: int, index: int) -> Tuple[int, int]:
    """Balanced contiguous split of range(n): bounds of part ``index``."""
    if not (0 <= index < parts):
        raise ValueError(f"part {index} outside [0, {parts})")
    return n * index // parts, n * (index + 1) // parts


def layers_for_rank(n_layers: int, world_size: int, rank: int) -> range:
    """Layers quantized by ``rank`` (contiguous block; no data-path collective)."""
    lo, hi = split_range(n_layers, world_size, rank)
    return range(lo, hi)


def row_bounds(n_rows: int, world_size: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """Rows of a column-parallel weight owned by ``rank``; bounds are multiples of ``multiple``."""
    units = n_rows // multiple
    if units * multiple != n_rows:
        raise ValueError(f"{n_rows} rows are not a multiple of {multiple}")
    lo, hi = split_range(units, world_size, rank)
    return lo * multiple, hi * multiple


def shard_rows(q: QuantizedTensor, row_lo: int, row_hi: int) -> QuantizedTensor:
    """The QuantizedTensor of rows [row_lo, row_hi) of a quantized [N, K] weight.

    Needs K % block_size == 0 (blocks never straddle rows).  Works on any device.
    """
    if len(q.original_shape) != 2:
        raise ValueError("shard_rows expects a 2-D weight")
    n, k = int(q.original_shape[0]), int(q.original_shape[1])
    bs = int(q.block_size)
    if k % bs != 0:
        raise NotImplementedError(f"in_features {k} is not a multiple of block_size {bs}")
    if not (0 <= row_lo <= row_hi <= n):
        raise ValueError(f"rows [{row_lo}, {row_hi}) outside [0, {n})")
    idx = q.outlier_indices
    bounds = torch.tensor([row_lo * k, row_hi * k], dtype=idx.dtype, device=idx.device)
    o_lo, o_hi = (int(v) for v in torch.searchsorted(idx, bounds).tolist())
    c_lo, c_hi = row_lo * k - o_lo, row_hi * k - o_hi  # codes before a position = position - outliers before it
    return QuantizedTensor(
        fp8_data=q.fp8_data[c_lo:c_hi],
        fp16_outliers=q.fp16_outliers[o_lo:o_hi],
        outlier_indices=idx[o_lo:o_hi] - row_lo * k,
        scale_factors=q.scale_factors[row_lo * k // bs: row_hi * k // bs],
        original_shape=torch.Size((row_hi - row_lo, k)),
        block_size=q.block_size,
    )


def gather_columns(y_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                   sizes: Optional[Sequence[int]] = None) -> torch.Tensor:
    """All-gather the per-rank output shards [..., N_r] into [..., sum N_r] (rank order)."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    y_local = y_local.contiguous()
    lead = y_local.shape[:-1]
    if sizes is None or len(set(sizes)) == 1:
        flat = y_local.reshape(-1, y_local.shape[-1])
        out = torch.empty((world * flat.shape[0], flat.shape[1]), dtype=flat.dtype, device=flat.device)
        dist.all_gather_into_tensor(out, flat, group=group)  # rank r's rows land at [r*M, (r+1)*M)
        out = out.view(world, flat.shape[0], flat.shape[1]).transpose(0, 1)
        return out.reshape(*lead, world * flat.shape[1])
    # shards of different widths: collectives want equal sizes, so every rank pads its shard to the widest one
    flat = y_local.reshape(-1, y_local.shape[-1])
    widest = max(int(s) for s in sizes)
    padded = flat if flat.shape[1] == widest else torch.nn.functional.pad(flat, (0, widest - flat.shape[1]))
    out = torch.empty((world * flat.shape[0], widest), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out, padded.contiguous(), group=group)
    out = out.view(world, flat.shape[0], widest)
    parts: List[torch.Tensor] = [out[r, :, :int(s)] for r, s in enumerate(sizes)]
    return torch.cat(parts, dim=-1).reshape(*lead, sum(int(s) for s in sizes))


class ColumnParallelQuantizedLinear(nn.Module):
    """Rank-local rows of a QuantizedLinear plus the all-gather of the outputs.

    ``local`` is a ``QuantizedLinear`` over this rank's rows (and bias slice);
    ``forward`` returns the full [..., N] output on every rank.
    """

    def __init__(self, local: nn.Module, shard_sizes: Sequence[int], group: Optional[dist.ProcessGroup] = None):
        super().__init__()
        self.local = local
        self.shard_sizes = [int(s) for s in shard_sizes]
        self.group = group

    @classmethod
    def from_full(cls, q: QuantizedTensor, bias: Optional[torch.Tensor], rank: int, world_size: int,
                  group: Optional[dist.ProcessGroup] = None, row_multiple: int = 16):
        from .integration.atlas_wrappers import QuantizedLinear
        n = int(q.original_shape[0])
        mult = row_multiple if n % (row_multiple * world_size) == 0 else 1
        bounds = [row_bounds(n, world_size, r, mult) for r in range(world_size)]
        lo, hi = bounds[rank]
        local = QuantizedLinear(shard_rows(q, lo, hi), None if bias is None else bias[lo:hi].clone())
        return cls(local, [b[1] - b[0] for b in bounds], group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return gather_columns(self.local(x), self.group, self.shard_sizes)
