"""Column-parallel quantized linear whose all-gather is done by the kernel itself.

The reference is single-process; this is the multi-GPU form of its linear for the 70B-shaped configuration:
rank r owns a slice of the output rows of every weight (``sharding.shard_rows``), and instead of writing its
[m, N/g] shard locally and calling an NCCL all-gather (``sharding.gather_columns``), the rank stores the shard
straight into every rank's gathered [m, N] buffer over NVLink and then publishes an arrival count; the next
kernel that consumes the buffer waits (bounded) until all ranks have arrived.  The shards are 64 KB - 1.8 MB,
so what this removes is the collective's launch and synchronisation latency, per linear.  The stores are either
the epilogue of the streaming linear kernel (``kernel="stream"``: one launch does the linear, the wait and the
gather), part of the tcgen05 path (``kernel="gemm"``, up to 64 rows of x: its fp16 copy kernel waits, the kernel
that adds the K slices stores to every rank; no extra launch), or a small push kernel behind the default linear
kernels (``kernel="push"``: any number of rows), with the wait as a kernel of its own in front.

One process per GPU of one node.  ``PeerArena`` owns the memory the ranks share: each rank allocates an arena
of the same size (``atlas_peer_alloc``: plain cudaMalloc memory), the ranks exchange CUDA IPC handles through
``torch.distributed`` and map each other's arenas; buffers are carved at the same offsets on every rank.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _capi
from .integration import atlas_wrappers as aw

DEFAULT_POLL_LIMIT = 1 << 22      # ~0.5 s of polling before a wait gives up


class PeerArena:
    """Symmetric device memory of the ranks of ``group`` (every rank calls this with the same ``nbytes``)."""

    HEADER = 4096   # arrival flags (world x uint32) and this rank's gather state (2 x uint32), zero-filled

    def __init__(self, nbytes: int, device: torch.device, group: Optional[dist.ProcessGroup] = None,
                 world: Optional[int] = None, rank: Optional[int] = None, exchange: bool = True):
        self.L = _capi.load()
        self.device = device
        self.group = group
        self.world = dist.get_world_size(group) if world is None else world
        self.rank = dist.get_rank(group) if rank is None else rank
        if self.world > _capi.MAX_PEERS:
            raise ValueError(f"at most {_capi.MAX_PEERS} ranks share a weight, got {self.world}")
        self.nbytes = self.HEADER + (int(nbytes) + 255) // 256 * 256
        self._cursor = self.HEADER
        self._imported = exchange
        with torch.cuda.device(device):
            base = ctypes.c_void_p()
            _capi.check(self.L.atlas_peer_alloc(self.nbytes, ctypes.byref(base)), "atlas_peer_alloc")
            self.base = int(base.value)
            self.bases: List[int] = [0] * self.world
            self.bases[self.rank] = self.base
            if self.world > 1 and exchange:
                handle = ctypes.create_string_buffer(_capi.PEER_HANDLE_BYTES)
                _capi.check(self.L.atlas_peer_export(self.base, handle), "atlas_peer_export")
                handles: List[Optional[bytes]] = [None] * self.world
                dist.all_gather_object(handles, handle.raw, group=group)
                for r, h in enumerate(handles):
                    if r == self.rank:
                        continue
                    ptr = ctypes.c_void_p()
                    _capi.check(self.L.atlas_peer_import(h, ctypes.byref(ptr)), "atlas_peer_import")
                    self.bases[r] = int(ptr.value)
        self._closed = False

    @classmethod
    def on_one_device(cls, nbytes: int, device: torch.device, world: int) -> List["PeerArena"]:
        """``world`` arenas in THIS process on one GPU, wired to each other like the arenas of ``world`` ranks.

        For single-GPU tests of the addressing and flag logic: the "ranks" are then run one after the other on one
        stream (kernels that wait for each other must never be separate launches on one GPU)."""
        arenas = [cls(nbytes, device, world=world, rank=r, exchange=False) for r in range(world)]
        for a in arenas:
            a.bases = [b.base for b in arenas]
        return arenas

    # flags live at offset 0, the gather state at offset 256 of every arena
    def flags_ptr(self, rank: int) -> int:
        return self.bases[rank]

    @property
    def state_ptr(self) -> int:
        return self.base + 256

    def carve(self, nbytes: int) -> int:
        """Offset of a fresh ``nbytes`` region (256-byte aligned); every rank must carve in the same order."""
        off = self._cursor
        self._cursor += (int(nbytes) + 255) // 256 * 256
        if self._cursor > self.nbytes:
            raise RuntimeError("PeerArena is full")
        return off

    def local_tensor(self, offset: int, shape, dtype) -> torch.Tensor:
        """A tensor view of this rank's own arena at ``offset`` (the arena must outlive it)."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        iface = {"shape": (nbytes,), "typestr": "|u1", "data": (self.base + offset, False), "version": 3}
        holder = type("_ArenaView", (), {"__cuda_array_interface__": iface})()
        return torch.as_tensor(holder, device=self.device).view(dtype).view(*shape)

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        if self.world > 1 and self._imported:
            dist.barrier(group=self.group)     # nobody unmaps while a peer may still store into its arena
        with torch.cuda.device(self.device):
            if self._imported:
                for r, b in enumerate(self.bases):
                    if r != self.rank and b:
                        self.L.atlas_peer_release(b)
            self.L.atlas_peer_free(self.base)


class GatheredLinear:
    """One column-parallel launch: this rank's rows of a (possibly fused) weight, output gathered on every rank.

    ``layout`` is the rank-local kernel layout; ``out`` is the gathered [m_max, world * n_local] buffer in the arena
    (same offset on every rank); ``__call__`` runs the kernel, which stores this rank's columns into every rank's
    ``out`` and publishes the arrival.  ``wait=True`` makes the kernel wait, before it reads x, until every rank has
    completed as many gather launches as this rank (x is the output of the previous gathered launch)."""

    def __init__(self, arena: PeerArena, layout: aw.KernelLayout, m_max: int, dtype: torch.dtype,
                 bias: Optional[torch.Tensor] = None, poll_limit: int = DEFAULT_POLL_LIMIT, kernel: str = "stream"):
        if kernel not in ("stream", "gemm", "push"):
            raise ValueError(f"kernel={kernel!r}")
        self.kernel = kernel
        self.arena = arena
        self.layout = layout
        self.bias = bias
        self.m_max = int(m_max)
        self.dtype = dtype
        self.width = layout.n_rows * arena.world
        self.offset = arena.carve(self.m_max * self.width * 2)
        self.out = arena.local_tensor(self.offset, (self.m_max, self.width), dtype)
        g = _capi.PeerGather()
        g.world, g.rank = arena.world, arena.rank
        for d in range(arena.world):
            g.y_dst[d] = arena.bases[d] + self.offset + arena.rank * layout.n_rows * 2
            g.flags_dst[d] = arena.flags_ptr(d)
        g.state = arena.state_ptr
        g.wait_flags = None
        g.poll_limit = int(poll_limit)
        self._desc = g
        self._desc_wait = _capi.PeerGather.from_buffer_copy(g)
        self._desc_wait.wait_flags = arena.flags_ptr(arena.rank)

    def __call__(self, x: torch.Tensor, wait: bool = False) -> torch.Tensor:
        L = self.arena.L
        lay = self.layout
        dev = x.device
        x2 = x.reshape(-1, lay.n_cols)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        m = x2.shape[0]
        if self.kernel == "push":
            if m > self.m_max:
                raise ValueError(f"{m} rows of x; this gathered linear was set up for {self.m_max}")
            if wait:
                self.wait_for_all()
            y = aw.quantized_linear_forward(x2, lay, self.bias)       # [m, n_local], this rank's columns
            with torch.cuda.device(dev):
                st = L.atlas_peer_push(y.data_ptr(), m, lay.n_rows * 2, y.stride(0) * 2, self.width * 2,
                                       ctypes.byref(self._desc), _capi.stream_ptr(dev))
            _capi.check(st, "atlas_peer_push")
            return self.out[:m]
        dtype = _capi.DTYPE_F16 if x.dtype == torch.float16 else _capi.DTYPE_BF16
        desc = self._desc_wait if wait else self._desc
        if self.kernel == "gemm":
            if m > self.m_max or m > 64:
                raise ValueError(f"{m} rows of x; this gathered linear was set up for {min(self.m_max, 64)}")
            if m == 0:
                return self.out[:0]
            ws_bytes = int(L.atlas_qlinear_gemm_workspace_bytes(m, lay.n_rows, lay.n_cols))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            with torch.cuda.device(dev):
                st = L.atlas_qlinear_gemm_gather(
                    x2.data_ptr(), dtype, m, x2.stride(0) if m > 1 else lay.n_cols, lay.tiles.data_ptr(),
                    lay.scales_tiled.data_ptr(), lay.chunk_ptr.data_ptr(), _capi.ptr(lay.entries), _capi.ptr(lay.vals_sorted),
                    lay.n_rows, lay.n_cols, lay.block_size, _capi.ptr(self.bias), self.width, ws.data_ptr(), ws_bytes,
                    aw.status_word(dev).data_ptr(), _capi.stream_ptr(dev), ctypes.byref(desc))
            _capi.check(st, "atlas_qlinear_gemm_gather")
            return self.out[:m]
        if m > self.m_max or m > aw.STREAM_MAX_ROWS:
            raise ValueError(f"{m} rows of x; this gathered linear was set up for {min(self.m_max, aw.STREAM_MAX_ROWS)}")
        ws = aw.stream_workspace(dev)
        with torch.cuda.device(dev):
            st = L.atlas_qlinear_stream_gather(
                x2.data_ptr(), dtype, m, x2.stride(0) if m > 1 else lay.n_cols, lay.tiles.data_ptr(),
                lay.scales_tiled.data_ptr(), lay.chunk_ptr.data_ptr(), _capi.ptr(lay.entries), _capi.ptr(lay.vals_sorted),
                lay.n_rows, lay.n_cols, lay.block_size, _capi.ptr(self.bias), self.width, ws.data_ptr(), ws.numel(),
                aw.status_word(dev).data_ptr(), _capi.stream_ptr(dev), ctypes.byref(desc))
        _capi.check(st, "atlas_qlinear_stream_gather")
        return self.out[:m]

    def wait_for_all(self) -> None:
        """Enqueue the stand-alone wait: later work on the stream sees every rank's columns in ``out``."""
        dev = self.arena.device
        with torch.cuda.device(dev):
            st = self.arena.L.atlas_peer_wait(self.arena.flags_ptr(self.arena.rank), self.arena.world, self.arena.state_ptr,
                                              self._desc.poll_limit, aw.status_word(dev).data_ptr(), _capi.stream_ptr(dev))
        _capi.check(st, "atlas_peer_wait")
