"""The allocation-free quantize entry point (collected last on purpose).

Some hosts may not allocate device memory where they quantize -- a serving loop
with a fixed arena, a plug-in that does not own the allocator -- so
``atlas_quantize_noalloc`` keeps its look-back scratch in a device array inside
the library.  This test calls it directly through the C ABI, twice in a row on
different inputs (the second call must not see the first call's scratch), and
requires every output stream to equal, bit for bit, what ``atlas_quantize``
writes for the same input and, once, what the CPU oracle computes.
"""
import ctypes

import pytest
import torch

from atlasinfer_b200 import _capi
from oracle import atlas_oracle as O
from tests.util import bits, config_weights

pytestmark = pytest.mark.gpu
MAX_ELEMENTS = 1 << 26


def _buffers(numel, bs, dev):
    nb = (numel + bs - 1) // bs
    padded = nb * bs
    return dict(
        codes=torch.full((padded,), 77, dtype=torch.int8, device=dev),
        ovals=torch.zeros(padded, dtype=torch.float16, device=dev),
        oidx=torch.zeros(padded, dtype=torch.int64, device=dev),
        scales=torch.zeros(nb, dtype=torch.float16, device=dev),
        counts=torch.zeros(4, dtype=torch.int64, device=dev), padded=padded)


def _run(w, bs, thr, use_noalloc):
    L = _capi.load()
    dev = w.device
    b = _buffers(w.numel(), bs, dev)
    stream = _capi.stream_ptr(dev)
    common = [w.data_ptr(), w.numel(), bs, float(thr), b["codes"].data_ptr(), b["ovals"].data_ptr(),
              b["oidx"].data_ptr(), b["padded"], b["scales"].data_ptr(), b["counts"].data_ptr()]
    if use_noalloc:
        st = L.atlas_quantize_noalloc(*common, stream)
        _capi.check(st, "atlas_quantize_noalloc")
    else:
        ws_bytes = int(L.atlas_quantize_workspace_bytes(w.numel(), bs))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        st = L.atlas_quantize(*common, ws.data_ptr(), ws_bytes, stream)
        _capi.check(st, "atlas_quantize")
    n_codes, n_out, timed_out, _ = b["counts"].tolist()
    assert timed_out == 0
    return b["codes"][:n_codes], b["ovals"][:n_out], b["oidx"][:n_out], b["scales"]


def test_noalloc_matches_workspace_entry_point_twice(cuda_device):
    cases = [(config_weights(512, 2048, 31), 128, 3.0),          # 128 tiles
             (config_weights(300, 1000, 32).reshape(-1)[:299_001], 64, 2.5)]  # fewer tiles, ragged, other block
    for w, bs, thr in cases:  # two calls in a row through the same static scratch
        wd = w.to(cuda_device).contiguous()
        got = _run(wd, bs, thr, use_noalloc=True)
        want = _run(wd, bs, thr, use_noalloc=False)
        for a, b_ in zip(got, want):
            assert a.shape == b_.shape and torch.equal(bits(a), bits(b_))
    # and once more with the first input: stale scratch from a smaller call must not matter
    w, bs, thr = cases[0]
    wd = w.to(cuda_device).contiguous()
    got = _run(wd, bs, thr, True)
    for a, b_ in zip(got, _run(wd, bs, thr, False)):
        assert torch.equal(bits(a), bits(b_))
    # the same streams as the CPU oracle, so the entry point is checked against the reference arithmetic itself
    o = O.quantize(w, bs, thr)
    for a, b_ in zip(got, (o.fp8_data, o.fp16_outliers, o.outlier_indices, o.scale_factors)):
        assert a.shape == b_.shape and torch.equal(bits(a.cpu()), bits(b_))


def test_noalloc_rejects_sizes_beyond_its_limit(cuda_device):
    L = _capi.load()
    counts = torch.zeros(4, dtype=torch.int64, device=cuda_device)
    st = L.atlas_quantize_noalloc(None, MAX_ELEMENTS + 1, 128, 3.0, None, None, None, 0, None,
                                  counts.data_ptr(), None)
    assert st == _capi.ERR_CAPACITY
    assert b"static scratch limit" in L.atlas_last_error()
