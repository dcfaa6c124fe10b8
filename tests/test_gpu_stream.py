"""Parity of the persistent streaming kernel (atlas_qlinear_stream) and of what is built on it:
fused sibling projections, host-resident canonical streams, row-sharded weights.

Every call goes through the C ABI.  Linear outputs are held to max|err| <= 1e-2 * rms(ref) against the
fp64-accumulated oracle product on the oracle's dequantized weight (raw for fp16 outputs; tests/util.py).
"""
import pytest
import torch

import atlasinfer_b200 as ab
from atlasinfer_b200 import _capi, sharding
from atlasinfer_b200.integration import atlas_wrappers
from oracle import atlas_oracle as O
from tests.util import bits, config_weights, rel_max_err

pytestmark = pytest.mark.gpu
LINEAR_TOL = 1e-2


def _case(n, k, m, dtype, seed, bias=True, bs=128, sigma=0.02, thr=3.0):
    w = config_weights(n, k, seed, sigma)
    o = O.quantize(w, bs, thr)
    gen = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(m, k, generator=gen).to(dtype)
    b = (torch.randn(n, generator=gen) * 0.02).half() if bias else None
    return o, x, b, O.linear(x, O.dequantize(o), b)


def _layout(o, dev):
    return atlas_wrappers.build_kernel_layout(ab.QuantizedTensor(*o).to(dev))


def _run(o, x, b, dev, force="stream"):
    y = atlas_wrappers.quantized_linear_forward(x.to(dev), _layout(o, dev), None if b is None else b.to(dev), force)
    atlas_wrappers.check_status(dev)
    return y


@pytest.mark.parametrize("m", [1, 2, 3, 4, 7, 8, 9, 15, 16, 17, 24, 31, 32, 33, 70])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_stream_matches_oracle(m, dtype, cuda_device):
    o, x, b, ref = _case(2048, 2048, m, dtype, 300 + m)
    y = _run(o, x, b, cuda_device)
    assert y.dtype == dtype and y.shape == (m, 2048)
    assert rel_max_err(y, ref, report=f"stream m={m}") < LINEAR_TOL


@pytest.mark.parametrize("n,k,bs", [(4096, 4096, 128), (11008, 4096, 128), (4096, 11008, 128), (1024, 8192, 128),
                                    (200, 256, 128), (16, 64, 64), (130, 192, 64), (3584, 8192, 128),
                                    (128, 28672, 128), (500, 1024, 32), (77, 512, 256), (300, 576, 96),
                                    (129, 64, 64), (1280, 8192, 128)])
def test_stream_shapes(n, k, bs, cuda_device):
    # row counts that are not multiples of 128, one-tile weights, K ranges cut between many CTAs (128 x 28672),
    # block sizes below / above / not commensurable with the 64-column tile
    for m, dtype in ((1, torch.bfloat16), (16, torch.bfloat16), (32, torch.float16)):
        o, x, b, ref = _case(n, k, m, dtype, n + k + m, bias=(m != 16), bs=bs)
        y = _run(o, x, b, cuda_device)
        err = rel_max_err(y, ref, report=f"stream {n}x{k} bs={bs} m={m}")
        assert err < LINEAR_TOL, f"{n}x{k} bs={bs} m={m} {dtype}: {err}"


@pytest.mark.parametrize("n,k,bs", [(256, 1024, 64), (200, 2048, 256), (512, 1024, 512), (130, 576, 96), (64, 320, 32),
                                    (1024, 11008, 128), (48, 256, 128)])
def test_per_strip_kernel_variants(n, k, bs, cuda_device):
    # the per-strip kernel's paths: one MMA tile with the single bf16 row staged in shared memory (m = 1), without
    # staging (m = 2..8, or fp16), two tiles (m = 9..16); whole 256-column chunks with whole-tile blocks (no bounds
    # predicates) and K / block sizes that need them; more than 16 rows (one launch per 16)
    for m, dtype in ((1, torch.bfloat16), (1, torch.float16), (2, torch.bfloat16), (7, torch.float16),
                     (9, torch.bfloat16), (16, torch.float16), (21, torch.bfloat16)):
        o, x, b, ref = _case(n, k, m, dtype, n + k + m + bs, bias=(m % 2 == 1), bs=bs)
        y = _run(o, x, b, cuda_device, "gemv")
        err = rel_max_err(y, ref, report=f"gemv {n}x{k} bs={bs} m={m} {dtype}")
        assert err < LINEAR_TOL, f"{n}x{k} bs={bs} m={m} {dtype}: {err}"
        # activations that do not allow 16-byte loads take the same kernels' two-byte path
        xs = torch.zeros(m, k + 3, dtype=dtype)
        xs[:, 3:] = x
        y2 = atlas_wrappers.quantized_linear_forward(xs.to(cuda_device)[:, 3:], _layout(o, cuda_device),
                                                     None if b is None else b.to(cuda_device), "gemv")
        assert rel_max_err(y2, ref, report=f"gemv unaligned {n}x{k} m={m}") < LINEAR_TOL


@pytest.mark.parametrize("thr", [1.0, 1.5])
def test_dense_outliers_reach_every_outlier_branch(thr, cuda_device):
    # tens of outliers per 16-row strip and 64-column tile: the streaming kernels' later outlier groups and entry
    # window refills and the tcgen05 kernel's "more than 16 outliers of one strip in one stage" branch run every time
    w = config_weights(512, 1024, 77)
    o = O.quantize(w, 128, thr)
    per_strip_stage = o.fp16_outliers.numel() / ((512 / 16) * (1024 / 128))
    assert per_strip_stage > 40, per_strip_stage
    gen = torch.Generator().manual_seed(5)
    wd = O.dequantize(o)
    for m, dtype, force in ((1, torch.float16, "stream"), (32, torch.bfloat16, "stream"), (5, torch.float16, "gemv"),
                            (12, torch.bfloat16, "gemv"),
                            (200, torch.float16, "gemm"), (40, torch.bfloat16, "gemm")):
        x = torch.randn(m, 1024, generator=gen).to(dtype)
        y = _run(o, x, None, cuda_device, force)
        assert rel_max_err(y, O.linear(x, wd), report=f"thr {thr} {force} m={m}") < LINEAR_TOL, (thr, force, m)


def test_stream_is_deterministic_and_workspace_is_reusable(cuda_device):
    # the same workspace serves launches of different shapes back to back; repeating a launch gives the same bits
    o1, x1, b1, ref1 = _case(4096, 4096, 16, torch.bfloat16, 21)
    o2, x2, b2, ref2 = _case(384, 11008, 3, torch.float16, 22)
    l1, l2 = _layout(o1, cuda_device), _layout(o2, cuda_device)
    ys = []
    for _ in range(3):
        ya = atlas_wrappers.quantized_linear_forward(x1.to(cuda_device), l1, b1.to(cuda_device), "stream")
        yb = atlas_wrappers.quantized_linear_forward(x2.to(cuda_device), l2, b2.to(cuda_device), "stream")
        ys.append((ya, yb))
    atlas_wrappers.check_status(cuda_device)
    assert rel_max_err(ys[0][0], ref1) < LINEAR_TOL and rel_max_err(ys[0][1], ref2) < LINEAR_TOL
    for ya, yb in ys[1:]:
        assert torch.equal(bits(ya), bits(ys[0][0])) and torch.equal(bits(yb), bits(ys[0][1]))
    ws = atlas_wrappers.stream_workspace(cuda_device)
    assert int(ws[:65536].count_nonzero()) == 0   # tickets are left as they were found


def test_stream_strided_and_unaligned_activations(cuda_device):
    o, x, b, ref = _case(512, 1024, 4, torch.float16, 5)
    wide = torch.zeros(4, 1024 + 40, dtype=torch.float16)
    wide[:, :1024] = x
    lay = _layout(o, cuda_device)
    y = atlas_wrappers.quantized_linear_forward(wide.to(cuda_device)[:, :1024], lay, b.to(cuda_device), "stream")
    assert rel_max_err(y, ref) < LINEAR_TOL
    # rows that start 2 bytes past a 16-byte boundary take the scalar activation loads
    base = torch.zeros(4 * 1024 + 1, dtype=torch.float16, device=cuda_device)
    base[1:] = x.reshape(-1).to(cuda_device)
    y2 = atlas_wrappers.quantized_linear_forward(base[1:].view(4, 1024), lay, b.to(cuda_device), "stream")
    assert torch.equal(bits(y2), bits(y))


def test_stream_through_the_c_abi_rejects_bad_arguments(cuda_device):
    L = _capi.load()
    o, x, b, _ = _case(128, 128, 1, torch.float16, 9)
    lay = _layout(o, cuda_device)
    xd = x.to(cuda_device)
    y = torch.empty(1, 128, dtype=torch.float16, device=cuda_device)
    small = torch.zeros(1024, dtype=torch.uint8, device=cuda_device)
    args = [xd.data_ptr(), _capi.DTYPE_F16, 1, 128, lay.tiles.data_ptr(), lay.scales_tiled.data_ptr(),
            lay.chunk_ptr.data_ptr(), _capi.ptr(lay.entries), _capi.ptr(lay.vals_sorted), 128, 128, 128, None,
            y.data_ptr(), 128]
    assert L.atlas_qlinear_stream(*args, small.data_ptr(), small.numel(), None, None) == _capi.ERR_CAPACITY
    assert L.atlas_qlinear_stream(*args, None, 0, None, None) == _capi.ERR_BAD_ARGUMENT
    bad = list(args)
    bad[10] = 100   # in_features not a multiple of 64
    ws = atlas_wrappers.stream_workspace(cuda_device)
    assert L.atlas_qlinear_stream(*bad, ws.data_ptr(), ws.numel(), None, None) in (_capi.ERR_UNSUPPORTED, _capi.ERR_BAD_ARGUMENT)


# ---------------------------------------------------------------- fused sibling projections
@pytest.mark.parametrize("m,dtype", [(1, torch.bfloat16), (5, torch.float16), (32, torch.bfloat16)])
def test_fused_group_equals_members(m, dtype, cuda_device):
    # q/k/v-like group with a member that is not a multiple of 128 rows and one without bias
    shapes = [(384, 512), (200, 512), (128, 512)]
    gen = torch.Generator().manual_seed(3)
    mods, refs = [], []
    x = torch.randn(1, m, 512, generator=gen).to(dtype)
    for i, (n, k) in enumerate(shapes):
        w = config_weights(n, k, 900 + i)
        b = (torch.randn(n, generator=gen) * 0.02).half() if i != 1 else None
        mods.append(ab.QuantizedLinear(ab.quantize_tensor(w.to(cuda_device)), None if b is None else b.to(cuda_device)))
        refs.append(O.linear(x.reshape(m, 512), O.dequantize(O.quantize(w)), b))
    xd = x.to(cuda_device)
    alone = [mod(xd) for mod in mods]
    group = ab.fuse_linears(mods)
    together = [mod(xd) for mod in mods]
    assert group.launches == 1                      # one launch served all three
    for y, ya, ref, (n, _) in zip(together, alone, refs, shapes):
        assert y.shape == (1, m, n) and y.dtype == dtype
        assert rel_max_err(y.reshape(m, n), ref, report="fused") < LINEAR_TOL
        # same numbers added in another order at most: a few output ulps between fused and stand-alone
        assert (y.float() - ya.float()).abs().max().item() <= 4 * 2.0 ** (-7 if dtype == torch.bfloat16 else -10) * \
            ya.float().abs().max().item()
    # another input object: a fresh launch; and a member alone on its own view of the joined layout
    xd2 = xd.clone()
    y0 = mods[0](xd2)
    assert group.launches == 2 and torch.equal(bits(y0), bits(together[0]))
    big = torch.randn(40, 512, generator=gen).to(dtype).to(cuda_device)   # prompt-sized input: the joined launch goes to the tcgen05 kernel
    yb = mods[1](big)
    refb = O.linear(big.cpu(), O.dequantize(O.quantize(config_weights(200, 512, 901))), None)
    assert group.launches == 3 and yb.shape == (40, 200) and rel_max_err(yb, refb) < LINEAR_TOL


def test_offloaded_canonical_streams_keep_the_layer_working(cuda_device):
    w = config_weights(256, 512, 41)
    layer = ab.QuantizedLinear(ab.quantize_tensor(w.to(cuda_device)), None)
    x = torch.randn(3, 512, generator=torch.Generator().manual_seed(2)).half().to(cuda_device)
    y = layer(x)
    before = torch.cuda.memory_allocated(cuda_device)
    layer.offload_canonical()
    assert layer.quantized_weights.fp8_data.device.type == "cpu"      # streams on the host, still complete
    assert layer.quantized_weights.memory_footprint(include_overhead=False) > 256 * 512
    assert torch.cuda.memory_allocated(cuda_device) < before
    assert torch.equal(bits(layer(x)), bits(y))                      # the forward keeps using the device layout


# ---------------------------------------------------------------- row-sharded weights (config 5 partitioning)
@pytest.mark.parametrize("n,k,world", [(8192, 8192, 8), (28672, 8192, 8), (1024, 8192, 8)])
def test_row_shards_concatenate_to_the_unsharded_product(n, k, world, cuda_device):
    # every rank's slice of a quantized weight (sharding.shard_rows), run through the kernel on this GPU and
    # concatenated, against the oracle product of the unsharded weight: m = 32 as in the 70B-shaped decode
    w = config_weights(n, k, n + k, 0.015)
    o = O.quantize(w)
    q = ab.QuantizedTensor(*o)
    gen = torch.Generator().manual_seed(8)
    x = torch.randn(32, k, generator=gen).to(torch.bfloat16)
    xd = x.to(cuda_device)
    parts = []
    for r in range(world):
        lo, hi = sharding.row_bounds(n, world, r, 16)
        shard = sharding.shard_rows(q, lo, hi)
        parts.append(atlas_wrappers.quantized_linear_forward(xd, atlas_wrappers.build_kernel_layout(shard.to(cuda_device)), None))
    atlas_wrappers.check_status(cuda_device)
    y = torch.cat(parts, dim=-1)
    assert y.shape == (32, n)
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = xd.float() @ O.dequantize(o).to(cuda_device).float().T     # fp32 on the GPU: the fp64 CPU loop would take minutes
    assert rel_max_err(y, ref, report=f"sharded {n}x{k}") < LINEAR_TOL
    spot = O.linear(x[:2], O.dequantize(o))                           # two rows against the fp64 oracle itself
    assert rel_max_err(y[:2], spot) < LINEAR_TOL


def test_gemm_llama_prefill_shape_11008(cuda_device):
    # 2048 tokens against 11008 x 4096 (the other half of the prefill config)
    w = config_weights(11008, 4096, 4243)
    o = O.quantize(w)
    x = torch.randn(2048, 4096, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    x[:, torch.randperm(4096, generator=torch.Generator().manual_seed(7))[:20]] *= 20
    y = _run(o, x, None, cuda_device, "gemm")
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = x.to(cuda_device).float() @ O.dequantize(o).to(cuda_device).float().T
    assert rel_max_err(y, ref, report="prefill 2048x11008x4096") < LINEAR_TOL
    spot = O.linear(x[:2], O.dequantize(o))
    assert rel_max_err(y[:2], spot) < LINEAR_TOL


# ---------------------------------------------------------------- batched quantize, on-disk format on the GPU path
def test_quantize_tensors_equals_one_by_one(cuda_device):
    ws = [config_weights(64, 1024, 1), config_weights(300, 256, 2), torch.empty(0, 8, dtype=torch.float16),
          config_weights(8, 128, 3)]
    batch = ab.quantize_tensors([w.to(cuda_device) for w in ws[:3]] + [ws[3]])   # the last one lives on the CPU
    for w, q in zip(ws, batch):
        o = O.quantize(w)
        for f in ("fp8_data", "fp16_outliers", "outlier_indices", "scale_factors"):
            assert torch.equal(bits(getattr(q, f).cpu()), bits(getattr(o, f))), f
        assert tuple(q.original_shape) == tuple(w.shape)
    assert batch[0].fp8_data.device.type == "cuda" and batch[3].fp8_data.device.type == "cpu"


def test_saved_layer_gives_identical_output(tmp_path, cuda_device):
    w = config_weights(256, 512, 77)
    b = (torch.randn(256, generator=torch.Generator().manual_seed(1)) * 0.02).half()
    q = ab.quantize_tensor(w.to(cuda_device))
    x = torch.randn(2, 512, generator=torch.Generator().manual_seed(2)).half().to(cuda_device)
    y = ab.QuantizedLinear(q, b.to(cuda_device))(x)
    path = str(tmp_path / "layer.atlq")
    ab.save_quantized(path, q, b)
    q2 = ab.load_quantized(path, cuda_device)
    for f in ("fp8_data", "fp16_outliers", "outlier_indices", "scale_factors"):
        assert torch.equal(bits(getattr(q2, f)), bits(getattr(q, f)))
    y2 = ab.QuantizedLinear(q2, b.to(cuda_device))(x)
    assert torch.equal(bits(y2), bits(y))


# ---------------------------------------------------------------- gather fused into the kernel (peer stores + arrival flags)
def _arena_u32(arena, offset, count):
    return arena.local_tensor(offset, (count,), torch.int32)


@pytest.mark.parametrize("kernel", ["stream", "gemm", "push"])
def test_peer_store_gather_with_emulated_ranks(kernel, cuda_device):
    # four "ranks" in this process on one GPU, run one after the other on one stream (never concurrently): every
    # rank's kernel stores its columns into all four gathered buffers and publishes its arrival; a second layer
    # then reads the gathered buffer as its input after waiting for the arrivals ("push": the default linear kernels
    # with the wait in front and the push kernel behind, instead of the one fused launch)
    from atlasinfer_b200 import peer
    world, m, k, n1, n2 = 4, 32, 512, 1024, 512
    w1, w2 = config_weights(n1, k, 61, 0.03), config_weights(n2, n1, 62, 0.03)
    o1, o2 = O.quantize(w1), O.quantize(w2)
    q1, q2 = ab.QuantizedTensor(*o1), ab.QuantizedTensor(*o2)
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    b1 = (torch.randn(n1, generator=gen) * 0.02).half()
    arenas = peer.PeerArena.on_one_device(1 << 20, cuda_device, world)
    try:
        layer1, layer2 = [], []
        for r, arena in enumerate(arenas):
            lo, hi = sharding.row_bounds(n1, world, r, 16)
            lay = atlas_wrappers.build_kernel_layout(sharding.shard_rows(q1, lo, hi).to(cuda_device))
            layer1.append(peer.GatheredLinear(arena, lay, m, torch.bfloat16, bias=b1[lo:hi].to(cuda_device), poll_limit=4000,
                                              kernel=kernel))
            lo, hi = sharding.row_bounds(n2, world, r, 16)
            lay = atlas_wrappers.build_kernel_layout(sharding.shard_rows(q2, lo, hi).to(cuda_device))
            layer2.append(peer.GatheredLinear(arena, lay, m, torch.bfloat16, poll_limit=4000, kernel=kernel))
        xd = x.to(cuda_device)
        for g in layer1:
            g(xd)                                      # local input: no wait
        for g in layer2:
            g(layer1[g.arena.rank].out, wait=True)      # input = this rank's gathered output of layer 1
        for g in layer2:
            g.wait_for_all()
        atlas_wrappers.check_status(cuda_device)       # no wait ran out
        ref1 = O.linear(x, O.dequantize(o1), b1)
        for r in range(world):
            y1 = layer1[r].out.clone()
            assert y1.shape == (m, n1)
            assert rel_max_err(y1, ref1, report=f"gathered layer 1 on rank {r}") < LINEAR_TOL
            assert torch.equal(bits(y1), bits(layer1[0].out))          # every rank holds the same gathered bits
            ref2 = O.linear(y1.cpu(), O.dequantize(o2))
            assert rel_max_err(layer2[r].out, ref2, report=f"gathered layer 2 on rank {r}") < LINEAR_TOL
        counts = _arena_u32(arenas[0], 0, world).tolist()
        assert counts == [2] * world                   # two gather launches per rank have arrived everywhere
    finally:
        for a in arenas:
            a.close()


def test_waits_on_peers_run_out_and_report_instead_of_hanging(cuda_device):
    # a flag that nothing sets: the stand-alone wait and the wait inside the linear kernel both give up after
    # their poll limit, set the status word and let the stream go on
    from atlasinfer_b200 import peer
    arenas = peer.PeerArena.on_one_device(1 << 18, cuda_device, 2)
    try:
        w = config_weights(128, 256, 71)
        lay = _layout(O.quantize(w), cuda_device)
        g0 = peer.GatheredLinear(arenas[0], lay, 4, torch.float16, poll_limit=2000)
        x = torch.randn(4, 256, generator=torch.Generator().manual_seed(1)).half().to(cuda_device)
        g0(x)                                          # rank 0 completes launch 1; "rank 1" never runs
        torch.cuda.synchronize()
        atlas_wrappers.check_status(cuda_device)
        g0.wait_for_all()                              # rank 1's arrival never comes
        with pytest.raises(_capi.AtlasError) as e:
            atlas_wrappers.check_status(cuda_device)
        assert e.value.status == _capi.ERR_TIMEOUT
        g0(x, wait=True)                               # same inside the kernel: it reports and still finishes
        with pytest.raises(_capi.AtlasError):
            atlas_wrappers.check_status(cuda_device)
        atlas_wrappers.stream_workspace(cuda_device).zero_()   # as the header asks after a reported timeout
    finally:
        for a in arenas:
            a.close()
