"""On-disk format of QuantizedTensor records (runs without a GPU)."""
import numpy as np
import torch
import torch.nn as nn

import atlasinfer_b200 as ab
from atlasinfer_b200.quant import serialization
from oracle import atlas_oracle as O
from tests.util import assert_streams_equal, bits, config_weights


def _q(rows, cols, seed, bs=128):
    return ab.QuantizedTensor(*O.quantize(config_weights(rows, cols, seed), bs, 3.0))


def test_round_trip_is_bit_exact(tmp_path):
    q = _q(48, 512, 5)
    bias = torch.randn(48).half()
    path = str(tmp_path / "w.atlq")
    ab.save_quantized(path, q, bias)
    back = ab.load_quantized(path)
    assert_streams_equal(back, q)
    assert back.original_shape == q.original_shape and back.block_size == q.block_size
    assert isinstance(back, ab.QuantizedTensor) and back.outlier_indices.dtype == torch.int64
    state = ab.load_quantized_state(path)
    assert torch.equal(bits(state["tensor"][1]), bits(bias))


def test_arrays_are_memmap_readable_at_their_offsets(tmp_path):
    q = _q(16, 256, 6, bs=64)
    path = str(tmp_path / "w.atlq")
    ab.save_quantized_state(path, {"a": q, "b": (_q(8, 128, 7), None)})
    header = serialization.read_header(path)
    assert set(header["records"]) == {"a", "b"}
    meta = header["records"]["a"]["arrays"]
    for field in ("fp8_data", "outlier_indices"):
        m = meta[field]
        assert m["offset"] % 64 == 0
        raw = np.memmap(path, dtype=np.dtype(m["dtype"]), mode="r", offset=m["offset"], shape=(m["count"],))
        assert np.array_equal(np.asarray(raw), getattr(q, field).numpy())
    m = meta["scale_factors"]
    raw = np.memmap(path, dtype=np.int16, mode="r", offset=m["offset"], shape=(m["count"],))
    assert np.array_equal(np.asarray(raw), q.scale_factors.view(torch.int16).numpy())


def test_empty_tensor_and_outlier_free_records(tmp_path):
    e = ab.quantize_tensor(torch.empty((0, 10), dtype=torch.float16))
    w = (torch.randn(4, 128, generator=torch.Generator().manual_seed(1)) * 0.02).clamp(-0.03, 0.03).half()
    q = ab.QuantizedTensor(*O.quantize(w))
    assert q.fp16_outliers.numel() == 0
    path = str(tmp_path / "w.atlq")
    ab.save_quantized_state(path, {"empty": e, "clean": q})
    st = ab.load_quantized_state(path)
    assert st["empty"][0].original_shape == torch.Size((0, 10)) and st["empty"][0].fp8_data.numel() == 0
    assert_streams_equal(st["clean"][0], q)


def test_model_level_save_and_load(tmp_path):
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(128, 32)
            self.b = nn.Sequential(nn.Linear(128, 16, bias=False))

    net = Net().half()
    src = {"a": (_q(32, 128, 1), torch.randn(32).half()), "b.0": (_q(16, 128, 2), None)}
    net.a = ab.QuantizedLinear(*src["a"])
    net.b[0] = ab.QuantizedLinear(*src["b.0"])
    path = str(tmp_path / "model.atlq")
    assert ab.save_quantized_model(net, path) == 2
    fresh = Net().half()
    assert ab.load_quantized_model(fresh, path) == 2
    for name, (q, bias) in src.items():
        mod = fresh.get_submodule(name)
        assert type(mod).__name__ == "QuantizedLinear"
        assert_streams_equal(mod.quantized_weights, q)
        assert (mod.bias is None) == (bias is None)
        if bias is not None:
            assert torch.equal(bits(mod.bias), bits(bias))
    assert not any(isinstance(m, nn.Linear) for m in fresh.modules())
