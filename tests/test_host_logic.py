"""Host-side mirror of the reference's Python surface (runs without a GPU)."""
import sys
import types

import pytest
import torch
import torch.nn as nn

import atlasinfer_b200 as ab
from atlasinfer_b200 import dropin, sharding
from atlasinfer_b200.integration import atlas_wrappers, model_modifier
from atlasinfer_b200.quant import adaptive_quantizer as aq
from oracle import atlas_oracle as O
from tests.util import assert_streams_equal, bits, config_weights


def test_quantized_tensor_surface():
    # adaptive_quantizer.py:8-42: field order, NamedTuple-ness, to(), memory_footprint()
    assert aq.QuantizedTensor._fields == ("fp8_data", "fp16_outliers", "outlier_indices", "scale_factors",
                                          "original_shape", "block_size")
    q = aq.QuantizedTensor(torch.zeros(100, dtype=torch.int8), torch.zeros(3, dtype=torch.float16),
                           torch.zeros(3, dtype=torch.long), torch.zeros(1, dtype=torch.float16),
                           torch.Size((103,)), 128)
    assert isinstance(q, tuple) and type(q).__name__ == "QuantizedTensor"
    assert q.memory_footprint(include_overhead=False) == 100 + 6 + 24 + 2
    assert q.memory_footprint() == 100 + 6 + 24 + 2 + 128
    assert q.to(torch.device("cpu")) is q
    assert type(q)(*list(q)) == q  # helpers.map_structure rebuilds it positionally


def test_quantize_tensor_signature_and_errors():
    import inspect
    sig = inspect.signature(aq.quantize_tensor)
    assert list(sig.parameters) == ["fp16_tensor", "block_size", "z_threshold"]
    assert sig.parameters["block_size"].default == 128 and sig.parameters["z_threshold"].default == 3.0
    assert list(inspect.signature(aq.dequantize_tensor).parameters) == ["quant_data", "target_device"]
    assert inspect.signature(aq.clear_dequantized_cache).parameters["quant_data_id"].default is None
    with pytest.raises(TypeError):
        aq.quantize_tensor([1.0, 2.0])


def test_empty_tensor_needs_no_gpu():
    # adaptive_quantizer.py:72-80 and tests/test_quantizer.py:51-56 of the reference
    q = aq.quantize_tensor(torch.empty((0, 10), dtype=torch.float16))
    assert q.fp8_data.numel() == 0 and q.fp8_data.dtype == torch.int8
    assert q.outlier_indices.dtype == torch.long and q.scale_factors.dtype == torch.float16
    assert q.original_shape == torch.Size((0, 10)) and q.block_size == 128


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_no_gpu_fails_loudly():
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        aq.quantize_tensor(torch.randn(256).half())
    q = O.quantize(torch.randn(4, 128).half())
    layer = ab.QuantizedLinear(aq.QuantizedTensor(*q), None)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        layer(torch.randn(1, 128).half())
    aq.clear_dequantized_cache()
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        aq.dequantize_tensor(aq.QuantizedTensor(*q), torch.device("cpu"))


def test_quantized_linear_surface():
    q = aq.QuantizedTensor(*O.quantize(torch.randn(8, 128).half()))
    bias = torch.zeros(8, dtype=torch.float16)
    layer = ab.QuantizedLinear(q, bias)
    assert type(layer).__name__ == "QuantizedLinear"
    assert layer.quantized_weights is q and layer.bias is bias and layer.original_shape == torch.Size((8, 128))
    assert len(layer.state_dict()) == 0  # plain attributes, as in the reference
    layer.quantized_weights = q.to(torch.device("cpu"))  # re-assignable (offload hook does setattr)
    layer.bias = None
    assert "bias=False" in layer.extra_repr()
    bad = ab.QuantizedLinear(torch.zeros(3), None)
    with pytest.raises(TypeError, match="not a valid QuantizedTensor"):
        bad(torch.zeros(1, 3, dtype=torch.float16))


def test_kernel_layout_supported():
    f = atlas_wrappers.kernel_layout_supported
    assert f((4096, 4096), 128) is None and f((10, 768), 64) is None
    assert "multiple of 64" in f((4, 100), 128)
    assert "block_size" in f((4, 192), 128)
    assert "2-D" in f((4,), 128)


class Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed_tokens = nn.Linear(4, 4)
        self.block = nn.Sequential(nn.Linear(4, 4), nn.ReLU(), nn.Linear(4, 2))
        self.lm_head = nn.Linear(2, 2)


def test_find_and_replace_modules():
    m = Tiny()
    found = model_modifier.find_modules(m, [nn.Linear], exclude_names=["lm_head", "embed_tokens", "embeddings"])
    assert [n for n, _ in found] == ["block.0", "block.2"]
    assert [n for n, _ in model_modifier.find_modules(m, [], target_names=["ReLU"])] == ["block.1"]
    new = nn.Identity()
    old = m.block[0]
    model_modifier._replace_module(m.block, "0", new)
    assert m.block[0] is new and len(old._parameters) == 0


def test_applier_unknown_model_type_and_unsupported_layers(capsys):
    m = Tiny()
    assert model_modifier.apply_atlas_quantization_to_model(m, "nope", {"block_size": 128}) is None
    assert "No layer patterns" in capsys.readouterr().out
    # in_features 4 cannot use the fused kernels: counted as failed, left as nn.Linear, no GPU touched
    model_modifier.apply_atlas_quantization_to_model(m, "opt", {"block_size": 128, "z_threshold": 3.0})
    out = capsys.readouterr().out
    assert "Replaced: 0, Failed/Skipped: 2" in out
    assert isinstance(m.block[0], nn.Linear)
    assert set(model_modifier.MODEL_LAYER_PATTERNS) == {"opt", "llama", "mistral", "gemma"}


def test_dropin_install_registers_reference_paths():
    saved = {k: sys.modules.get(k) for k in list(sys.modules)
             if k.split(".")[0] in ("atlasinfer_core", "integration")}
    try:
        dropin.install(replace_model_modifier=True)
        from atlasinfer_core.quant.adaptive_quantizer import QuantizedTensor, quantize_tensor  # noqa
        from integration.atlas_wrappers import QuantizedLinear  # noqa
        from integration.model_modifier import apply_atlas_quantization_to_model  # noqa
        assert QuantizedTensor is aq.QuantizedTensor and quantize_tensor is aq.quantize_tensor
        assert QuantizedLinear is atlas_wrappers.QuantizedLinear
        assert isinstance(sys.modules["atlasinfer_core"], types.ModuleType)
    finally:
        for k in [k for k in sys.modules if k.split(".")[0] in ("atlasinfer_core", "integration")]:
            del sys.modules[k]
        sys.modules.update({k: v for k, v in saved.items() if v is not None})


def test_shard_rows_equals_quantizing_the_shard():
    w = config_weights(64, 256, 7)
    whole = aq.QuantizedTensor(*O.quantize(w))
    for world in (2, 4):
        for rank in range(world):
            lo, hi = sharding.row_bounds(64, world, rank, 16)
            part = sharding.shard_rows(whole, lo, hi)
            assert_streams_equal(part, O.quantize(w[lo:hi]), what=f"world {world} rank {rank}: ")
            assert part.original_shape == torch.Size((hi - lo, 256))
    assert list(sharding.layers_for_rank(80, 8, 3)) == list(range(30, 40))
    assert sum(len(sharding.layers_for_rank(10, 4, r)) for r in range(4)) == 10
    with pytest.raises(ValueError):
        sharding.shard_rows(whole, 10, 100)
