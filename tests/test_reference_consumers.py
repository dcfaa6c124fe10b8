"""The reference's own consumers of the quantizer types, run unmodified against this package's classes.

Skipped unless ATLASINFER_REFERENCE points at a checkout of nishantkluhera/AtlasInfer (as
tests/golden/make_golden.py does).  ``dropin.install()`` makes the reference's import paths resolve to the
B200 implementations; then the reference's ``estimate_quantized_model_vram`` and ``map_structure``
(atlasinfer_core/utils/helpers.py:9-45, 54-82) and -- when ``accelerate`` is installed --
``QuantizedTensorOffloadHook._move_to_device`` (atlasinfer_core/utils/weight_offloader.py:61-88) are called on
``QuantizedTensor`` / ``QuantizedLinear`` objects of this package.  Runs without a GPU (streams from the oracle).
"""
import importlib
import os
import sys

import pytest
import torch
import torch.nn as nn

REF = os.environ.get("ATLASINFER_REFERENCE")
pytestmark = pytest.mark.skipif(not REF or not os.path.isdir(REF), reason="ATLASINFER_REFERENCE is not set")


@pytest.fixture(scope="module")
def ref_helpers():
    import atlasinfer_b200 as ab  # noqa: F401
    from atlasinfer_b200 import dropin
    saved = {k: v for k, v in sys.modules.items() if k.split(".")[0] in ("atlasinfer_core", "integration")}
    sys.path.insert(0, REF)
    try:
        dropin.install(replace_model_modifier=True)
        helpers = importlib.import_module("atlasinfer_core.utils.helpers")
        yield helpers
    finally:
        sys.path.remove(REF)
        for k in [k for k in sys.modules if k.split(".")[0] in ("atlasinfer_core", "integration")]:
            del sys.modules[k]
        sys.modules.update(saved)


def _model():
    import atlasinfer_b200 as ab
    from oracle import atlas_oracle as O
    from tests.util import config_weights

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.q = ab.QuantizedLinear(ab.QuantizedTensor(*O.quantize(config_weights(64, 256, 1))), torch.zeros(64).half())
            self.k = ab.QuantizedLinear(ab.QuantizedTensor(*O.quantize(config_weights(32, 256, 2))), None)
            self.norm = nn.LayerNorm(64).half()

    return Net()


def test_estimate_quantized_model_vram_counts_our_layers(ref_helpers):
    net = _model()
    want = 0
    for lin in (net.q, net.k):
        want += lin.quantized_weights.memory_footprint(include_overhead=False)
        if lin.bias is not None:
            want += lin.bias.numel() * lin.bias.element_size()
    want += sum(p.numel() * p.element_size() for p in net.norm.parameters())
    assert ref_helpers.estimate_quantized_model_vram(net) == want      # the helper reports bytes


def test_map_structure_rebuilds_our_named_tuple(ref_helpers):
    import atlasinfer_b200 as ab
    net = _model()
    q = net.q.quantized_weights
    moved = ref_helpers.map_structure(lambda t: t.clone() if isinstance(t, torch.Tensor) else t, {"w": [q, 3]})
    q2 = moved["w"][0]
    assert isinstance(q2, ab.QuantizedTensor) and q2 is not q and moved["w"][1] == 3
    assert torch.equal(q2.fp8_data, q.fp8_data) and q2.original_shape == q.original_shape and q2.block_size == q.block_size


def test_offload_hook_moves_our_types(ref_helpers):
    pytest.importorskip("accelerate")
    import atlasinfer_b200 as ab
    off = importlib.import_module("atlasinfer_core.utils.weight_offloader")
    hook = off.QuantizedTensorOffloadHook(execution_device=torch.device("cpu"))
    net = _model()
    moved = hook._move_to_device(net.q.quantized_weights, torch.device("cpu"))
    assert isinstance(moved, ab.QuantizedTensor)
    hook._move_to_device(net.q, torch.device("cpu"))
    assert net.q.quantized_weights.fp8_data.device.type == "cpu"
