"""The CPU oracle must reproduce every fixture made by the unmodified reference."""
import pytest
import torch

from oracle import atlas_oracle as O
from tests.util import assert_streams_equal, bits, golden_names, load_golden, rel_max_err

NAMES = golden_names()


def test_fixtures_present():
    assert len(NAMES) >= 20


@pytest.mark.parametrize("name", NAMES)
def test_quantize_matches_reference(name):
    g = load_golden(name)
    q = O.quantize(g["input"], g["block_size"], g["z_threshold"])
    assert_streams_equal(q, g, what=name + ": ")
    assert tuple(q.original_shape) == g["shape"]


@pytest.mark.parametrize("name", NAMES)
def test_dequantize_matches_reference(name):
    g = load_golden(name)
    q = O.OracleQuantized(g["fp8_data"], g["fp16_outliers"], g["outlier_indices"], g["scale_factors"],
                          torch.Size(g["shape"]), g["block_size"])
    d = O.dequantize(q)
    assert d.shape == g["dequantized"].shape
    assert torch.equal(bits(d), bits(g["dequantized"]))


@pytest.mark.parametrize("name", [n for n in NAMES if n.startswith("cfg_")])
def test_linear_close_to_reference_forward(name):
    # the reference's own fp16 F.linear deviates ~2e-3 * rms from the exact product
    g = load_golden(name)
    y = O.linear(g["x"], g["dequantized"], g["bias"])
    assert rel_max_err(g["y"], y) < 1e-2


def test_row_sum_order_matches_torch():
    # the fp32 block sum must follow torch's vectorised order (it feeds torch.mean)
    gen = torch.Generator().manual_seed(5)
    for n in (32, 64, 128, 256, 100, 8, 24):
        for _ in range(50):
            e = torch.randint(-12, 12, (n,), generator=gen).float()
            x = (torch.randn(n, generator=gen) * torch.pow(2.0, e)).half().float()
            assert O.row_sum_f32(x) == torch.sum(x).item()


def test_mse_bound_of_reference_tests():
    # tests/test_quantizer.py:40,49 of the reference: round-trip MSE < 1e-3
    for name in ("ref_standard_bs64_thr3p5", "ref_small_10_bs64"):
        g = load_golden(name)
        d = O.dequantize(O.quantize(g["input"], g["block_size"], g["z_threshold"]))
        assert torch.mean((d.float() - g["input"].float()) ** 2).item() < 1e-3
