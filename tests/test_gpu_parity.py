"""Parity of the CUDA path against the CPU oracle and the reference's golden fixtures.

Every call goes through the C ABI (``atlasinfer_b200._capi`` -> libatlas_b200.so).
Integer / byte / index outputs must be bit-exact; linear outputs are held to
max|err| <= 1e-2 * rms(ref), ref = x.float() @ dequantized.float().T (+ bias).
"""
import pytest
import torch

import atlasinfer_b200 as ab
from atlasinfer_b200 import _capi
from atlasinfer_b200.integration import atlas_wrappers
from atlasinfer_b200.quant import adaptive_quantizer as aq
from oracle import atlas_oracle as O
from tests.util import assert_streams_equal, bits, config_weights, golden_names, load_golden, rel_max_err

pytestmark = pytest.mark.gpu
LINEAR_TOL = 1e-2  # max|err| / rms(ref), the tolerance of the path's specification

GPU_BLOCK_SIZES = {32, 64, 128, 256}


def _fast_path(name):
    g = load_golden(name)
    return g["block_size"] % 32 == 0 and 32 <= g["block_size"] <= 512


# ---------------------------------------------------------------- quantizer
@pytest.mark.parametrize("name", [n for n in golden_names() if _fast_path(n)])
def test_quantize_bit_exact_vs_reference_fixture(name, cuda_device):
    g = load_golden(name)
    q = ab.quantize_tensor(g["input"].to(cuda_device), g["block_size"], g["z_threshold"])
    assert q.fp8_data.device.type == "cuda" or g["input"].numel() == 0
    assert_streams_equal(q, g, what=name + ": ")
    assert tuple(q.original_shape) == g["shape"] and q.block_size == g["block_size"]


@pytest.mark.parametrize("name", golden_names())
def test_dequantize_bit_exact_vs_reference_fixture(name, cuda_device):
    g = load_golden(name)
    q = ab.QuantizedTensor(g["fp8_data"], g["fp16_outliers"], g["outlier_indices"], g["scale_factors"],
                           torch.Size(g["shape"]), g["block_size"])
    ab.clear_dequantized_cache()
    d = ab.dequantize_tensor(q, cuda_device)
    assert d.device.type == "cuda" and d.dtype == torch.float16 and tuple(d.shape) == g["shape"]
    assert torch.equal(bits(d.cpu()), bits(g["dequantized"]))
    assert ab.dequantize_tensor(q, cuda_device) is d  # second call is served from the cache
    ab.clear_dequantized_cache()


def test_cpu_input_returns_cpu_streams(cuda_device):
    # model_modifier.py:128-131 of the reference always hands CPU weights; results stay on the CPU
    g = load_golden("cfg_opt_32x2048")
    q = ab.quantize_tensor(g["input"], g["block_size"], g["z_threshold"])
    assert all(t.device.type == "cpu" for t in q[:4])
    assert_streams_equal(q, g)
    ab.clear_dequantized_cache()
    d = ab.dequantize_tensor(q, torch.device("cpu"))
    assert d.device.type == "cpu" and torch.equal(bits(d), bits(g["dequantized"]))
    ab.clear_dequantized_cache()


def test_non_fp16_input_is_converted_with_warning(cuda_device, capsys):
    w = torch.randn(4, 256, generator=torch.Generator().manual_seed(1)) * 0.02
    q = ab.quantize_tensor(w.to(cuda_device))
    assert "converting to FP16" in capsys.readouterr().out
    assert_streams_equal(q, O.quantize(w.half()))


def test_unsupported_block_size_is_loud(cuda_device):
    with pytest.raises(NotImplementedError, match="block_size"):
        ab.quantize_tensor(torch.randn(1000, device=cuda_device).half(), block_size=100)


@pytest.mark.parametrize("shape,seed", [((2048, 2048), 1234), ((8192, 2048), 1238), ((2048, 8192), 1239),
                                        ((11008, 4096), 1240), ((4096, 11008), 1241)])
def test_quantize_bit_exact_vs_oracle_full_shapes(shape, seed, cuda_device):
    # the benchmark configs' own tensor shapes, every stream compared in full
    w = config_weights(*shape, seed)
    q = ab.quantize_tensor(w.to(cuda_device))
    o = O.quantize(w)
    assert_streams_equal(q, o, what=f"{shape}: ")
    n_out = q.fp16_outliers.numel()
    assert q.fp8_data.numel() + n_out == w.numel()
    assert 0.002 < n_out / w.numel() < 0.004
    idx = q.outlier_indices
    assert bool((idx[1:] > idx[:-1]).all())  # strictly ascending
    # round trip: outliers come back exactly, the rest within half a quantization step (+ fp16 rounding)
    ab.clear_dequantized_cache()
    d = ab.dequantize_tensor(q, cuda_device)
    assert torch.equal(bits(d.cpu()), bits(O.dequantize(o)))
    wd = w.to(cuda_device)
    assert torch.equal(d.view(-1)[idx], wd.view(-1)[idx])
    step = q.scale_factors.float().repeat_interleave(128).view(shape)
    # the quotient x/scale is rounded to fp16 (ulp 1/16 in [64, 128)) before it is rounded to an integer,
    # and the product code*scale is rounded to fp16 again: 0.5 + 1/32 steps plus one fp16 ulp of slack
    bound = step * (0.5 + 1.0 / 32 + 1e-3) + wd.float().abs() * 2.0 ** -10 + 1e-7
    assert bool(((d.float() - wd.float()).abs() <= bound).all())
    ab.clear_dequantized_cache()


@pytest.mark.parametrize("bs,thr,n", [(32, 3.0, 40000), (64, 2.5, 70001), (256, 3.0, 300000), (512, 3.5, 100000),
                                      (128, 0.1, 50000), (128, 1.0, 8192 * 5)])
def test_quantize_other_block_sizes_and_dense_outliers(bs, thr, n, cuda_device):
    # ragged sizes (padding), many tiles, and thresholds low enough to overflow the first outlier buffer
    gen = torch.Generator().manual_seed(bs + n)
    e = torch.randint(-10, 4, (n,), generator=gen).float()
    w = (torch.randn(n, generator=gen) * torch.pow(2.0, e)).half()
    q = ab.quantize_tensor(w.to(cuda_device), bs, thr)
    assert_streams_equal(q, O.quantize(w, bs, thr), what=f"bs {bs} thr {thr}: ")


def test_quantize_unaligned_view(cuda_device):
    w = config_weights(64, 1024, 77)
    base = torch.zeros(w.numel() + 3, dtype=torch.float16, device=cuda_device)
    base[3:] = w.view(-1).to(cuda_device)
    q = ab.quantize_tensor(base[3:].view(64, 1024))  # data pointer 6 bytes past a 16-byte boundary
    assert_streams_equal(q, O.quantize(w))


# ---------------------------------------------------------------- quantized linear
def _linear_case(n, k, m, dtype, seed, bias=True, bs=128, sigma=0.02):
    w = config_weights(n, k, seed, sigma)
    o = O.quantize(w, bs, 3.0)
    gen = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(m, k, generator=gen).to(dtype)
    b = (torch.randn(n, generator=gen) * 0.02).half() if bias else None
    ref = O.linear(x, O.dequantize(o), b)
    return o, x, b, ref


def _run_linear(o, x, b, dev, force=None):
    q = ab.QuantizedTensor(*o).to(dev)
    lay = atlas_wrappers.build_kernel_layout(q)
    y = atlas_wrappers.quantized_linear_forward(x.to(dev), lay, None if b is None else b.to(dev), force)
    atlas_wrappers.check_status(dev)
    return y


@pytest.mark.parametrize("m", [1, 3, 4, 8, 9, 16, 17, 32, 33, 70])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemv_matches_oracle(m, dtype, cuda_device):
    o, x, b, ref = _linear_case(2048, 2048, m, dtype, 300 + m)
    y = _run_linear(o, x, b, cuda_device, "gemv")
    assert y.dtype == dtype and y.shape == (m, 2048)
    assert rel_max_err(y, ref) < LINEAR_TOL


@pytest.mark.parametrize("n,k,bs", [(4096, 4096, 128), (11008, 4096, 128), (4096, 11008, 128), (1024, 8192, 128),
                                    (200, 256, 128), (16, 64, 64), (130, 192, 64), (3584, 8192, 128),
                                    (128, 28672, 128), (500, 1024, 32), (77, 512, 256)])
def test_gemv_shapes(n, k, bs, cuda_device):
    for m, dtype in ((1, torch.bfloat16), (16, torch.bfloat16), (32, torch.float16)):
        o, x, b, ref = _linear_case(n, k, m, dtype, n + k + m, bias=(m != 16), bs=bs)
        y = _run_linear(o, x, b, cuda_device, "gemv")
        err = rel_max_err(y, ref)
        assert err < LINEAR_TOL, f"{n}x{k} m={m} {dtype}: {err}"


def test_gemv_strided_activations_and_outlier_free_weight(cuda_device):
    o, x, b, ref = _linear_case(512, 1024, 4, torch.float16, 5)
    wide = torch.zeros(4, 1024 + 40, dtype=torch.float16)
    wide[:, :1024] = x
    q = ab.QuantizedTensor(*o).to(cuda_device)
    lay = atlas_wrappers.build_kernel_layout(q)
    y = atlas_wrappers.quantized_linear_forward(wide.to(cuda_device)[:, :1024], lay, b.to(cuda_device), "gemv")
    assert rel_max_err(y, ref) < LINEAR_TOL
    w = (torch.randn(256, 512, generator=torch.Generator().manual_seed(2)) * 0.02).clamp(-0.04, 0.04).half()
    o2 = O.quantize(w)
    assert o2.fp16_outliers.numel() == 0
    x2 = torch.randn(2, 512).half()
    y2 = _run_linear(o2, x2, None, cuda_device, "gemv")
    assert rel_max_err(y2, O.linear(x2, O.dequantize(o2))) < LINEAR_TOL


def test_gemv_is_deterministic(cuda_device):
    o, x, b, _ = _linear_case(4096, 4096, 16, torch.bfloat16, 21)
    y1 = _run_linear(o, x, b, cuda_device, "gemv")
    y2 = _run_linear(o, x, b, cuda_device, "gemv")
    assert torch.equal(bits(y1), bits(y2))


@pytest.mark.parametrize("m", [128, 200, 2048])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemm_matches_oracle(m, dtype, cuda_device):
    o, x, b, ref = _linear_case(1024, 2048, m, dtype, 900 + m)
    if dtype == torch.bfloat16:  # activation outliers: 0.5 % of the channels scaled x20
        ch = torch.randperm(2048, generator=torch.Generator().manual_seed(4))[:10]
        x[:, ch] *= 20
        ref = O.linear(x, O.dequantize(o), b)
    y = _run_linear(o, x, b, cuda_device, "gemm")
    assert rel_max_err(y, ref) < LINEAR_TOL


@pytest.mark.parametrize("m", [1, 9, 16, 32, 33, 64, 100])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1024, 8192), (200, 1024), (11008, 4096)])
def test_gemm_small_batches_and_k_slices(m, n, k, cuda_device):
    # decode-sized batches through the tcgen05 kernel: narrow token tiles, K sliced over CTAs
    dtype = torch.bfloat16 if m % 2 else torch.float16
    o, x, b, ref = _linear_case(n, k, m, dtype, 40 + m + n, bias=(m != 16))
    y = _run_linear(o, x, b, cuda_device, "gemm")
    assert rel_max_err(y, ref) < LINEAR_TOL
    y2 = _run_linear(o, x, b, cuda_device, "gemm")
    assert torch.equal(bits(y), bits(y2))  # slices are added in a fixed order


@pytest.mark.parametrize("n,k,bs,m", [(256, 192, 64, 40), (128, 64, 64, 300), (300, 320, 32, 17), (512, 1088, 64, 130),
                                      (130, 448, 64, 257)])
def test_gemm_odd_k_tile_counts_and_block_sizes(n, k, bs, m, cuda_device):
    # an odd number of 64-column k-tiles leaves the last pipeline stage half full; block sizes below 64 take the
    # scales from global memory instead of the staged copy
    dtype = torch.float16 if m % 2 else torch.bfloat16
    o, x, b, ref = _linear_case(n, k, m, dtype, 900 + n + k, bias=True, bs=bs)
    y = _run_linear(o, x, b, cuda_device, "gemm")
    assert rel_max_err(y, ref) < LINEAR_TOL, f"{n}x{k} bs={bs} m={m}"


def test_gemm_llama_prefill_shape(cuda_device):
    # 2048 tokens against 4096 x 4096; the reference product is evaluated on the GPU in fp32
    # from the oracle's dequantized weight (the CPU oracle's fp64 loop would take minutes here)
    w = config_weights(4096, 4096, 4242)
    o = O.quantize(w)
    x = torch.randn(2048, 4096, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    x[:, torch.randperm(4096, generator=torch.Generator().manual_seed(7))[:20]] *= 20
    y = _run_linear(o, x, None, cuda_device, "gemm")
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = x.to(cuda_device).float() @ O.dequantize(o).to(cuda_device).float().T
    assert rel_max_err(y, ref) < LINEAR_TOL
    spot = O.linear(x[:2], O.dequantize(o))  # and two rows against the fp64 oracle itself
    assert rel_max_err(y[:2], spot) < LINEAR_TOL


# ---------------------------------------------------------------- module level
@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith("cfg_")])
def test_quantized_linear_vs_reference_forward_fixture(name, cuda_device):
    # the stored y is the reference QuantizedLinear.forward (fp16 F.linear on CPU)
    g = load_golden(name)
    q = ab.quantize_tensor(g["input"])          # CPU in, CPU streams out, as model_modifier does
    layer = ab.QuantizedLinear(q, g["bias"].clone())
    y = layer(g["x"].to(cuda_device))
    assert layer.quantized_weights.fp8_data.device.type == "cuda"   # moved lazily and re-assigned
    assert layer.bias.device.type == "cuda"
    assert y.shape == g["y"].shape and y.dtype == torch.float16
    assert rel_max_err(y, g["y"]) < LINEAR_TOL
    y_cpu = layer(g["x"])                        # CPU activations are staged through the GPU
    assert y_cpu.device.type == "cpu" and torch.equal(bits(y_cpu), bits(y.cpu()))


def test_opt_layer_shapes_config(cuda_device):
    # one OPT-1.3B decoder layer's linears, activations [1, 128, K] fp16
    for i, (n, k) in enumerate([(2048, 2048), (8192, 2048), (2048, 8192)]):
        w = config_weights(n, k, 1234 + i)
        gen = torch.Generator().manual_seed(50 + i)
        bias = (torch.randn(n, generator=gen) * 0.02).half()
        x = torch.randn(1, 128, k, generator=gen).half()
        layer = ab.QuantizedLinear(ab.quantize_tensor(w), bias)
        y = layer(x.to(cuda_device))
        ref = O.linear(x, O.dequantize(O.quantize(w)), bias)
        assert y.shape == (1, 128, n) and rel_max_err(y, ref) < LINEAR_TOL


def test_apply_to_tiny_opt_model_and_generate(cuda_device):
    from transformers import OPTConfig, OPTForCausalLM
    torch.manual_seed(0)
    cfg = OPTConfig(vocab_size=512, hidden_size=256, ffn_dim=512, num_hidden_layers=2, num_attention_heads=4,
                    max_position_embeddings=128, word_embed_proj_dim=256)
    model = OPTForCausalLM(cfg).half().eval()
    import copy
    ref_model = copy.deepcopy(model)
    ab.apply_atlas_quantization_to_model(model, "opt", {"block_size": 128, "z_threshold": 3.0}, verbose=False)
    qlayers = [m for m in model.modules() if type(m).__name__ == "QuantizedLinear"]
    assert len(qlayers) == 12 and all(l.quantized_weights.fp8_data.device.type == "cpu" for l in qlayers)
    # reference semantics of the same surgery: every linear weight replaced by its dequantized image
    for (name, lin) in [(n, m) for n, m in ref_model.named_modules() if isinstance(m, torch.nn.Linear)]:
        if any(ex in name for ex in ("lm_head", "embed_tokens")):
            continue
        lin.weight.data = O.dequantize(O.quantize(lin.weight.data)).to(lin.weight.dtype)
    model.to(cuda_device)
    ref_model.to(cuda_device)
    ids = torch.randint(0, 512, (1, 16), generator=torch.Generator().manual_seed(9)).to(cuda_device)
    with torch.no_grad():
        out = model.generate(ids, max_new_tokens=12, do_sample=False)
        logits = model(ids).logits.float()
        ref_logits = ref_model(ids).logits.float()
    assert out.shape == (1, 28)
    assert rel_max_err(logits, ref_logits) < 2e-2
