"""Generate the golden fixtures in this folder from the UNMODIFIED reference.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/AtlasInfer

It imports the reference's own ``quantize_tensor`` / ``dequantize_tensor``
(atlasinfer_core/quant/adaptive_quantizer.py) and ``QuantizedLinear``
(integration/atlas_wrappers.py), runs them on seeded inputs, and stores inputs
and outputs as ``<case>.npz`` (fp16 arrays as raw int16 patterns).  The
fixtures pin the CPU oracle (tests/test_oracle_golden.py) and, through the
same files, the CUDA path (tests/test_gpu_parity.py).  The reference checkout
itself is never needed at test time.
"""
import contextlib
import io
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def config_weights(rows, cols, seed, sigma=0.02):
    """fp16 N(0, sigma) with 0.1 % of entries replaced by +-U(0.1, 0.5)."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * sigma
    n = w.numel()
    k = round(1e-3 * n)
    pos = torch.randperm(n, generator=g)[:k]
    mag = torch.rand(k, generator=g) * 0.4 + 0.1
    sign = torch.where(torch.rand(k, generator=g) < 0.5, -1.0, 1.0)
    w.view(-1)[pos] = mag * sign
    return w.to(torch.float16)


def cases():
    g = torch.Generator().manual_seed(20240607)
    out = {}
    # the reference's own three test cases (tests/test_quantizer.py:11-56), seeded
    t = (torch.randn(128, 256, generator=g) * 5).to(torch.float16)
    t.view(-1)[::150] *= 10
    out["ref_standard_bs64_thr3p5"] = (t, 64, 3.5)
    out["ref_small_10_bs64"] = (torch.randn(10, generator=g).to(torch.float16), 64, 3.0)
    out["ref_empty_0x10"] = (torch.empty(0, 10, dtype=torch.float16), 128, 3.0)
    # the benchmark configs' distribution, small slices
    out["cfg_opt_32x2048"] = (config_weights(32, 2048, 1234), 128, 3.0)
    out["cfg_llama_8x4096"] = (config_weights(8, 4096, 1235), 128, 3.0)
    out["cfg_70b_4x8192_sigma015"] = (config_weights(4, 8192, 1236, 0.015), 128, 3.0)
    # wide dynamic range: the fp32 block sum is inexact, so its order matters
    for bs in (32, 64, 128, 256):
        e = torch.randint(-14, 10, (96 * bs,), generator=g).float()
        x = (torch.randn(96 * bs, generator=g) * torch.pow(2.0, e)).to(torch.float16)
        out[f"wide_range_bs{bs}"] = (x, bs, 3.0)
    e = torch.randint(-14, 10, (5000,), generator=g).float()
    x = (torch.randn(5000, generator=g) * torch.pow(2.0, e)).to(torch.float16)
    out["wide_range_padded_thr2p9"] = (x, 128, 2.9)
    # degenerate statistics
    x = torch.full((512,), 0.37)
    x[5] += 0.001
    out["near_constant"] = (x.to(torch.float16), 128, 3.0)
    out["all_zero_300"] = (torch.zeros(300, dtype=torch.float16), 128, 3.0)
    out["low_threshold_0p1"] = ((1.0 + torch.randn(1024, generator=g) * 1e-3).to(torch.float16), 128, 0.1)
    out["subnormal_inputs"] = ((torch.randn(2048, generator=g) * 1e-6).to(torch.float16), 128, 3.0)
    out["tiny_scale"] = ((torch.randn(2048, generator=g) * 1e-4).to(torch.float16), 128, 3.0)
    # padding zeros flagged as outliers (indices >= numel)
    x = torch.cat([torch.randn(128, generator=g), torch.full((120,), 5.0)]).to(torch.float16)
    out["padding_flagged"] = (x, 128, 3.0)
    out["single_element"] = (torch.full((1,), 3.0, dtype=torch.float16), 128, 3.0)
    # the most outliers a 128-block can hold at threshold 3: floor(127 / 9) = 14
    x = torch.zeros(128)
    x[:14] = torch.tensor([1.0, -1.0] * 7)
    out["max_outliers_14"] = (x.to(torch.float16), 128, 3.0)
    # 3-D shape and odd trailing size
    out["shape_3x5x77"] = ((torch.randn(3, 5, 77, generator=g) * 0.1).to(torch.float16), 64, 3.0)
    # block sizes that do not divide the CUDA quantizer's 8192-element tile, more than three tiles, ragged end;
    # wide dynamic range so that the order of the fp32 block sum matters for these sizes too
    for bs, n in ((96, 30001), (160, 26000), (384, 33333), (512, 20000)):
        e = torch.randint(-12, 6, (n,), generator=g).float()
        x = (torch.randn(n, generator=g) * torch.pow(2.0, e)).to(torch.float16)
        out[f"odd_block_bs{bs}"] = (x, bs, 3.0)
    return out


def i16(t):
    return t.contiguous().view(torch.int16).numpy()


def main(ref_root):
    sys.path.insert(0, ref_root)
    from atlasinfer_core.quant.adaptive_quantizer import (  # noqa: E402
        clear_dequantized_cache, dequantize_tensor, quantize_tensor)
    from integration.atlas_wrappers import QuantizedLinear  # noqa: E402

    torch.set_num_threads(1)
    for name, (w, bs, thr) in cases().items():
        if os.path.exists(os.path.join(HERE, name + ".npz")) and not os.environ.get("ATLAS_GOLDEN_OVERWRITE"):
            continue   # fixtures already in the tree stay as they are
        q = quantize_tensor(w, block_size=bs, z_threshold=thr)
        clear_dequantized_cache()
        d = dequantize_tensor(q, torch.device("cpu"))
        rec = dict(
            shape=np.array(list(w.shape), dtype=np.int64), block_size=np.int64(bs),
            z_threshold=np.float64(thr), input=i16(w.reshape(-1)),
            fp8_data=q.fp8_data.numpy(), fp16_outliers=i16(q.fp16_outliers),
            outlier_indices=q.outlier_indices.numpy(), scale_factors=i16(q.scale_factors),
            dequantized=i16(d.reshape(-1)))
        if name.startswith("cfg_"):
            # reference QuantizedLinear forward (atlas_wrappers.py:30-74) on fp16 activations
            g = torch.Generator().manual_seed(99)
            x = torch.randn(1, 4, w.shape[1], generator=g).to(torch.float16)
            bias = (torch.randn(w.shape[0], generator=g) * 0.02).to(torch.float16)
            layer = QuantizedLinear(q, bias)
            with contextlib.redirect_stdout(io.StringIO()):
                y = layer(x)
            rec.update(x=i16(x.reshape(-1)), x_shape=np.array(list(x.shape), dtype=np.int64),
                       bias=i16(bias), y=i16(y.reshape(-1)))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
        print(f"{name}: numel={w.numel()} codes={q.fp8_data.numel()} outliers={q.fp16_outliers.numel()}")
        clear_dequantized_cache()


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("ATLASINFER_REFERENCE"):
        sys.exit("usage: make_golden.py <path to an AtlasInfer checkout>  (or set ATLASINFER_REFERENCE)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["ATLASINFER_REFERENCE"])
