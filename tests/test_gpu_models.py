"""Whole models through the applier: the OPT-1.3B-architecture config at full size (quantize end to end, greedy
decode 128 + 128) and a small Llama (fused q/k/v and gate/up), against the same HF model whose linears hold the
oracle-dequantized weights -- the reference's semantics (integration/model_modifier.py:95-143 followed by
QuantizedLinear.forward = dequantize + F.linear, integration/atlas_wrappers.py:56,67).
"""
import copy
import time

import pytest
import torch

import atlasinfer_b200 as ab
from oracle import atlas_oracle as O
from tests.util import assert_streams_equal, rel_max_err

pytestmark = pytest.mark.gpu
EXCLUDED = ("lm_head", "embed_tokens", "embeddings")


def _init_like_config(model, seed, sigma=0.02, outlier_rate=1e-3):
    """Random-init on the model's device: weights N(0, sigma), norms 1 / 0, biases small; every linear that will be
    quantized gets 0.1 % of its entries replaced by +-U(0.1, 0.5) (seeded), as the benchmark configs prescribe."""
    dev = next(model.parameters()).device
    gen = torch.Generator(device=dev).manual_seed(seed)
    for name, p in model.named_parameters():
        if p.dim() >= 2:
            p.data.copy_((torch.randn(p.shape, generator=gen, device=dev) * sigma).to(p.dtype))
        elif "norm" in name and name.endswith("weight"):
            p.data.fill_(1.0)
        elif "norm" in name:
            p.data.zero_()
        else:
            p.data.copy_((torch.randn(p.shape, generator=gen, device=dev) * 0.01).to(p.dtype))
    for name, mod in model.named_modules():
        if isinstance(mod, torch.nn.Linear) and not any(ex in name for ex in EXCLUDED):
            w = mod.weight.data
            cnt = round(outlier_rate * w.numel())
            pos = torch.randint(0, w.numel(), (cnt,), generator=gen, device=dev)
            mag = torch.rand(cnt, generator=gen, device=dev) * 0.4 + 0.1
            sgn = torch.where(torch.rand(cnt, generator=gen, device=dev) < 0.5, -1.0, 1.0)
            w.view(-1)[pos] = (mag * sgn).to(w.dtype)


def _reference_semantics(model):
    """Replace every quantizable linear's weight by the oracle's dequantize(quantize(w)); returns the oracle streams."""
    streams = {}
    for name, mod in model.named_modules():
        if isinstance(mod, torch.nn.Linear) and not any(ex in name for ex in EXCLUDED):
            o = O.quantize(mod.weight.data.cpu())
            streams[name] = o
            mod.weight.data.copy_(O.dequantize(o).to(mod.weight.device))
    return streams


def _greedy_check(model, ref_model, ids, new_tokens, dev):
    """Greedy decode with both models; our tokens must be (numerically tied) argmaxes of the reference model."""
    with torch.no_grad():
        t0 = time.perf_counter()
        out = model.generate(ids, max_new_tokens=new_tokens, min_new_tokens=new_tokens, do_sample=False)
        torch.cuda.synchronize()
        secs = time.perf_counter() - t0
        ref_out = ref_model.generate(ids, max_new_tokens=new_tokens, min_new_tokens=new_tokens, do_sample=False)
        # teacher-forced: the reference model's logits along OUR sequence
        ref_logits = ref_model(out[:, :-1]).logits.float()[0]
        our_logits = model(out[:, :-1]).logits.float()[0]
    p = ids.shape[1]
    assert out.shape == (1, p + new_tokens)
    agree = int((out[0, p:] == ref_out[0, p:]).sum())
    steps = ref_logits[p - 1:]                       # positions whose argmax produced our new tokens
    chosen = steps.gather(1, out[0, p:].unsqueeze(1)).squeeze(1)
    gap = steps.max(dim=1).values - chosen           # 0 where our token is the reference model's argmax
    spread = steps.std(dim=1)
    print(f"[greedy] {new_tokens} tokens in {secs:.2f} s ({new_tokens / secs:.1f} tok/s eager); identical to the "
          f"reference-semantics model's greedy tokens: {agree}/{new_tokens}; worst argmax gap {gap.max().item():.3e} "
          f"(logit std {spread.mean().item():.3e})")
    # every token we chose is the reference model's argmax up to the fp16 noise both models carry through their
    # layers (near-ties); the two models differ only in the order of fp32 additions inside the linears
    logit_err = rel_max_err(our_logits[-1], ref_logits[-1], discount_output_rounding=False)
    print(f"[greedy] last-step logits: max|err|/rms = {logit_err:.3e}")
    assert bool((gap <= 5e-2 * spread).all()), (gap / spread).max().item()
    assert logit_err < 5e-2
    return agree


def test_opt_1p3b_architecture_quantize_and_greedy_decode(cuda_device):
    from transformers import OPTConfig, OPTForCausalLM
    cfg = OPTConfig(vocab_size=50272, hidden_size=2048, ffn_dim=8192, num_hidden_layers=24, num_attention_heads=32,
                    max_position_embeddings=2048, word_embed_proj_dim=2048)
    with torch.device(cuda_device):
        model = OPTForCausalLM(cfg).half().eval()
    _init_like_config(model, 1234)
    ref_model = copy.deepcopy(model)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ab.apply_atlas_quantization_to_model(model, "opt", {"block_size": 128, "z_threshold": 3.0},
                                         keep_on_device=True, fuse=True, verbose=False)
    torch.cuda.synchronize()
    t_quant = time.perf_counter() - t0
    qlayers = {n: m for n, m in model.named_modules() if type(m).__name__ == "QuantizedLinear"}
    n_weights = sum(m.original_shape[0] * m.original_shape[1] for m in qlayers.values())
    assert len(qlayers) == 144 and n_weights == 24 * (4 * 2048 * 2048 + 2 * 8192 * 2048)
    print(f"[opt-1.3b] quantized 144 linears / {n_weights / 1e9:.2f} G weights on the GPU in {t_quant:.2f} s")
    # all four streams of every layer, bit for bit, against the oracle on the same weights
    streams = _reference_semantics(ref_model)
    assert set(streams) == set(qlayers)
    for name, o in streams.items():
        assert_streams_equal(qlayers[name].quantized_weights, o, what=name + ": ")
    groups = {id(m._group) for m in qlayers.values() if m._group is not None}
    assert len(groups) == 24                                    # q/k/v of every layer share a launch
    ids = torch.randint(0, 50272, (1, 128), generator=torch.Generator().manual_seed(9)).to(cuda_device)
    _greedy_check(model, ref_model, ids, 128, cuda_device)


def test_cpu_hop_default_equals_on_device_quantization(cuda_device):
    # the reference-compatible default (model and weights through the CPU, model_modifier.py:104,128) and the
    # on-device path must produce the same streams; one OPT-1.3B-width layer
    from transformers import OPTConfig, OPTForCausalLM
    cfg = OPTConfig(vocab_size=512, hidden_size=2048, ffn_dim=8192, num_hidden_layers=1, num_attention_heads=32,
                    max_position_embeddings=64, word_embed_proj_dim=2048)
    torch.manual_seed(3)
    a = OPTForCausalLM(cfg).half().eval()
    b = copy.deepcopy(a).to(cuda_device)
    ab.apply_atlas_quantization_to_model(a, "opt", {"block_size": 128, "z_threshold": 3.0}, verbose=False)
    ab.apply_atlas_quantization_to_model(b, "opt", {"block_size": 128, "z_threshold": 3.0}, keep_on_device=True,
                                         offload_canonical=True, verbose=False)
    la = {n: m for n, m in a.named_modules() if type(m).__name__ == "QuantizedLinear"}
    lb = {n: m for n, m in b.named_modules() if type(m).__name__ == "QuantizedLinear"}
    assert len(la) == 6 and set(la) == set(lb)
    for n in la:
        assert la[n].quantized_weights.fp8_data.device.type == "cpu"
        assert lb[n].quantized_weights.fp8_data.device.type == "cpu"      # offloaded after the layout was built
        assert lb[n]._kernel_layout is not None and lb[n]._kernel_layout.tiles.device.type == "cuda"
        assert_streams_equal(la[n].quantized_weights, lb[n].quantized_weights, what=n + ": ")
    ids = torch.randint(0, 512, (1, 8), generator=torch.Generator().manual_seed(1)).to(cuda_device)
    a.to(cuda_device)
    with torch.no_grad():
        assert rel_max_err(b(ids).logits.float(), a(ids).logits.float(), discount_output_rounding=False) < 1e-3


def test_llama_pattern_with_fused_projections(cuda_device):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=704, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128)
    with torch.device(cuda_device):
        model = LlamaForCausalLM(cfg).half().eval()
    _init_like_config(model, 77)
    ref_model = copy.deepcopy(model)
    ab.apply_atlas_quantization_to_model(model, "llama", {"block_size": 64, "z_threshold": 3.0},
                                         keep_on_device=True, fuse=True, verbose=False)
    qlayers = {n: m for n, m in model.named_modules() if type(m).__name__ == "QuantizedLinear"}
    assert len(qlayers) == 14                                     # 7 per layer, lm_head excluded
    groups = {id(m._group): m._group for m in qlayers.values() if m._group is not None}
    assert len(groups) == 4 and sorted(len(g.members) for g in groups.values()) == [2, 2, 3, 3]
    for name, mod in ref_model.named_modules():
        if isinstance(mod, torch.nn.Linear) and not any(ex in name for ex in EXCLUDED):
            mod.weight.data.copy_(O.dequantize(O.quantize(mod.weight.data.cpu(), 64, 3.0)).to(cuda_device))
    ids = torch.randint(0, 512, (1, 16), generator=torch.Generator().manual_seed(9)).to(cuda_device)
    _greedy_check(model, ref_model, ids, 24, cuda_device)
    launches = sum(g.launches for g in groups.values())
    assert launches > 0                                           # the decode steps went through the joined launches
