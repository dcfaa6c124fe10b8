"""Swaps a model's ``nn.Linear`` layers for ``QuantizedLinear`` (reference surface).

Mirrors the quantization half of ``integration/model_modifier.py`` of AtlasInfer
(``MODEL_LAYER_PATTERNS`` :21-50, ``find_modules`` :78-92, ``_replace_module``
:58-76, ``apply_atlas_quantization_to_model`` :95-143).  The attention-wrapper
and offload-hook halves of that file are not part of the quantization path and
are not provided here.
"""
from __future__ import annotations

import gc
import traceback
from typing import Dict, List, Optional, Tuple, Type

import torch
import torch.nn as nn

from ..quant.adaptive_quantizer import QuantizedTensor, quantize_tensor  # noqa: F401
from .atlas_wrappers import QuantizedLinear, fuse_linears, kernel_layout_supported

# Sibling projections that read the same activations: one launch per group when the applier is asked to fuse.
FUSABLE_SIBLINGS = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))


def fuse_sibling_linears(model: nn.Module) -> int:
    """Join q/k/v and gate/up ``QuantizedLinear`` siblings of every parent module into fused groups.

    The reference calls each projection separately (integration/atlas_wrappers.py:67); joined, the decode
    step issues 4 launches per Llama layer instead of 7.  Returns the number of groups made."""
    made = 0
    for parent in model.modules():
        for names in FUSABLE_SIBLINGS:
            members = [getattr(parent, n, None) for n in names]
            if not all(type(m).__name__ == "QuantizedLinear" for m in members):
                continue
            if any(getattr(m, "_group", None) is not None for m in members):
                continue
            try:
                fuse_linears(members)
                made += 1
            except ValueError:
                pass   # different in_features / block sizes: leave them as they are
    return made

# Which module types are quantized per model family (reference :21-50; only the entries the
# quantization applier reads).
MODEL_LAYER_PATTERNS = {
    family: {
        "linear_types": [nn.Linear],
        "attention_type": [f"{cls}Attention", f"{cls}SdpaAttention"],
        "decoder_layer_type": f"{cls}DecoderLayer",
        "decoder_block_path": path,
        "attention_subpath": "self_attn",
    }
    for family, cls, path in (
        ("opt", "OPT", "model.decoder.layers"),
        ("llama", "Llama", "model.layers"),
        ("mistral", "Mistral", "model.layers"),
        ("gemma", "Gemma", "model.layers"),
    )
}


def _get_model_patterns(model_type: str) -> Optional[Dict]:
    patterns = MODEL_LAYER_PATTERNS.get(model_type)
    if patterns is None:
        print(f"Warning: No layer patterns for '{model_type}'.")
    return patterns


def _as_list(v) -> list:
    if isinstance(v, list):
        return v
    return [v] if v else []


def find_modules(model: nn.Module, target_types: List[Type], target_names: List[str] = [],
                 exclude_names: List[str] = []) -> List[Tuple[str, nn.Module]]:
    """Modules whose type is in ``target_types`` or class name in ``target_names``, skipping
    any whose qualified name contains an entry of ``exclude_names`` (reference :78-92)."""
    target_types = tuple(t for t in _as_list(target_types) if t is not None)
    target_names, exclude_names = _as_list(target_names), _as_list(exclude_names)
    found = []
    for name, module in model.named_modules():
        if any(ex and ex in name for ex in exclude_names):
            continue
        if (target_types and isinstance(module, target_types)) or type(module).__name__ in target_names:
            found.append((name, module))
    return found


def _replace_module(parent_module: nn.Module, child_name: str, new_module: nn.Module):
    """Install ``new_module`` and strip the old one so its weights can be freed (reference :58-76)."""
    old = getattr(parent_module, child_name, None)
    setattr(parent_module, child_name, new_module)
    if old is None or old is new_module:
        return
    for store in ("_modules", "_parameters", "_buffers"):
        d = getattr(old, store, None)
        if d is not None:
            d.clear()


def _cleanup():
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def _split(name: str) -> Tuple[str, str]:
    return tuple(name.rsplit(".", 1)) if "." in name else ("", name)


def apply_atlas_quantization_to_model(
    model: nn.Module, model_type: str, quantization_config: Dict,
    excluded_layers: List[str] = ["lm_head", "embed_tokens", "embeddings"],
    *, quantize_device: Optional[torch.device] = None, keep_on_device: bool = False,
    fuse: bool = False, offload_canonical: bool = False, verbose: bool = True,
):
    """Quantize every non-excluded linear layer of ``model`` in place (reference :95-143).

    As in the reference the model is first brought to fp16 on the CPU and each
    ``QuantizedLinear`` holds CPU streams (they move lazily on the first forward).
    Extensions, all keyword-only: ``keep_on_device=True`` leaves the streams on the GPU
    that quantized them (no device-to-host copy and no later re-upload), and
    ``quantize_device`` picks that GPU; ``fuse=True`` joins q/k/v and gate/up siblings into one
    launch each (``fuse_sibling_linears``); ``offload_canonical=True`` (with ``keep_on_device``)
    builds every layer's kernel layout right away and moves the canonical streams to the host, so
    the GPU holds ~1.03 bytes per weight instead of ~2.07.  Layers the fused kernels cannot serve
    (in_features not a multiple of 64 or of the block size) are reported, counted as
    failed and left as ``nn.Linear``.  Returns None; failures are printed and counted.
    """
    say = print if verbose else (lambda *a, **k: None)
    say(f"\n--- Applying Atlas Quantization ({model_type}) ---")
    patterns = _get_model_patterns(model_type)
    if patterns is None:
        print("ERROR: No patterns.")
        return
    try:
        if not keep_on_device:
            model.to(dtype=torch.float16, device="cpu")
        else:
            model.to(dtype=torch.float16)
        _cleanup()
    except Exception as e:  # noqa: BLE001 - same tolerance as the reference
        print(f"Warning: Pre-quant move failed: {e}")

    linear_types = patterns.get("linear_types", [])
    if not linear_types:
        print("Warning: No linear types.")
        return
    todo = find_modules(model, target_types=linear_types, exclude_names=excluded_layers)
    if not todo:
        print("Warning: No linear layers found.")
        return

    say(f"Found {len(todo)} linear layers to quantize...")
    block_size = int(quantization_config.get("block_size", 128))
    replaced = failed = 0
    for name, module in list(todo):
        parent_name, child_name = _split(name)
        try:
            parent = model.get_submodule(parent_name) if parent_name else model
            if type(getattr(parent, child_name, None)).__name__ == "QuantizedLinear":
                continue
        except AttributeError:
            print(f"Warn: Re-verify fail {name}.")
        try:
            weight = getattr(module, "weight", None)
            if weight is None:
                print(f"Warn: No weight {name}. Skip.")
                failed += 1
                continue
            reason = kernel_layout_supported(weight.shape, block_size)
            if reason is not None:
                print(f"!! FAILED quant layer {name}: {reason}")
                failed += 1
                continue
            if keep_on_device:
                from .. import _capi
                dev = _capi.require_cuda(quantize_device or weight.device)
                w16 = weight.data.to(dtype=torch.float16, device=dev)
            else:
                w16 = weight.data.to(dtype=torch.float16, device="cpu")
            bias = module.bias.data if getattr(module, "bias", None) is not None else None
            new_bias = bias.to(dtype=torch.float16, device=w16.device).clone() if bias is not None else None
            q = quantize_tensor(w16, **quantization_config)
            parent = model.get_submodule(parent_name) if parent_name else model
            _replace_module(parent, child_name, QuantizedLinear(q, new_bias))
            replaced += 1
            del w16, q, new_bias
            if (replaced + failed) % 20 == 0:
                _cleanup()
        except Exception as e:  # noqa: BLE001 - per-layer failures are counted, as in the reference
            print(f"!! FAILED quant layer {name}: {e}")
            traceback.print_exc()
            failed += 1
    say(f"--- Quantization complete. Replaced: {replaced}, Failed/Skipped: {failed} ---")
    if fuse:
        say(f"Fused {fuse_sibling_linears(model)} groups of sibling projections.")
    if offload_canonical and keep_on_device:
        groups = set()
        for mod in model.modules():
            if type(mod).__name__ != "QuantizedLinear" or mod.quantized_weights.fp8_data.device.type != "cuda":
                continue
            g = getattr(mod, "_group", None)
            if g is not None and g.layout is None and id(g) not in groups:
                g.build(mod.quantized_weights.fp8_data.device)
                groups.add(id(g))
        for mod in model.modules():
            if type(mod).__name__ == "QuantizedLinear":
                mod.offload_canonical()
    _cleanup()
