"""Registers this package's modules under the reference project's import paths.

AtlasInfer's callers import ``atlasinfer_core.quant.adaptive_quantizer`` and
``integration.atlas_wrappers`` / ``integration.model_modifier`` (found through
``sys.path``, e.g. ``examples/run_atlas_inference.py:15-23``).  ``install()``
puts the B200 implementations of exactly those modules into ``sys.modules``,
so the reference's other files (memory manager, helpers, offload hook, CLI)
keep working unmodified from their own checkout and pick up the CUDA path.
Call it before the first import of the reference's modules.
"""
from __future__ import annotations

import importlib
import sys
import types

_TARGETS = {
    "atlasinfer_core.quant.adaptive_quantizer": "atlasinfer_b200.quant.adaptive_quantizer",
    "integration.atlas_wrappers": "atlasinfer_b200.integration.atlas_wrappers",
}


def _ensure_package(name: str) -> types.ModuleType:
    """Import package ``name`` if a checkout provides it, else create an empty namespace."""
    if name in sys.modules:
        return sys.modules[name]
    try:
        return importlib.import_module(name)
    except Exception:  # noqa: BLE001 - any import problem of the checkout: provide a bare package
        mod = types.ModuleType(name)
        mod.__path__ = []  # mark as package
        sys.modules[name] = mod
        if "." in name:
            parent, child = name.rsplit(".", 1)
            setattr(_ensure_package(parent), child, mod)
        return mod


def install(replace_model_modifier: bool = False) -> None:
    """Make the reference's import paths resolve to the B200 implementations.

    ``integration.atlas_wrappers`` additionally keeps the reference's
    ``AtlasAttentionWrapper`` when the reference checkout is importable (it is
    outside the quantization path and left as it is).  With
    ``replace_model_modifier=True`` ``integration.model_modifier`` is replaced as
    well (quantization applier only -- use it when ``accelerate`` / ``lmdb``,
    which the reference's module imports at the top, are not installed).
    """
    targets = dict(_TARGETS)
    if replace_model_modifier:
        targets["integration.model_modifier"] = "atlasinfer_b200.integration.model_modifier"
    # the quantizer first: the reference's atlas_wrappers imports it at module level
    for ref_name in sorted(targets, key=lambda n: 0 if "quant" in n else 1):
        ours = importlib.import_module(targets[ref_name])
        parent_name, child = ref_name.rsplit(".", 1)
        parent = _ensure_package(parent_name)
        if ref_name == "integration.atlas_wrappers":
            ours = _wrappers_with_reference_attention(ours)
        sys.modules[ref_name] = ours
        setattr(parent, child, ours)


def _wrappers_with_reference_attention(ours: types.ModuleType) -> types.ModuleType:
    """Our wrappers module plus the reference's AtlasAttentionWrapper, if it can be imported."""
    sys.modules.pop("integration.atlas_wrappers", None)
    try:
        ref = importlib.import_module("integration.atlas_wrappers")
    except Exception:  # noqa: BLE001 - no reference checkout on sys.path
        return ours
    if ref is ours or not hasattr(ref, "AtlasAttentionWrapper"):
        return ours
    merged = types.ModuleType("integration.atlas_wrappers")
    merged.__dict__.update({k: v for k, v in ours.__dict__.items() if not k.startswith("__")})
    merged.__doc__ = ours.__doc__
    merged.AtlasAttentionWrapper = ref.AtlasAttentionWrapper
    return merged
