"""B200-native implementation of AtlasInfer's adaptive hybrid quantization path.

Public surface (same names as the reference project):

* ``QuantizedTensor``, ``quantize_tensor``, ``dequantize_tensor``,
  ``clear_dequantized_cache``  -- ``atlasinfer_b200.quant.adaptive_quantizer``
* ``QuantizedLinear``          -- ``atlasinfer_b200.integration.atlas_wrappers``
* ``apply_atlas_quantization_to_model`` -- ``atlasinfer_b200.integration.model_modifier``
* ``dropin.install()`` registers these under the reference's module paths.

Additions next to that surface: ``quantize_tensors`` (batched), ``fuse_linears`` /
``fuse_sibling_linears`` (q/k/v and gate/up as one launch), ``save_quantized*`` /
``load_quantized*`` (on-disk format).

All arithmetic runs in ``lib/libatlas_b200.so`` (build: ``python -m atlasinfer_b200.build``).
"""
from .quant.adaptive_quantizer import (QuantizedTensor, clear_dequantized_cache, dequantize_tensor,
                                       quantize_tensor, quantize_tensors)
from .quant.serialization import (load_quantized, load_quantized_model, load_quantized_state, save_quantized,
                                  save_quantized_model, save_quantized_state)
from .integration.atlas_wrappers import FusedLinearGroup, QuantizedLinear, fuse_linears
from .integration.model_modifier import apply_atlas_quantization_to_model, fuse_sibling_linears

__all__ = [
    "QuantizedTensor", "quantize_tensor", "dequantize_tensor", "clear_dequantized_cache",
    "QuantizedLinear", "apply_atlas_quantization_to_model",
    # additions to the reference's surface
    "quantize_tensors", "fuse_linears", "fuse_sibling_linears", "FusedLinearGroup",
    "save_quantized", "load_quantized", "save_quantized_state", "load_quantized_state",
    "save_quantized_model", "load_quantized_model",
]
__version__ = "0.1.0"
