"""B200-native implementation of AtlasInfer's adaptive hybrid quantization path.

Public surface (same names as the reference project):

* ``QuantizedTensor``, ``quantize_tensor``, ``dequantize_tensor``,
  ``clear_dequantized_cache``  -- ``atlasinfer_b200.quant.adaptive_quantizer``
* ``QuantizedLinear``          -- ``atlasinfer_b200.integration.atlas_wrappers``
* ``apply_atlas_quantization_to_model`` -- ``atlasinfer_b200.integration.model_modifier``
* ``dropin.install()`` registers these under the reference's module paths.

All arithmetic runs in ``lib/libatlas_b200.so`` (build: ``python -m atlasinfer_b200.build``).
"""
from .quant.adaptive_quantizer import (QuantizedTensor, clear_dequantized_cache, dequantize_tensor,
                                       quantize_tensor)
from .integration.atlas_wrappers import QuantizedLinear
from .integration.model_modifier import apply_atlas_quantization_to_model

__all__ = [
    "QuantizedTensor", "quantize_tensor", "dequantize_tensor", "clear_dequantized_cache",
    "QuantizedLinear", "apply_atlas_quantization_to_model",
]
__version__ = "0.1.0"
