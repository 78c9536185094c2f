"""LayerNorm with a compressed saved input (reference: operators/efficient_layernorm.py:203-405)."""
from ._norm_common import make_norm

EfficientMemoryLayerNormFunc, EfficientMemoryLayerNorm = make_norm(
    "ln", "EfficientMemoryLayerNormFunc", "EfficientMemoryLayerNorm",
    "LayerNorm whose saved input is compressed (reference: operators/efficient_layernorm.py:203-405).")
