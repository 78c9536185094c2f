"""RMSNorm with a compressed saved input (reference: operators/efficient_rmsnorm.py:146-339)."""
from ._norm_common import make_norm

EfficientMemoryRMSNormFunc, EfficientMemoryRMSNorm = make_norm(
    "rms", "EfficientMemoryRMSNormFunc", "EfficientMemoryRMSNorm",
    "RMSNorm whose saved input is compressed (reference: operators/efficient_rmsnorm.py:146-339).")
