"""Gemma RMSNorm ((1 + w) scaling) with a compressed saved input (reference: operators/efficient_rmsnorm_gemma.py)."""
from ._norm_common import make_norm

EfficientMemoryRMSNormGemmaFunc, EfficientMemoryRMSNormGemma = make_norm(
    "rms_gemma", "EfficientMemoryRMSNormGemmaFunc", "EfficientMemoryRMSNormGemma",
    "Gemma RMSNorm whose saved input is compressed (reference: operators/efficient_rmsnorm_gemma.py:147-340).")
