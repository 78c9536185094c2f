"""Module replacement: install the compression operators into a host model.

Restates the rule set of the reference's drivers (train_gsm8k.py:426-592,
train_glue.py:391-493): walk ``named_children``; the first matching rule wins, otherwise
recurse.  Rules, in order:
  trainable nn.Linear with in_features > 100 that is not lm_head  -> EfficientMemoryLinear (LoRA-A)
  class name contains SiLU / GELU                                  -> EfficientMemorySiLU / GELU ("silu" group)
  class name contains RMSNorm / LayerNorm                          -> EfficientMemoryRMSNorm / LayerNorm
  nn.Softmax                                                       -> EfficientMemorySoftmax
  nn.Dropout                                                       -> EfficientMemoryDropout(0.0)
  class name contains Hadamard                                     -> EfficientMemoryHadamard
  class name contains GEMM: attribute name has "gemm1"             -> EfficientMemoryGEMM, else ...WithSoftmax
``compress_config`` maps the reference's six groups (linear, silu, layernorm, softmax, gemm,
hadamard) to {outlier_ratio, sub_outlier_ratio, sub_outlier_bit, sub_outlier_quantize_method, rank};
``extra`` carries the channel-mode keywords (outlier_mode, group_size, rotate).
"""
from __future__ import annotations

import torch.nn as nn

from ..operators.efficient_dropout import EfficientMemoryDropout
from ..operators.efficient_gelu import EfficientMemoryGELU
from ..operators.efficient_gemm import EfficientMemoryGEMM, EfficientMemoryGEMMWithSoftmax
from ..operators.efficient_hadamard import EfficientMemoryHadamard
from ..operators.efficient_layernorm import EfficientMemoryLayerNorm
from ..operators.efficient_linear import EfficientMemoryLinear
from ..operators.efficient_rmsnorm import EfficientMemoryRMSNorm
from ..operators.efficient_silu import EfficientMemorySiLU
from ..operators.efficient_softmax import EfficientMemorySoftmax

GROUPS = ("linear", "silu", "layernorm", "softmax", "gemm", "hadamard")


def uniform_config(outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=4,
                   sub_outlier_quantize_method="per-channel", rank=0, softmax_outlier_ratio=0.05):
    cfg = {g: dict(outlier_ratio=outlier_ratio, sub_outlier_ratio=sub_outlier_ratio, sub_outlier_bit=sub_outlier_bit,
                   sub_outlier_quantize_method=sub_outlier_quantize_method, rank=rank) for g in GROUPS}
    cfg["softmax"]["outlier_ratio"] = softmax_outlier_ratio
    return cfg


def _single(cfg):
    return dict(outlier_ratio=cfg["outlier_ratio"], sub_outlier_ratio=cfg["sub_outlier_ratio"],
                sub_outlier_bit=cfg["sub_outlier_bit"],
                sub_outlier_quantize_method=cfg["sub_outlier_quantize_method"], rank=cfg["rank"])


def _double(cfg):
    out = {"rank": cfg["rank"]}
    for i in (1, 2):
        out[f"outlier_ratio_{i}"] = cfg["outlier_ratio"]
        out[f"sub_outlier_ratio_{i}"] = cfg["sub_outlier_ratio"]
        out[f"sub_outlier_bit_{i}"] = cfg["sub_outlier_bit"]
        out[f"sub_outlier_quantize_method_{i}"] = cfg["sub_outlier_quantize_method"]
    return out


SKIP_NAMES = ("lm_head", "class_intermediate", "out_proj", "classifier")


def replace_module(module: nn.Module, compress_config: dict, extra: dict | None = None) -> int:
    """Swap in place; returns the number of modules replaced.  Output heads (``SKIP_NAMES``)
    are left alone: their inputs are 2-D pooled vectors, not [B, S, D] activations."""
    extra = extra or {}
    count = 0
    for name, child in module.named_children():
        cls = child.__class__.__name__
        new = None
        if (isinstance(child, nn.Linear) and not isinstance(child, EfficientMemoryLinear) and child.weight.requires_grad
                and child.in_features > 100 and name not in SKIP_NAMES):
            new = EfficientMemoryLinear(child.in_features, child.out_features, bias=child.bias is not None,
                                        **_single(compress_config["linear"]), **extra)
            new = new.to(device=child.weight.device, dtype=child.weight.dtype)
            new.weight.data = child.weight.data
            if child.bias is not None:
                new.bias.data = child.bias.data
        elif cls.startswith("EfficientMemory"):
            pass
        elif "SiLU" in cls:
            new = EfficientMemorySiLU(**_single(compress_config["silu"]), **extra)
        elif "GELU" in cls:
            new = EfficientMemoryGELU(**_single(compress_config["silu"]), **extra)
        elif "RMSNorm" in cls:
            new = EfficientMemoryRMSNorm(child.weight.shape[0], eps=getattr(child, "variance_epsilon", 1e-5), bias=False,
                                         **_single(compress_config["layernorm"]), **extra)
            new = new.to(device=child.weight.device, dtype=child.weight.dtype)
            new.weight.data = child.weight.data
            new.weight.requires_grad_(child.weight.requires_grad)
        elif "LayerNorm" in cls:
            # the reference does not forward eps here and so runs LayerNorm with 1e-5 (train_glue.py:436-447)
            new = EfficientMemoryLayerNorm(child.weight.shape[0], **_single(compress_config["layernorm"]), **extra)
            new = new.to(device=child.weight.device, dtype=child.weight.dtype)
            new.weight.data, new.bias.data = child.weight.data, child.bias.data
            new.weight.requires_grad_(child.weight.requires_grad)
            new.bias.requires_grad_(child.bias.requires_grad)
        elif isinstance(child, nn.Softmax):
            new = EfficientMemorySoftmax(compress_config["softmax"]["outlier_ratio"])
        elif isinstance(child, nn.Dropout):
            new = EfficientMemoryDropout(0.0)
        elif "Hadamard" in cls:
            new = EfficientMemoryHadamard(**_double(compress_config["hadamard"]), **extra)
        elif "GEMM" in cls:
            g = compress_config["gemm"]
            if "gemm1" in name:
                new = EfficientMemoryGEMM(**_double(g), **extra)
            else:
                new = EfficientMemoryGEMMWithSoftmax(
                    outlier_ratio_1=compress_config["softmax"]["outlier_ratio"], outlier_ratio_2=g["outlier_ratio"],
                    sub_outlier_ratio_2=g["sub_outlier_ratio"], sub_outlier_bit_2=g["sub_outlier_bit"],
                    sub_outlier_quantize_method_2=g["sub_outlier_quantize_method"], rank=g["rank"], **extra)
        if new is not None:
            setattr(module, name, new)
            count += 1
        else:
            count += replace_module(child, compress_config, extra)
    return count


replace_module_for_quantization = replace_module
