"""Synthetic-data fine-tuning step on a host model with the compression operators installed.

``build_trainer`` makes the model (random-init frozen base, LoRA adapters), installs the
operators with the replacement rules, and returns a ``Trainer`` whose ``step(ids)`` runs
forward, backward, the LoRA-gradient exchange across ranks and the optimizer update."""
from __future__ import annotations

import torch

from ..ddp import FlatGradSync
from .llama import DecoderConfig, DecoderLM
from .lora import lora_parameters
from .replace import replace_module, uniform_config


class Trainer:
    def __init__(self, model, lr: float = 1e-4):
        self.model = model
        self.params = lora_parameters(model)
        self.sync = FlatGradSync(self.params)
        self.opt = torch.optim.AdamW(self.params, lr=lr, fused=True)

    def trainable(self) -> int:
        return self.sync.numel()

    def step(self, ids: torch.Tensor) -> torch.Tensor:
        self.sync.zero()
        loss = self.model(ids)
        loss.backward()
        self.sync.sync()
        self.opt.step()
        return loss.detach()


def build_trainer(arch: str = "llama2_7b", layers: int | None = None, bits: int = 4, outlier_ratio: float = 0.01,
                  rotate: int = 256, group_size: int = 0, outlier_mode: str = "channel", base_quant: str = "nf4",
                  lora_r: int = 64, device="cuda", seed: int = 0, compress: bool = True) -> Trainer:
    kw = dict(lora_r=lora_r, base_quant=base_quant)
    if layers is not None:
        kw["layers"] = layers
    cfg = DecoderConfig.mistral_7b(**kw) if arch == "mistral_7b" else DecoderConfig.llama2_7b(**kw)
    model = DecoderLM(cfg, device=device, seed=seed)
    # LoRA-B starts at zero (as in the reference's adapters); training moves it at once
    if compress:
        extra = dict(outlier_mode=outlier_mode, group_size=group_size, rotate=rotate) if outlier_mode == "channel" else {}
        replace_module(model, uniform_config(outlier_ratio=outlier_ratio, sub_outlier_bit=bits,
                                             sub_outlier_quantize_method="per-channel"), extra)
    return Trainer(model)
