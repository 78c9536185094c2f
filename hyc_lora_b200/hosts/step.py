"""Synthetic-data fine-tuning step on a host model with the compression operators installed.

``build_trainer`` makes the model (random-init frozen base, LoRA adapters), installs the
operators with the replacement rules, and returns a ``Trainer`` whose ``step(ids)`` runs
forward, backward, the LoRA-gradient exchange across ranks and the optimizer update."""
from __future__ import annotations

import torch

from .. import packed
from ..ddp import FlatGradSync
from .llama import DecoderConfig, DecoderLM
from .lora import lora_parameters
from .replace import replace_module, uniform_config


class Trainer:
    """Forward, backward, LoRA-gradient exchange and AdamW update of one step.

    ``capture()`` records the whole step into a CUDA graph once every site has finished
    calibrating (three eager steps): the step launches a few thousand small kernels, and
    replaying them from a graph removes the host-side launch cost that otherwise leaves the
    GPU idle between them.  Calibration state lives in Python and is frozen by then, and no
    steady-state operator call synchronises with the host, so the recorded step is the
    steady-state step."""

    def __init__(self, model, lr: float = 1e-4):
        self.model = model
        self.params = lora_parameters(model)
        self.sync = FlatGradSync(self.params, overlap=True, fused_accumulate=True)
        self.opt = torch.optim.AdamW(self.params, lr=lr, fused=True, capturable=True)
        self.graph = None
        self.static_ids = None
        self.static_loss = None
        self.eager_steps = 0

    def trainable(self) -> int:
        return self.sync.numel()

    def _step(self, ids: torch.Tensor) -> torch.Tensor:
        self.sync.zero()
        loss = self.model(ids)
        self.sync.begin()                    # buckets of the flat gradient go out as backward completes them
        loss.backward()
        self.sync.sync()
        self.opt.step()
        packed.fold_status(loss.device)      # OR this step's status words into the device accumulator
        return loss.detach()

    def capture(self, ids: torch.Tensor) -> bool:
        """Record the step for ``ids``' shape.  Returns False (and stays eager) if capture fails."""
        while self.eager_steps < 3:          # calibration calls and optimizer state first
            self.step(ids)
        try:
            torch.cuda.synchronize()
            self.static_ids = ids.clone()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.static_loss = self._step(self.static_ids)
            torch.cuda.synchronize()
            self.graph = graph
            return True
        except Exception:
            self.graph = None
            torch.cuda.synchronize()
            return False

    def step(self, ids: torch.Tensor) -> torch.Tensor:
        # what the device flagged during earlier steps (pool overflow: warning; expired wait: error); no blocking
        packed.poll_status()
        if self.graph is not None:
            self.static_ids.copy_(ids, non_blocking=True)
            self.graph.replay()
            return self.static_loss
        self.eager_steps += 1
        return self._step(ids)


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
