"""RoBERTa-shaped encoder host (post-LayerNorm, GELU FFN, eager attention).

Swap points as in the reference's model file (models/modeling_roberta.py:55, 130, 239-279,
303, 376, 391): ``gemm1`` / ``gemm2`` (class ``RobertaGEMM``), ``softmax`` (``nn.Softmax``),
``dropout`` (``nn.Dropout``), ``LayerNorm`` modules, ``intermediate_act_fn`` (class name contains
"GELU").  LoRA adapters sit on the projections named in ``lora_targets``."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .lora import FrozenLinear, LoRALinear


@dataclass
class EncoderConfig:
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    ffn: int = 3072
    vocab: int = 50265
    max_pos: int = 514
    eps: float = 1e-5
    labels: int = 2
    lora_r: int = 16
    lora_alpha: float = 16.0
    lora_targets: tuple = ("query", "value")
    dtype: torch.dtype = torch.float32


class RobertaGEMM(nn.Module):
    def forward(self, x1, x2):
        return x1 @ x2


class RobertaGELU(nn.Module):
    def forward(self, x):
        return F.gelu(x)


class _Proj(nn.Module):
    """Frozen projection with bias, optionally wrapped by a LoRA adapter."""

    def __init__(self, c, i, o, lora, device, gen):
        super().__init__()
        if lora:
            self.inner = LoRALinear(i, o, c.lora_r, c.lora_alpha, "bf16", device=device, dtype=c.dtype, generator=gen)
            self.inner.base_layer.weight.data = self.inner.base_layer.weight.data.to(c.dtype)
        else:
            self.inner = FrozenLinear(i, o, "bf16", device=device, generator=gen)
            self.inner.weight.data = self.inner.weight.data.to(c.dtype)
        self.bias = nn.Parameter(torch.zeros(o, device=device, dtype=c.dtype), requires_grad=False)

    def forward(self, x):
        return self.inner(x) + self.bias


class SelfAttention(nn.Module):
    def __init__(self, c, device, gen):
        super().__init__()
        self.c = c
        self.query = _Proj(c, c.hidden, c.hidden, "query" in c.lora_targets, device, gen)
        self.key = _Proj(c, c.hidden, c.hidden, "key" in c.lora_targets, device, gen)
        self.value = _Proj(c, c.hidden, c.hidden, "value" in c.lora_targets, device, gen)
        self.gemm1, self.gemm2 = RobertaGEMM(), RobertaGEMM()
        self.softmax = nn.Softmax(dim=-1)
        self.dropout = nn.Dropout(0.1)

    def _heads(self, x):
        b, s, _ = x.shape
        return x.view(b, s, self.c.heads, -1).permute(0, 2, 1, 3)

    def forward(self, x):
        q, k, v = self._heads(self.query(x)), self._heads(self.key(x)), self._heads(self.value(x))
        scores = self.gemm1(q, k.transpose(-1, -2)) / math.sqrt(q.shape[-1])
        probs = self.dropout(self.softmax(scores))
        ctx = self.gemm2(probs, v)
        b, h, s, hd = ctx.shape
        return ctx.permute(0, 2, 1, 3).reshape(b, s, h * hd)


class EncoderLayer(nn.Module):
    def __init__(self, c, device, gen):
        super().__init__()
        self.attention = SelfAttention(c, device, gen)
        self.attn_out = _Proj(c, c.hidden, c.hidden, "dense" in c.lora_targets, device, gen)
        self.attn_LayerNorm = nn.LayerNorm(c.hidden, eps=c.eps, device=device, dtype=c.dtype)
        self.intermediate = _Proj(c, c.hidden, c.ffn, "dense" in c.lora_targets, device, gen)
        self.intermediate_act_fn = RobertaGELU()
        self.output = _Proj(c, c.ffn, c.hidden, "dense" in c.lora_targets, device, gen)
        self.out_LayerNorm = nn.LayerNorm(c.hidden, eps=c.eps, device=device, dtype=c.dtype)
        for ln in (self.attn_LayerNorm, self.out_LayerNorm):
            ln.weight.requires_grad_(False)
            ln.bias.requires_grad_(False)

    def forward(self, x):
        x = self.attn_LayerNorm(self.attn_out(self.attention(x)) + x)
        return self.out_LayerNorm(self.output(self.intermediate_act_fn(self.intermediate(x))) + x)


class EncoderClassifier(nn.Module):
    """Sequence classifier host; ``forward(ids, labels)`` returns the cross-entropy loss."""

    def __init__(self, c: EncoderConfig, device="cuda", seed: int = 0, init_on_cpu: bool = False):
        super().__init__()
        # init_on_cpu draws every weight from a CPU generator (identical on any machine) and moves it
        gen = torch.Generator(device="cpu" if init_on_cpu else device)
        gen.manual_seed(seed)
        self.config = c
        self.word = nn.Embedding(c.vocab, c.hidden, device=device, dtype=c.dtype)
        self.pos = nn.Embedding(c.max_pos, c.hidden, device=device, dtype=c.dtype)
        for e in (self.word, self.pos):
            w = torch.empty(e.weight.shape, device=gen.device, dtype=torch.float32).normal_(0, 0.02, generator=gen)
            e.weight.data.copy_(w)
            e.weight.requires_grad_(False)
        self.emb_LayerNorm = nn.LayerNorm(c.hidden, eps=c.eps, device=device, dtype=c.dtype)
        self.emb_LayerNorm.weight.requires_grad_(False)
        self.emb_LayerNorm.bias.requires_grad_(False)
        self.layers = nn.ModuleList(EncoderLayer(c, device, gen) for _ in range(c.layers))
        # the head trains, as in the reference (its dense layer is renamed so LoRA skips it)
        self.class_intermediate = nn.Linear(c.hidden, c.hidden, device=device, dtype=c.dtype)
        self.out_proj = nn.Linear(c.hidden, c.labels, device=device, dtype=c.dtype)
        if init_on_cpu:
            for lin in (self.class_intermediate, self.out_proj):
                bound = 1.0 / math.sqrt(lin.in_features)
                for p in (lin.weight, lin.bias):
                    p.data.copy_(torch.empty(p.shape, dtype=torch.float32).uniform_(-bound, bound, generator=gen))

    def forward(self, ids, labels):
        s = ids.shape[1]
        x = self.word(ids) + self.pos(torch.arange(2, s + 2, device=ids.device))
        x = self.emb_LayerNorm(x).requires_grad_(True)
        for layer in self.layers:
            x = layer(x)
        logits = self.out_proj(torch.tanh(self.class_intermediate(x[:, 0])))
        return F.cross_entropy(logits.float(), labels)
