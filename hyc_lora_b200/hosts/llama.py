"""LLaMA / Mistral-shaped decoder host (RMSNorm, RoPE, SiLU-gated MLP, optional GQA).

Swap points carry the names the reference's model file gives them
(models/modeling_llama.py:103-125, 293, 817, 833, 1109): ``input_layernorm``,
``post_attention_layernorm``, ``norm`` (class name contains "RMSNorm"), ``act_fn`` (class name
contains "SiLU"), ``hadamard`` (class ``LlamaHadamard``).  Attention runs on the library's fused
causal attention (``F.scaled_dot_product_attention``), which stands in for the flash-attn call of
the reference and is not part of the compression path."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .lora import FrozenLinear, LoRALinear


@dataclass
class DecoderConfig:
    hidden: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 32
    ffn: int = 11008
    vocab: int = 32000
    eps: float = 1e-5
    rope_theta: float = 10000.0
    lora_r: int = 64
    lora_alpha: float = 16.0
    base_quant: str = "nf4"
    dtype: torch.dtype = torch.bfloat16

    @staticmethod
    def llama2_7b(**kw):
        return DecoderConfig(**kw)

    @staticmethod
    def mistral_7b(**kw):
        return DecoderConfig(kv_heads=8, ffn=14336, **kw)


class LlamaRMSNorm(nn.Module):
    def __init__(self, hidden, eps, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden, device=device), requires_grad=False)
        self.variance_epsilon = eps

    def forward(self, x):
        v = x.float().pow(2).mean(-1, keepdim=True)
        return (self.weight * (x.float() * torch.rsqrt(v + self.variance_epsilon))).to(x.dtype)


class LlamaSiLU(nn.Module):
    def forward(self, x):
        return F.silu(x)


class LlamaHadamard(nn.Module):
    def forward(self, x1, x2):
        return x1 * x2


_ROPE_TABLES = {}


def _rope_table(seq: int, head_dim: int, theta: float, device) -> torch.Tensor:
    """fp32 [seq, head_dim/2, 2] = (cos, sin) of (position, pair index), cached per device."""
    key = (seq, head_dim, float(theta), str(device))
    tab = _ROPE_TABLES.get(key)
    if tab is None:
        pos = torch.arange(seq, device=device, dtype=torch.float32)
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
        ang = torch.outer(pos, inv)
        tab = torch.stack((ang.cos(), ang.sin()), dim=-1).contiguous()
        _ROPE_TABLES[key] = tab
    return tab


class _RopeFunc(torch.autograd.Function):
    """Rotary embedding of the query and key projections ([b * s, heads * hd] bf16 in memory, contiguous, not views) by one
    in-place kernel launch; the backward is the rotation by the negative angle, applied in place to the
    incoming gradients."""

    @staticmethod
    def forward(ctx, q, k, table, hq, hk, hd, b, s):
        from .. import _lib
        from ..packed import _stream
        ctx.table, ctx.dims = table, (b * s, s, hq, hk, hd)
        _lib.check(_lib.lib.hyc_rope(q.data_ptr(), k.data_ptr(), table.data_ptr(), b * s, s, hq, hk, hd, 0, _stream()),
                   "hyc_rope")
        ctx.mark_dirty(q, k)
        return q, k

    @staticmethod
    def backward(ctx, gq, gk):
        from .. import _lib
        from ..packed import _stream
        tokens, s, hq, hk, hd = ctx.dims
        gq, gk = gq.contiguous().clone(), gk.contiguous().clone()
        _lib.check(_lib.lib.hyc_rope(gq.data_ptr(), gk.data_ptr(), ctx.table.data_ptr(), tokens, s, hq, hk, hd, 1,
                                     _stream()), "hyc_rope")
        return gq, gk, None, None, None, None, None, None


def _rope(q, k, theta, hq, hk):
    """q [b, s, hq * hd], k [b, s, hk * hd] -> rotated [b, s, heads, hd].  CUDA bf16 projections go through the
    fused kernel (in place: they are fresh tensors); anything else (the CPU hosts the fixtures are made from)
    through tensor ops."""
    b, s, _ = q.shape
    d = q.shape[-1] // hq
    tab = _rope_table(s, d, theta, q.device)
    if q.is_cuda and q.dtype == torch.bfloat16 and d % 16 == 0:
        # the kernel rotates whole tensors in place; a projection that hands out a reshaped view of its
        # (contiguous) output is rotated through that output, since an in-place Function with two results
        # may not be given views
        qb = q._base if q._base is not None else q
        kb = k._base if k._base is not None else k
        if (q.is_contiguous() and k.is_contiguous() and qb.is_contiguous() and kb.is_contiguous()
                and qb.numel() == q.numel() and kb.numel() == k.numel() and qb._base is None and kb._base is None
                and qb.data_ptr() == q.data_ptr() and kb.data_ptr() == k.data_ptr()):
            qb, kb = _RopeFunc.apply(qb, kb, tab, hq, hk, d, b, s)
            return qb.view(b, s, hq, d), kb.view(b, s, hk, d)
    q, k = q.reshape(b, s, hq, d), k.reshape(b, s, hk, d)
    cos = torch.cat((tab[..., 0], tab[..., 0]), -1).to(q.dtype)[None, :, None, :]
    sin = torch.cat((tab[..., 1], tab[..., 1]), -1).to(q.dtype)[None, :, None, :]

    def rot(x):
        x1, x2 = x[..., : d // 2], x[..., d // 2:]
        return torch.cat((-x2, x1), dim=-1)

    return q * cos + rot(q) * sin, k * cos + rot(k) * sin


class Attention(nn.Module):
    def __init__(self, c: DecoderConfig, device, gen):
        super().__init__()
        self.c = c
        hd = c.hidden // c.heads
        mk = lambda i, o: LoRALinear(i, o, c.lora_r, c.lora_alpha, c.base_quant, device=device, dtype=c.dtype,
                                     generator=gen)
        self.q_proj, self.k_proj = mk(c.hidden, c.heads * hd), mk(c.hidden, c.kv_heads * hd)
        self.v_proj, self.o_proj = mk(c.hidden, c.kv_heads * hd), mk(c.heads * hd, c.hidden)

    def forward(self, x):
        b, s, _ = x.shape
        c = self.c
        hd = c.hidden // c.heads
        # the three projections read the same x: their input gradients travel back along one carry and
        # are summed by the GEMMs that make them
        v, carry = self.v_proj(x, carry=x)
        q, carry = self.q_proj(x, carry=carry)
        k, carry = self.k_proj(x, carry=carry)
        v = v.view(b, s, c.kv_heads, hd).transpose(1, 2)
        q, k = _rope(q, k, c.rope_theta, c.heads, c.kv_heads)
        q, k = q.transpose(1, 2), k.transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=c.kv_heads != c.heads)
        return self.o_proj(o.transpose(1, 2).reshape(b, s, c.heads * hd))


class MLP(nn.Module):
    def __init__(self, c: DecoderConfig, device, gen):
        super().__init__()
        mk = lambda i, o: LoRALinear(i, o, c.lora_r, c.lora_alpha, c.base_quant, device=device, dtype=c.dtype,
                                     generator=gen)
        self.gate_proj, self.up_proj, self.down_proj = mk(c.hidden, c.ffn), mk(c.hidden, c.ffn), mk(c.ffn, c.hidden)
        self.act_fn = LlamaSiLU()
        self.hadamard = LlamaHadamard()

    def forward(self, x):
        gate, carry = self.gate_proj(x, carry=x)
        up, carry = self.up_proj(x, carry=carry)
        return self.down_proj(self.hadamard(self.act_fn(gate), up))


class DecoderLayer(nn.Module):
    def __init__(self, c, device, gen):
        super().__init__()
        self.input_layernorm = LlamaRMSNorm(c.hidden, c.eps, device)
        self.self_attn = Attention(c, device, gen)
        self.post_attention_layernorm = LlamaRMSNorm(c.hidden, c.eps, device)
        self.mlp = MLP(c, device, gen)

    def forward(self, x):
        x = x + self.self_attn(self.input_layernorm(x))
        return x + self.mlp(self.post_attention_layernorm(x))


class DecoderLM(nn.Module):
    """Causal LM host; ``forward(ids)`` returns the mean next-token cross-entropy with labels = ids."""

    def __init__(self, c: DecoderConfig, device="cuda", seed: int = 0, init_on_cpu: bool = False):
        super().__init__()
        # init_on_cpu draws every weight from a CPU generator (identical on any machine) and moves it
        gen = torch.Generator(device="cpu" if init_on_cpu else device)
        gen.manual_seed(seed)
        self.config = c
        self.embed_tokens = nn.Embedding(c.vocab, c.hidden, device=device, dtype=c.dtype)
        emb = torch.empty(c.vocab, c.hidden, device=gen.device, dtype=torch.float32).normal_(0, 1, generator=gen)
        self.embed_tokens.weight.data.copy_(emb)
        self.embed_tokens.weight.requires_grad_(False)
        self.layers = nn.ModuleList(DecoderLayer(c, device, gen) for _ in range(c.layers))
        self.norm = LlamaRMSNorm(c.hidden, c.eps, device)
        self.lm_head = FrozenLinear(c.hidden, c.vocab, "bf16", device=device, generator=gen, dtype=c.dtype)

    def forward(self, ids):
        x = self.embed_tokens(ids)
        # the first activation has no trainable producer; it must require grad for the LoRA chain rule
        x = x.requires_grad_(True) if not x.requires_grad else x
        for layer in self.layers:
            x = layer(x)
        logits = self.lm_head(self.norm(x))
        return F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), ids[:, 1:].reshape(-1))
