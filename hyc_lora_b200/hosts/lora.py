"""LoRA adapter around a frozen base linear.

The arithmetic is the published LoRA forward ``base(x) + B(A(x)) * (alpha / r)`` (what the
peft wrapper used by the reference computes, train_gsm8k.py:698-722).  ``lora_A`` is a
trainable ``nn.Linear`` with ``in_features > 100`` and is therefore the module the
replacement rules turn into ``EfficientMemoryLinear``; ``lora_B`` (``in_features = r``)
is left alone, as in the reference (train_gsm8k.py:428-451).

The base weight is frozen and either bf16 or held as blockwise 4-bit codebook weights.
Either way the base layer keeps NO activation for backward -- the behaviour the
reference's bitsandbytes patch exists for (bitsandbytes_fix/_function.py:515-518).
"""
from __future__ import annotations

import ctypes as C
import math

import torch
import torch.nn as nn

_CODEBOOK = None


def nf4_codebook() -> torch.Tensor:
    """The 16 levels of the 4-bit NormalFloat codebook, built from its published
    construction: 8 positive and 7 negative quantiles of N(0,1) taken at evenly spaced
    probabilities between 0.5 and an offset close to 1, plus an exact zero, normalised
    to [-1, 1]."""
    global _CODEBOOK
    if _CODEBOOK is None:
        from scipy.stats import norm
        offset = 0.5 * (1 - 1 / 32 + 1 - 1 / 30)          # midway between the two tail conventions
        pos = norm.ppf(torch.linspace(offset, 0.5, 9)[:-1].double().numpy())
        neg = -norm.ppf(torch.linspace(offset, 0.5, 8)[:-1].double().numpy())
        vals = torch.tensor(sorted(list(pos) + [0.0] + list(neg)), dtype=torch.float64)
        _CODEBOOK = (vals / vals.abs().max()).float()
    return _CODEBOOK


_CODEBOOK_DEV = {}


def _codebook_on(device) -> torch.Tensor:
    """Device copy of the codebook, made once per device (no host->device copy per call)."""
    key = str(device)
    if key not in _CODEBOOK_DEV:
        _CODEBOOK_DEV[key] = nf4_codebook().to(device)
    return _CODEBOOK_DEV[key]


@torch.no_grad()
def nf4_quantize(w: torch.Tensor, block: int = 64):
    """Blockwise absmax quantisation to the codebook.  Returns (codes uint8 [n/2], absmax fp32 [n/block])."""
    flat = w.reshape(-1, block).float()
    absmax = flat.abs().amax(dim=1).clamp_min(1e-12)
    book = nf4_codebook().to(w.device)
    idx = torch.empty(flat.shape, dtype=torch.uint8, device=w.device)
    step = max(1, (1 << 24) // block)
    for i in range(0, flat.shape[0], step):                    # chunked: the distance tensor is 16x the weight
        norm = flat[i:i + step] / absmax[i:i + step, None]
        idx[i:i + step] = (norm.unsqueeze(-1) - book).abs().argmin(dim=-1).to(torch.uint8)
    idx = idx.reshape(-1, 2)
    return ((idx[:, 0] << 4) | idx[:, 1]).contiguous(), absmax.contiguous()


def nf4_dequantize(codes: torch.Tensor, absmax: torch.Tensor, shape) -> torch.Tensor:
    from .. import _lib
    n = codes.numel() * 2
    out = torch.empty(n, dtype=torch.bfloat16, device=codes.device)
    book = _codebook_on(codes.device)
    _lib.check(_lib.lib.hyc_nf4_dequant(C.c_void_p(codes.data_ptr()), C.c_void_p(absmax.data_ptr()),
                                        C.c_void_p(book.data_ptr()), n, C.c_void_p(out.data_ptr()),
                                        C.c_void_p(torch.cuda.current_stream().cuda_stream)), "hyc_nf4_dequant")
    return out.view(shape)


def _into_carry(carry_grad, grad_out, weight, shape):
    """``carry_grad += grad_out @ weight`` in the GEMM's epilogue, or the plain product where no gradient
    has been carried this far.  The carried buffer is owned by the chain (each link hands it to exactly one
    other link), so it is updated in place."""
    g2 = grad_out.reshape(-1, grad_out.shape[-1]).to(weight.dtype)
    if carry_grad is None or not carry_grad.is_contiguous() or carry_grad.dtype != weight.dtype:
        out = (g2 @ weight).view(shape)
        return out if carry_grad is None else carry_grad + out
    carry_grad.view(-1, carry_grad.shape[-1]).addmm_(g2, weight)
    return carry_grad


class _FrozenLinearFunc(torch.autograd.Function):
    """``y = x W^T`` for a frozen W (rebuilt from 4-bit storage in forward and again in backward, or a
    frozen bf16 parameter); nothing is saved.  ``carry`` is a tensor of x's shape that is handed through
    unchanged: the gradient with respect to x is not returned for ``x`` but added, by the GEMM that makes
    it, to the gradient that arrives for the carried tensor.  A host strings the projections that read one
    activation along one carry that starts at the activation itself, and the sum of their input gradients
    costs no elementwise kernel."""

    @staticmethod
    def forward(ctx, x, carry, layer):
        ctx.layer, ctx.shape = layer, carry.shape
        ctx.set_materialize_grads(False)
        return x @ layer.dense_weight().t(), carry

    @staticmethod
    def backward(ctx, grad_out, carry_grad):
        if grad_out is None:
            return None, carry_grad, None
        return None, _into_carry(carry_grad, grad_out, ctx.layer.dense_weight(), ctx.shape), None


class FrozenLinear(nn.Module):
    """Frozen base projection (no bias).  ``quant="nf4"`` stores 4-bit codes; ``"bf16"`` a frozen
    bf16 parameter (autograd keeps no input for a weight that does not train)."""

    def __init__(self, in_features: int, out_features: int, quant: str = "bf16", device=None, std: float = 0.02,
                 generator=None, dtype=torch.bfloat16):
        super().__init__()
        self.in_features, self.out_features, self.quant = in_features, out_features, quant
        # drawn on the generator's device (CPU for reproducible small models), then moved
        gdev = generator.device if generator is not None else device
        w = torch.empty(out_features, in_features, device=gdev, dtype=torch.float32)
        w.normal_(0.0, std, generator=generator)
        w = w.to(device=device, dtype=dtype)
        if quant == "nf4":
            codes, absmax = nf4_quantize(w)
            self.register_buffer("codes", codes)
            self.register_buffer("absmax", absmax)
        else:
            self.weight = nn.Parameter(w, requires_grad=False)

    def dequantized(self) -> torch.Tensor:
        return nf4_dequantize(self.codes, self.absmax, (self.out_features, self.in_features))

    def dense_weight(self) -> torch.Tensor:
        return self.dequantized() if self.quant == "nf4" else self.weight

    def forward(self, x, carry=None):
        """``carry=None``: x W^T.  With a carry (see ``_FrozenLinearFunc``): (x W^T, the carry handed on)."""
        if carry is not None:
            return _FrozenLinearFunc.apply(x, carry, self)
        if self.quant == "nf4":
            return _FrozenLinearFunc.apply(x, x, self)[0]
        return nn.functional.linear(x, self.weight)


class _LoraMergeFunc(torch.autograd.Function):
    """``base += scaling * h @ B^T`` in place, the scale and the add in the GEMM's epilogue; backward keeps the
    scale in the two small GEMMs' epilogues too (autograd's own addmm backward multiplies in separate kernels)."""

    @staticmethod
    def forward(ctx, base, h, weight_b, scaling):
        ctx.scaling = scaling
        ctx.save_for_backward(h, weight_b)
        base.addmm_(h, weight_b.t(), alpha=scaling)
        ctx.mark_dirty(base)
        return base

    @staticmethod
    def backward(ctx, grad):
        h, weight_b = ctx.saved_tensors
        grad = grad.contiguous()
        # beta = 0: the first argument only gives shape and dtype, its contents are not read
        grad_h = torch.addmm(torch.empty_like(h), grad, weight_b, beta=0, alpha=ctx.scaling)
        sink = getattr(weight_b, "hyc_grad_sink", None)
        if sink is not None and weight_b.grad is not None and weight_b.grad.dtype == grad.dtype:
            # the owner of the gradient buffer asked for it (ddp.FlatGradSync(fused_accumulate=True)): the GEMM
            # adds into the buffer (beta = 1), which is the engine's accumulation step without a kernel of its own
            weight_b.grad.addmm_(grad.t(), h, alpha=ctx.scaling)
            sink()
            return grad, grad_h, None, None
        grad_b = torch.addmm(torch.empty_like(weight_b), grad.t(), h, beta=0, alpha=ctx.scaling)
        return grad, grad_h, grad_b, None


class LoRALinear(nn.Module):
    """``base(x) + lora_B(lora_A(x)) * scaling`` with B initialised to zero."""

    def __init__(self, in_features: int, out_features: int, r: int = 64, alpha: float = 16.0, quant: str = "bf16",
                 device=None, dtype=torch.bfloat16, generator=None):
        super().__init__()
        self.base_layer = FrozenLinear(in_features, out_features, quant, device=device, generator=generator,
                                       dtype=dtype)
        self.lora_A = nn.Linear(in_features, r, bias=False, device=device, dtype=dtype)
        self.lora_B = nn.Linear(r, out_features, bias=False, device=device, dtype=dtype)
        gdev = generator.device if generator is not None else device
        bound = 1.0 / math.sqrt(in_features)           # kaiming-uniform with a = sqrt(5)
        a = torch.empty(r, in_features, device=gdev, dtype=torch.float32).uniform_(-bound, bound, generator=generator)
        self.lora_A.weight.data.copy_(a)
        nn.init.zeros_(self.lora_B.weight)
        self.scaling = alpha / r

    def forward(self, x, carry=None):
        """``carry=None``: the adapter's output.  With a carry -- a tensor of x's shape, x itself for the
        first projection that reads x, the carry the previous one returned for the others -- the result is
        (output, carry to hand on): the input gradients of the base projection and of ``lora_A`` are added
        into the gradient that travels back along the carry by the GEMMs that make them, and x receives
        their sum without an elementwise add."""
        # base + scaling * (A x) B^T with the scale and the add in the GEMM's epilogue (no separate
        # elementwise kernels); lora_A stays a module so that it can be swapped for the compressing linear
        # (the base output is produced 2-D so that the in-place update is not an update through a view,
        # which autograd would undo with full-size copies in backward)
        chain = x if carry is None else carry
        if torch.is_grad_enabled() and chain.requires_grad:
            base, chain = self.base_layer(x.reshape(-1, x.shape[-1]), carry=chain)
            if getattr(self.lora_A, "takes_carry", False):
                h, chain = self.lora_A(x, carry=chain)
            else:
                h = self.lora_A(x)
        else:
            base = self.base_layer(x.reshape(-1, x.shape[-1]))
            h = self.lora_A(x)
        base = _LoraMergeFunc.apply(base, h.reshape(-1, h.shape[-1]), self.lora_B.weight, self.scaling)
        out = base.view(*x.shape[:-1], base.shape[-1])
        return out if carry is None else (out, chain)


def lora_parameters(model: nn.Module):
    return [p for n, p in model.named_parameters() if p.requires_grad]
