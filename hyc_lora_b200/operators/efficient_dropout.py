"""Dropout whose mask is regenerated in backward from a seed instead of being
stored (reference: operators/efficient_dropout.py).  The reference's drivers
always build it with ``p = 0`` (train_gsm8k.py:540-541), where it is the
identity; for ``p > 0`` the mask comes from a seeded device generator."""
import torch


class EfficientMemoryDropoutFunc(torch.autograd.Function):
    @staticmethod
    def _mask(x, p, seed):
        gen = torch.Generator(device=x.device)
        gen.manual_seed(int(seed))
        return torch.rand(x.shape, device=x.device, generator=gen) > p

    @staticmethod
    def forward(ctx, x, p, seed):
        ctx.p, ctx.seed = p, seed
        if p == 0.0:
            return x.clone()
        return torch.where(EfficientMemoryDropoutFunc._mask(x, p, seed), x / (1 - p), torch.zeros_like(x))

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.p == 0.0:
            return grad_output, None, None
        keep = EfficientMemoryDropoutFunc._mask(grad_output, ctx.p, ctx.seed)
        return torch.where(keep, grad_output / (1 - ctx.p), torch.zeros_like(grad_output)), None, None


class EfficientMemoryDropout(torch.nn.Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p
        self.seed = 0

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        self.seed += 1
        return EfficientMemoryDropoutFunc.apply(x, self.p, self.seed)
