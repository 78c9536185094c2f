"""SiLU with a compressed saved input (reference: operators/efficient_silu.py).

Forward is the exact activation; backward decompresses the saved input and
applies the reference's derivative formula in one kernel (efficient_silu.py:44-53)."""
import torch
import torch.nn.functional as F

from .. import packed as _pk
from ._common import SiteOptions, compress_site, fused_site, norm_output_ready, site_options, update_static
from .compress_function import StaticList


class EfficientMemorySiLUFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, outlier_ratio, sub_outlier_ratio, sub_outlier_bit, sub_outlier_quantize_method, rank,
                iteration, static_value, *extra):
        ctx.n_extra = len(extra)
        opts = site_options(extra)
        fused = fused_site("silu", x, sub_outlier_bit, iteration, opts)
        if fused is not None:
            # one kernel: the activation, the record of its input and (once a reader is known) of its output
            packed, result = fused
            outlier, L, R, scale = opts.dummy_stats(x.device)
        else:
            result = F.silu(x)
            packed, (outlier, L, R, scale), _ = compress_site(
                x, outlier_ratio, sub_outlier_ratio, sub_outlier_bit, sub_outlier_quantize_method, rank, iteration,
                static_value, opts)
        ctx.x_outlier_compressed = packed
        # the statistics carry no gradient: without this autograd would fill a zero tensor for each of them
        # on every backward call
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(outlier, L, R, scale)
        return result, outlier, L, R, scale

    @staticmethod
    def backward(ctx, grad_output, grad_outlier, grad_L, grad_R, grad_scale):
        packed = ctx.x_outlier_compressed
        # the result has the dtype torch's promotion gives bf16 (the reconstruction) and the gradient
        g = grad_output if grad_output.dtype in (torch.bfloat16, torch.float32) else grad_output.float()
        grad_input = _pk.act_bwd("silu", packed, g.reshape(-1, g.shape[-1])).reshape(grad_output.shape)
        ctx.x_outlier_compressed = None
        return (grad_input,) + (None,) * (7 + ctx.n_extra)


class EfficientMemorySiLU(torch.nn.Module):
    def __init__(self, outlier_ratio: float = 0.01, sub_outlier_ratio: float = 0.2, sub_outlier_bit: int = 8,
                 sub_outlier_quantize_method: str = "per-tensor", rank: int = 16, *,
                 outlier_mode: str = "element", group_size: int = 0, rotate: int = 0):
        super().__init__()
        self.outlier_ratio = outlier_ratio
        self.sub_outlier_ratio = sub_outlier_ratio
        self.sub_outlier_bit = sub_outlier_bit
        self.sub_outlier_quantize_method = sub_outlier_quantize_method
        self.rank = rank
        self.iteration = 0
        self.static_value = StaticList()
        self.site = SiteOptions(outlier_ratio, outlier_mode, group_size, rotate)

    def forward(self, input):
        result, outlier, L, R, scale = EfficientMemorySiLUFunc.apply(
            input, self.outlier_ratio, self.sub_outlier_ratio, self.sub_outlier_bit,
            self.sub_outlier_quantize_method, self.rank, self.iteration, self.static_value, self.site)
        if not self.site.channel:
            update_static(self.static_value, self.iteration, outlier, L, scale, R)
        else:
            # the site behind this one saves ``result``: hand it the record made in the same pass
            norm_output_ready(result, self.site, self.iteration)
        self.iteration += 1
        return result
