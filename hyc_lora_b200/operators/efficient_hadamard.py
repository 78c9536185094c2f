"""Element-wise product ``x1 * x2`` of the gated MLP with both operands compressed
(reference: operators/efficient_hadamard.py; despite the name it is a Hadamard
PRODUCT, not a transform).  Backward ``g * x2_hat`` and ``x1_hat * g`` runs in
one kernel over both packed operands (efficient_hadamard.py:56-66)."""
import torch

from .. import packed as _pk
from ._common import SiteOptions, compress_site, fused_site, norm_output_ready, update_static
from .compress_function import StaticList


def _same_format(p1, p2) -> bool:
    return (p1.mode == p2.mode and p1.bits == p2.bits and p1.group == p2.group and p1.rotate == p2.rotate
            and p1.rows == p2.rows and p1.cols == p2.cols)


class EfficientMemoryHadamardFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x1, x2, outlier_ratio_1, sub_outlier_ratio_1, sub_outlier_bit_1, sub_outlier_quantize_method_1,
                outlier_ratio_2, sub_outlier_ratio_2, sub_outlier_bit_2, sub_outlier_quantize_method_2, rank,
                iteration, static_value_1, static_value_2, *extra):
        ctx.n_extra = len(extra)
        o1, o2 = (extra[0], extra[1]) if len(extra) >= 2 else (None, None)
        # x1 is, in the gated MLP, the activation's output: its record usually exists already (shared table)
        p1, (outlier_1, L_1, R_1, scale_1), _ = compress_site(
            x1, outlier_ratio_1, sub_outlier_ratio_1, sub_outlier_bit_1, sub_outlier_quantize_method_1, rank,
            iteration, static_value_1, o1)
        fused = fused_site("product", x2, sub_outlier_bit_2, iteration, o2, x1=x1)
        if fused is not None:
            # one kernel: the product, the record of x2 and (once a reader is known) of the product
            p2, result = fused
            outlier_2, L_2, R_2, scale_2 = o2.dummy_stats(x2.device)
        else:
            result = x1 * x2
            p2, (outlier_2, L_2, R_2, scale_2), _ = compress_site(
                x2, outlier_ratio_2, sub_outlier_ratio_2, sub_outlier_bit_2, sub_outlier_quantize_method_2, rank,
                iteration, static_value_2, o2)
        ctx.x_outlier_compressed = (p1, p2)
        # the statistics carry no gradient: without this autograd would fill a zero tensor for each of them
        # on every backward call
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(outlier_1, outlier_2, L_1, R_1, scale_1, L_2, R_2, scale_2)
        return result, outlier_1, L_1, R_1, scale_1, outlier_2, L_2, R_2, scale_2

    @staticmethod
    def backward(ctx, grad_output, *unused):
        p1, p2 = ctx.x_outlier_compressed
        g = grad_output if grad_output.dtype in (torch.bfloat16, torch.float32) else grad_output.float()
        g2d = g.reshape(-1, g.shape[-1])
        if _same_format(p1, p2):
            d1, d2 = _pk.act_bwd("product", p1, g2d, p2)
        else:
            # operands stored in different formats: rebuild each and multiply
            d1 = g2d * _pk.decompress(p2).reshape(g2d.shape)
            d2 = _pk.decompress(p1).reshape(g2d.shape) * g2d
        ctx.x_outlier_compressed = None
        return (d1.reshape(grad_output.shape), d2.reshape(grad_output.shape)) + (None,) * (12 + ctx.n_extra)


class EfficientMemoryHadamard(torch.nn.Module):
    def __init__(self, outlier_ratio_1: float = 0.01, sub_outlier_ratio_1: float = 0.2, sub_outlier_bit_1: int = 8,
                 sub_outlier_quantize_method_1: str = "per-tensor", outlier_ratio_2: float = 0.01,
                 sub_outlier_ratio_2: float = 0.2, sub_outlier_bit_2: int = 8,
                 sub_outlier_quantize_method_2: str = "per-tensor", rank: int = 16, *,
                 outlier_mode: str = "element", group_size: int = 0, rotate: int = 0):
        super().__init__()
        self.outlier_ratio_1, self.sub_outlier_ratio_1 = outlier_ratio_1, sub_outlier_ratio_1
        self.sub_outlier_bit_1, self.sub_outlier_quantize_method_1 = sub_outlier_bit_1, sub_outlier_quantize_method_1
        self.outlier_ratio_2, self.sub_outlier_ratio_2 = outlier_ratio_2, sub_outlier_ratio_2
        self.sub_outlier_bit_2, self.sub_outlier_quantize_method_2 = sub_outlier_bit_2, sub_outlier_quantize_method_2
        self.rank = rank
        self.iteration = 0
        self.static_value_1 = StaticList()
        self.static_value_2 = StaticList()
        self.site_1 = SiteOptions(outlier_ratio_1, outlier_mode, group_size, rotate)
        self.site_2 = SiteOptions(outlier_ratio_2, outlier_mode, group_size, rotate)

    def forward(self, x1, x2):
        (result, outlier_1, L_1, R_1, scale_1, outlier_2, L_2, R_2, scale_2) = EfficientMemoryHadamardFunc.apply(
            x1, x2, self.outlier_ratio_1, self.sub_outlier_ratio_1, self.sub_outlier_bit_1,
            self.sub_outlier_quantize_method_1, self.outlier_ratio_2, self.sub_outlier_ratio_2,
            self.sub_outlier_bit_2, self.sub_outlier_quantize_method_2, self.rank, self.iteration,
            self.static_value_1, self.static_value_2, self.site_1, self.site_2)
        if not self.site_1.channel:
            update_static(self.static_value_1, self.iteration, outlier_1, L_1, scale_1, R_1)
            update_static(self.static_value_2, self.iteration, outlier_2, L_2, scale_2, R_2)
        else:
            # the linear behind the product saves ``result``: hand it the record made in the same pass
            norm_output_ready(result, self.site_2, self.iteration)
        self.iteration += 1
        # the reference empties the CUDA cache here on every call (efficient_hadamard.py:181); that
        # stalls the allocator and is left out
        return result
