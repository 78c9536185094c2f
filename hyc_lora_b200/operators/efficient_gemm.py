"""Attention GEMMs with compressed saved operands (reference: operators/efficient_gemm.py).

``EfficientMemoryGEMM``            Q @ K^T : saves C(Q) and C(K) (K through ``.mT``)
``EfficientMemoryGEMMWithSoftmax`` P @ V   : saves the thresholded P and C(V)
The products themselves and their backward GEMMs stay library calls; operands
are rebuilt by the decompress kernel straight into the [B,H,S,hd] layout
(efficient_gemm.py:68-72, 241-244)."""
import torch

from .. import packed as _pk
from ._common import SiteOptions, compress_site, update_static
from .compress_function import (StaticList, get_statistics_softmax, true_compress_softmax, true_decompress_softmax)


class EfficientMemoryGEMMFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x1, x2, outlier_ratio_1, sub_outlier_ratio_1, sub_outlier_bit_1, sub_outlier_quantize_method_1,
                outlier_ratio_2, sub_outlier_ratio_2, sub_outlier_bit_2, sub_outlier_quantize_method_2, rank,
                iteration, static_value_1, static_value_2, *extra):
        ctx.n_extra = len(extra)
        result = x1 @ x2
        ctx.num_heads = x1.shape[1]
        o1, o2 = (extra[0], extra[1]) if len(extra) >= 2 else (None, None)
        p1, (outlier_1, L_1, R_1, scale_1), _ = compress_site(
            x1, outlier_ratio_1, sub_outlier_ratio_1, sub_outlier_bit_1, sub_outlier_quantize_method_1, rank,
            iteration, static_value_1, o1)
        p2, (outlier_2, L_2, R_2, scale_2), _ = compress_site(
            x2.mT, outlier_ratio_2, sub_outlier_ratio_2, sub_outlier_bit_2, sub_outlier_quantize_method_2, rank,
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
        x1 = _pk.decompress(p1, num_heads=ctx.num_heads)
        x2 = _pk.decompress(p2, num_heads=ctx.num_heads).mT
        grad_input1 = grad_output @ x2.transpose(-2, -1).to(grad_output.dtype)
        grad_input2 = x1.transpose(-2, -1).to(grad_output.dtype) @ grad_output
        ctx.x_outlier_compressed = None
        return (grad_input1, grad_input2) + (None,) * (12 + ctx.n_extra)


class EfficientMemoryGEMM(torch.nn.Module):
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
        (result, outlier_1, L_1, R_1, scale_1, outlier_2, L_2, R_2, scale_2) = EfficientMemoryGEMMFunc.apply(
            x1, x2, self.outlier_ratio_1, self.sub_outlier_ratio_1, self.sub_outlier_bit_1,
            self.sub_outlier_quantize_method_1, self.outlier_ratio_2, self.sub_outlier_ratio_2,
            self.sub_outlier_bit_2, self.sub_outlier_quantize_method_2, self.rank, self.iteration,
            self.static_value_1, self.static_value_2, self.site_1, self.site_2)
        if not self.site_1.channel:
            update_static(self.static_value_1, self.iteration, outlier_1, L_1, scale_1, R_1)
            update_static(self.static_value_2, self.iteration, outlier_2, L_2, scale_2, R_2)
        self.iteration += 1
        return result


class EfficientMemoryGEMMWithSoftmaxFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x1, x2, outlier_ratio_1, outlier_ratio_2, sub_outlier_ratio_2, sub_outlier_bit_2,
                sub_outlier_quantize_method_2, rank, iteration, static_value_1, static_value_2, *extra):
        ctx.n_extra = len(extra)
        result = x1 @ x2
        ctx.num_heads = x1.shape[1]
        outlier_1 = get_statistics_softmax(x1, iteration, outlier_ratio_1) if iteration < 2 else static_value_1
        ctx.x_sparse = true_compress_softmax(x1, outlier_1, outlier_ratio_1)
        p2, (outlier_2, L_2, R_2, scale_2), _ = compress_site(
            x2, outlier_ratio_2, sub_outlier_ratio_2, sub_outlier_bit_2, sub_outlier_quantize_method_2, rank,
            iteration, static_value_2, extra[0] if extra else None)
        ctx.x_outlier_compressed = p2
        # the statistics carry no gradient: without this autograd would fill a zero tensor for each of them
        # on every backward call
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(outlier_1, outlier_2, L_2, R_2, scale_2)
        return result, outlier_1, outlier_2, L_2, R_2, scale_2

    @staticmethod
    def backward(ctx, grad_output, *unused):
        x1 = true_decompress_softmax(ctx.x_sparse)
        x2 = _pk.decompress(ctx.x_outlier_compressed, num_heads=ctx.num_heads)
        grad_input1 = grad_output @ x2.transpose(-2, -1).to(grad_output.dtype)
        grad_input2 = x1.transpose(-2, -1).to(grad_output.dtype) @ grad_output
        ctx.x_sparse = ctx.x_outlier_compressed = None
        return (grad_input1, grad_input2) + (None,) * (9 + ctx.n_extra)


class EfficientMemoryGEMMWithSoftmax(torch.nn.Module):
    def __init__(self, outlier_ratio_1: float = 0.01, outlier_ratio_2: float = 0.01, sub_outlier_ratio_2: float = 0.2,
                 sub_outlier_bit_2: int = 8, sub_outlier_quantize_method_2: str = "per-tensor", rank: int = 16, *,
                 outlier_mode: str = "element", group_size: int = 0, rotate: int = 0):
        super().__init__()
        self.outlier_ratio_1 = outlier_ratio_1
        self.outlier_ratio_2, self.sub_outlier_ratio_2 = outlier_ratio_2, sub_outlier_ratio_2
        self.sub_outlier_bit_2, self.sub_outlier_quantize_method_2 = sub_outlier_bit_2, sub_outlier_quantize_method_2
        self.rank = rank
        self.iteration = 0
        self.static_value_1 = None
        self.static_value_2 = StaticList()
        self.site_2 = SiteOptions(outlier_ratio_2, outlier_mode, group_size, rotate)

    def forward(self, x1, x2):
        result, outlier_1, outlier_2, L_2, R_2, scale_2 = EfficientMemoryGEMMWithSoftmaxFunc.apply(
            x1, x2, self.outlier_ratio_1, self.outlier_ratio_2, self.sub_outlier_ratio_2, self.sub_outlier_bit_2,
            self.sub_outlier_quantize_method_2, self.rank, self.iteration, self.static_value_1, self.static_value_2,
            self.site_2)
        if self.iteration < 2:
            self.static_value_1 = (outlier_1 if self.static_value_1 is None
                                   else (self.iteration * self.static_value_1 + outlier_1) / (self.iteration + 1))
        if not self.site_2.channel:
            update_static(self.static_value_2, self.iteration, outlier_2, L_2, scale_2, R_2)
        self.iteration += 1
        return result
