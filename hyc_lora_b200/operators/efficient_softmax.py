"""Softmax that keeps only the probabilities above a calibrated threshold for
backward (reference: operators/efficient_softmax.py).  The kept entries are a
compact per-row list written without a host sync; backward evaluates
``(g - sum(g * y_kept)) * y_kept`` from the list (efficient_softmax.py:35-45)."""
import torch
import torch.nn.functional as F

from .. import packed as _pk
from .compress_function import get_statistics_softmax, true_compress_softmax


class EfficientMemorySoftmaxFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, outlier_ratio, iteration, static_value):
        y_return = F.softmax(x, dim=-1)
        outlier = get_statistics_softmax(y_return, iteration, outlier_ratio) if iteration < 2 else static_value
        ctx.y_sparse = true_compress_softmax(y_return, outlier, outlier_ratio)
        # the statistics carry no gradient: without this autograd would fill a zero tensor for each of them
        # on every backward call
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(outlier)
        return y_return, outlier

    @staticmethod
    def backward(ctx, grad_output, grad_outlier):
        grad_input = _pk.softmax_bwd(ctx.y_sparse, grad_output)
        ctx.y_sparse = None
        return grad_input, None, None, None


class EfficientMemorySoftmax(torch.nn.Module):
    def __init__(self, outlier_ratio: float = 0.01):
        super().__init__()
        self.outlier_ratio = outlier_ratio
        self.iteration = 0
        self.static_value = None

    def forward(self, x):
        result, outlier = EfficientMemorySoftmaxFunc.apply(x, self.outlier_ratio, self.iteration, self.static_value)
        if self.iteration < 2:
            self.static_value = (outlier if self.static_value is None
                                 else (self.iteration * self.static_value + outlier) / (self.iteration + 1))
        self.iteration += 1
        return result
