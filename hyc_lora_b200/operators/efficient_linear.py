"""LoRA-A linear with a compressed saved input (reference: operators/efficient_linear.py).

Forward ``y = x W^T (+ b)`` and ``dX = dY W`` stay library GEMMs.  The weight
gradient ``dW = sum_b dY_b^T X_b`` consumes the packed activation: through the
dequant-fused tensor-core kernel when the library has it for the site's format,
else through a bf16 reconstruction and a library GEMM, as the reference does
(efficient_linear.py:61-67).

Beyond the reference: ``EfficientMemoryLinear.forward(x, carry=t)`` also hands the tensor ``t`` (of x's
shape) through unchanged, and backward adds ``dX`` into the gradient that arrives for it -- in the epilogue
of the GEMM that makes ``dX`` -- instead of returning it for ``x``.  A host that strings the projections
reading one activation along one such carry, starting at the activation itself, gets the sum of their
input gradients without elementwise adds.  And a weight that carries a ``hyc_grad_sink`` callable (set by the
owner of its gradient buffer, ``ddp.FlatGradSync(fused_accumulate=True)``) has its gradient added into
``weight.grad`` by the kernel that finishes the sums; backward then returns no gradient for it and calls the
sink."""
import torch

from .. import packed as _pk
from ._common import SiteOptions, compress_site, site_options, update_static
from .compress_function import StaticList


class EfficientMemoryLinearFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, use_bias, outlier_ratio, sub_outlier_ratio, sub_outlier_bit,
                sub_outlier_quantize_method, rank, iteration, static_value, *extra):
        ctx.use_bias = use_bias
        ctx.n_extra = len(extra)
        carry = extra[1] if len(extra) > 1 else None
        output = x @ w.transpose(0, 1) + b[None, ...] if use_bias else x @ w.transpose(0, 1)
        packed, (outlier, L, R, scale), _ = compress_site(
            x, outlier_ratio, sub_outlier_ratio, sub_outlier_bit, sub_outlier_quantize_method, rank, iteration,
            static_value, site_options(extra))
        # the statistics carry no gradient: without this autograd would fill a zero tensor for each of them
        # on every backward call
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(outlier, L, R, scale)
        ctx.x_outlier_compressed = packed
        ctx.save_for_backward(w)
        if carry is not None:
            return output, outlier, L, R, scale, carry
        return output, outlier, L, R, scale

    @staticmethod
    def backward(ctx, grad_output, grad_outlier, grad_L, grad_R, grad_scale, *grad_carry):
        (w,) = ctx.saved_tensors
        packed = ctx.x_outlier_compressed
        ctx.x_outlier_compressed = None
        grad_input = grad_weight = grad_bias = None
        carried = grad_carry[0] if grad_carry else None
        if grad_output is not None:
            if grad_carry:
                if ctx.needs_input_grad[12]:
                    g2 = grad_output.reshape(-1, grad_output.shape[-1]).to(w.dtype)
                    if carried is None:
                        carried = (g2 @ w).view(*grad_output.shape[:-1], w.shape[1])
                    elif carried.is_contiguous() and carried.dtype == w.dtype:
                        # the buffer travels from one link of the chain to the next and belongs to nobody else
                        carried.view(-1, w.shape[1]).addmm_(g2, w)
                    else:
                        carried = carried + (g2 @ w).view(carried.shape)
            elif ctx.needs_input_grad[0]:
                grad_input = grad_output.to(w.dtype) @ w
            if ctx.needs_input_grad[1]:
                sink = getattr(w, "hyc_grad_sink", None)
                if sink is not None and w.grad is not None and w.grad.dtype == w.dtype:
                    # the owner of the gradient buffer asked for it (see ddp.FlatGradSync): the kernel that finishes
                    # the sums adds them into ``w.grad`` -- the engine's accumulation step without a kernel of its
                    # own -- and the owner is told that this gradient is in
                    _pk.lora_wgrad(packed, grad_output, accumulate_into=w.grad)
                    sink()
                else:
                    out_dtype = w.dtype if w.dtype in (torch.bfloat16, torch.float32) else torch.float32
                    grad_weight = _pk.lora_wgrad(packed, grad_output, out_dtype=out_dtype).to(w.dtype)
            if ctx.use_bias and ctx.needs_input_grad[2]:
                grad_bias = grad_output.to(torch.bfloat16).sum(0)
        grads = [grad_input, grad_weight, grad_bias] + [None] * (8 + ctx.n_extra)
        if grad_carry:
            grads[12] = carried
        return tuple(grads)


class EfficientMemoryLinear(torch.nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, outlier_ratio: float = 0.01,
                 sub_outlier_ratio: float = 0.2, sub_outlier_bit: int = 8,
                 sub_outlier_quantize_method: str = "per-tensor", rank: int = 16, *,
                 outlier_mode: str = "element", group_size: int = 0, rotate: int = 0):
        super().__init__(in_features, out_features, bias)
        self.outlier_ratio = outlier_ratio
        self.sub_outlier_ratio = sub_outlier_ratio
        self.sub_outlier_bit = sub_outlier_bit
        self.sub_outlier_quantize_method = sub_outlier_quantize_method
        self.rank = rank
        self.iteration = 0
        self.static_value = StaticList()
        self.site = SiteOptions(outlier_ratio, outlier_mode, group_size, rotate)

    takes_carry = True

    def forward(self, input: torch.Tensor, carry: torch.Tensor = None):
        extra = (self.site,) if carry is None else (self.site, carry)
        result, outlier, L, R, scale, *carried = EfficientMemoryLinearFunc.apply(
            input, self.weight, self.bias, self.bias is not None, self.outlier_ratio, self.sub_outlier_ratio,
            self.sub_outlier_bit, self.sub_outlier_quantize_method, self.rank, self.iteration, self.static_value,
            *extra)
        if not self.site.channel:
            update_static(self.static_value, self.iteration, outlier, L, scale, R)
        self.iteration += 1
        return result if carry is None else (result, carried[0])
