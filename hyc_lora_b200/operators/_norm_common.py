"""One implementation behind the three norm operator files (the reference duplicates the file three
times: operators/efficient_rmsnorm.py, efficient_rmsnorm_gemma.py, efficient_layernorm.py).

``make_norm(kind, ...)`` returns the autograd Function and the module class for one norm kind.  One fused
kernel computes the norm output and compresses the norm INPUT (what the reference saves,
efficient_rmsnorm.py:179-205, efficient_layernorm.py:236-262); backward decompresses and applies the
reference's formula in one kernel (efficient_rmsnorm.py:214-269, efficient_layernorm.py:275-335), with fp32
lock-free partials for the weight gradient."""
import torch

from .. import packed as _pk
from ._common import SiteOptions, compress_site, norm_output_ready, site_options, update_static
from .compress_function import StaticList


def make_norm(kind: str, func_name: str, module_name: str, doc: str):
    class NormFunc(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, normalized_shape, outlier_ratio, sub_outlier_ratio, sub_outlier_bit,
                    sub_outlier_quantize_method, rank, weight, bias, eps, iteration, static_value, *extra):
            ctx.n_extra = len(extra)
            x = x.contiguous()
            if x.shape[-1] * x.element_size() >= 65536:
                raise RuntimeError("This layer norm doesn't support feature dim >= 64KB.")
            norm = dict(kind=kind, weight=weight, bias=bias, eps=eps)
            packed, (outlier, L, R, scale), (y, rstd, mean) = compress_site(
                x, outlier_ratio, sub_outlier_ratio, sub_outlier_bit, sub_outlier_quantize_method, rank, iteration,
                static_value, site_options(extra), norm=norm)
            # the statistics carry no gradient: without this autograd would fill a zero tensor for each of them
            # on every backward call
            ctx.set_materialize_grads(False)
            ctx.mark_non_differentiable(outlier, L, R, scale)
            ctx.x_outlier_compressed = packed
            ctx.save_for_backward(weight, mean if mean is not None else rstd, rstd)
            ctx.has_mean = mean is not None
            ctx.ref_compat_c2 = getattr(site_options(extra), "ref_compat_c2", True) if extra else True
            return y, outlier, L, R, scale

        @staticmethod
        def backward(ctx, dy, grad_outlier, grad_L, grad_R, grad_scale):
            weight, mean, rstd = ctx.saved_tensors
            packed = ctx.x_outlier_compressed
            need_dw = ctx.needs_input_grad[7]
            dx, dw, _db = _pk.norm_bwd(packed, dy.reshape(-1, dy.shape[-1]), weight, rstd, mean if ctx.has_mean else None,
                                       kind, ref_compat_c2=ctx.ref_compat_c2, need_dweight=need_dw, need_dbias=False)
            ctx.x_outlier_compressed = None
            dx = dx.reshape(dy.shape)
            if dw is not None:
                dw = dw.to(weight.dtype)
            # the reference returns no gradient for the bias (last line of its backward)
            return (dx, None, None, None, None, None, None, dw, None, None, None, None) + (None,) * ctx.n_extra

    class NormModule(torch.nn.LayerNorm):
        def __init__(self, normalized_shape, eps=1e-05, elementwise_affine=True, bias=True, outlier_ratio: float = 0.01,
                     sub_outlier_ratio: float = 0.2, sub_outlier_bit: int = 8,
                     sub_outlier_quantize_method: str = "per-tensor", rank: int = 16, *,
                     outlier_mode: str = "element", group_size: int = 0, rotate: int = 0, ref_compat_c2: bool = True):
            super().__init__(normalized_shape, eps, elementwise_affine, bias)
            self.outlier_ratio = outlier_ratio
            self.sub_outlier_ratio = sub_outlier_ratio
            self.sub_outlier_bit = sub_outlier_bit
            self.sub_outlier_quantize_method = sub_outlier_quantize_method
            self.rank = rank
            self.iteration = 0
            self.static_value = StaticList()
            self.site = SiteOptions(outlier_ratio, outlier_mode, group_size, rotate)
            # keep the reference's mean(w*dy) term in the RMSNorm backward unless told otherwise
            self.site.ref_compat_c2 = ref_compat_c2

        def forward(self, x):
            result, outlier, L, R, scale = NormFunc.apply(
                x, self.normalized_shape, self.outlier_ratio, self.sub_outlier_ratio, self.sub_outlier_bit,
                self.sub_outlier_quantize_method, self.rank, self.weight, self.bias, self.eps, self.iteration,
                self.static_value, self.site)
            if not self.site.channel:
                update_static(self.static_value, self.iteration, outlier, L, scale, R)
            else:
                # the sites behind this norm save ``result``: hand them the record made in the same pass
                norm_output_ready(result, self.site, self.iteration)
            self.iteration += 1
            return result

    NormFunc.__name__ = NormFunc.__qualname__ = func_name
    NormModule.__name__ = NormModule.__qualname__ = module_name
    NormFunc.__doc__ = NormModule.__doc__ = doc
    return NormFunc, NormModule
