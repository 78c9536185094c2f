"""Pin the oracle's norm formulas independently of how they were written down.

``oracle.hyc_oracle.norm_forward`` / ``norm_backward`` restate the reference's Triton kernels
(operators/efficient_rmsnorm.py:40-60,92-108, operators/efficient_layernorm.py:33-62,131-148), which
cannot run without a GPU.  Here the same quantities are derived a second way: the forward formula is
written in fp64 and differentiated by autograd.  LayerNorm's dx must equal the autograd gradient; the
RMSNorm dx must equal it once the reference's extra ``mean(w * dy) * rstd`` term (the LayerNorm term its
RMSNorm kernel keeps, efficient_rmsnorm.py:103-104) is subtracted, and must equal it exactly as it stands
with ``ref_compat_c2=False``.  Tolerance: the oracle returns dx in bf16 (2^-8 relative) from fp32 math."""
import pytest
import torch

from oracle import hyc_oracle as oc


def _problem(kind, rows=24, d=768, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, d, generator=g) * 1.5 + 0.3).to(torch.bfloat16)
    w = (1 + 0.2 * torch.randn(d, generator=g)).to(torch.bfloat16)
    b = (0.1 * torch.randn(d, generator=g)).to(torch.bfloat16) if kind == "ln" else None
    dy = (torch.randn(rows, d, generator=g) + 0.75).to(torch.bfloat16)   # a non-zero mean makes the mean(w*dy) term matter
    return x, w, b, dy


def _forward64(x, w, b, eps, kind):
    w = w + 1.0 if kind == "rms_gemma" else w
    if kind == "ln":
        mu = x.mean(-1, keepdim=True)
        xc = x - mu
        return xc * torch.rsqrt((xc * xc).mean(-1, keepdim=True) + eps) * w + b
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


@pytest.mark.parametrize("kind", ["rms", "rms_gemma", "ln"])
def test_norm_forward_matches_the_formula_and_the_library_norms(kind):
    x, w, b, _ = _problem(kind)
    y, mean, rstd = oc.norm_forward(x, w, b, 1e-5, kind)
    want = _forward64(x.double(), w.double(), None if b is None else b.double(), 1e-5, kind)
    assert y.dtype == x.dtype
    assert torch.equal(y, want.to(torch.bfloat16)) or (y.double() - want).abs().max() <= 2 ** -8 * want.abs().max()
    x64 = x.double()
    if kind == "ln":
        lib = torch.nn.functional.layer_norm(x64, (x.shape[-1],), w.double(), b.double(), 1e-5)
        assert (want - lib).abs().max() < 1e-9
        assert torch.allclose(mean.double(), x64.mean(-1), atol=1e-6)
        var = x64.var(-1, unbiased=False)
    else:
        # the formula of the model file's own RMSNorm module (models/modeling_llama.py:136-141)
        ww = w.double() + (1.0 if kind == "rms_gemma" else 0.0)
        lib = ww * (x64 * torch.rsqrt(x64.pow(2).mean(-1, keepdim=True) + 1e-5))
        assert (want - lib).abs().max() < 1e-9
        var = x64.pow(2).mean(-1)
    assert torch.allclose(rstd.double(), torch.rsqrt(var + 1e-5), rtol=1e-5)


@pytest.mark.parametrize("kind", ["rms", "rms_gemma", "ln"])
def test_norm_backward_matches_autograd_of_the_forward_formula(kind):
    x, w, b, dy = _problem(kind, seed=1)
    _, mean, rstd = oc.norm_forward(x, w, b, 1e-5, kind)
    x64 = x.double().requires_grad_(True)
    w64 = w.double().requires_grad_(True)
    b64 = None if b is None else b.double().requires_grad_(True)
    y64 = _forward64(x64, w64, b64, 1e-5, kind)
    grads = torch.autograd.grad(y64, [x64, w64] + ([b64] if b64 is not None else []), dy.double())
    dx_true, dw_true = grads[0], grads[1]
    tol = lambda t: 2 ** -7 * t.abs().max()

    dx, dw, db = oc.norm_backward(x, dy, w, mean, rstd, kind, ref_compat_c2=False)
    assert dx.dtype == torch.bfloat16
    assert (dx.double() - dx_true).abs().max() <= tol(dx_true)
    assert (dw.double() - dw_true).abs().max() <= 1e-4 * dw_true.abs().max()
    if kind == "ln":
        assert (db.double() - grads[2]).abs().max() <= 1e-4 * grads[2].abs().max()
        # LayerNorm has the mean(w*dy) term by right: the flag changes nothing
        dx2, _, _ = oc.norm_backward(x, dy, w, mean, rstd, kind, ref_compat_c2=True)
        assert torch.equal(dx, dx2)
        return
    # the reference's RMSNorm backward: the true gradient minus mean(w*dy)*rstd per row
    ww = w.double() + (1.0 if kind == "rms_gemma" else 0.0)
    extra = (ww * dy.double()).mean(-1, keepdim=True) * rstd.double()[:, None]
    dx_ref, _, _ = oc.norm_backward(x, dy, w, mean, rstd, kind, ref_compat_c2=True)
    assert (dx_ref.double() - (dx_true - extra)).abs().max() <= tol(dx_true)
    # and that term is not negligible, so the two variants are told apart by this test
    assert extra.abs().max() > 4 * tol(dx_true)
