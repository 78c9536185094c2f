"""The reference's own norm sites, run on the GPU beside this library's fused kernel.

Each case calls the FORWARD of the reference's autograd Function directly (its Triton forward norm
kernel, operators/efficient_rmsnorm.py:15-60 / efficient_rmsnorm_gemma.py / efficient_layernorm.py:15-62,
then its own ``get_statistics`` and eager compress chain on the device) with a stand-in for the autograd
context, and compares what it saved with the output of ``hyc_norm_compress`` given the same threshold
and scale: norm output and statistics within 1e-2 relative (they agree far closer), packed codes and
the outlier set bit-exactly.  Only forward kernels are launched: the reference's backward kernels take
a spin lock without a bound and are never run here.  The reference is imported from its checkout or
from the staged copy (oracle/make_ref.py); without either, or without a working Triton, the cases skip."""
import pytest
import torch

from hyc_lora_b200 import synthetic
from oracle import ref_loader

pytestmark = pytest.mark.gpu


class _Ctx:
    """What the reference's forward needs from an autograd context."""

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors

    def mark_non_differentiable(self, *tensors):
        pass


def _reference_forward(kind, x, w, b, eps, bits, method, ratio):
    ref = ref_loader.load_norms()
    if ref is None:
        pytest.skip("reference operators (or Triton) not available on this machine")
    func = {"rms": lambda: ref.efficient_rmsnorm.EfficientMemoryRMSNormFunc,
            "rms_gemma": lambda: ref.efficient_rmsnorm_gemma.EfficientMemoryRMSNormGemmaFunc,
            "ln": lambda: ref.efficient_layernorm.EfficientMemoryLayerNormFunc}[kind]()
    ctx = _Ctx()
    try:
        y, thr, L, R, scale = func.forward(ctx, x, (x.shape[-1],), ratio, 1.0, bits, method, 0, w, b, eps, 0,
                                           [None, None, None, None])
        torch.cuda.synchronize()
    except AssertionError:
        raise
    except Exception as e:                     # a Triton that cannot compile here is not this library's failure
        pytest.skip(f"the reference's Triton kernel did not run here: {type(e).__name__}: {e}"[:200])
    saved = ctx.saved_tensors
    codes = saved[0]
    mean, rstd = (saved[4], saved[5]) if kind == "ln" else (None, saved[4])
    return y, thr, scale, codes, ctx.x_outlier_compressed, mean, rstd


@pytest.mark.parametrize("kind,shape,dtype,bits,method", [
    ("rms", (2, 64, 4096), torch.bfloat16, 4, "per-channel"),
    ("rms", (2, 64, 4096), torch.bfloat16, 8, "per-token"),
    ("rms", (1, 96, 11008), torch.bfloat16, 2, "per-channel"),
    ("rms_gemma", (2, 64, 1024), torch.bfloat16, 4, "per-tensor"),
    ("ln", (4, 128, 768), torch.float32, 4, "per-token"),
    ("ln", (2, 128, 3072), torch.float32, 4, "per-channel"),
])
def test_norm_site_forward_matches_the_reference_on_the_device(kind, shape, dtype, bits, method):
    from hyc_lora_b200 import packed as pk
    b, s, d = shape
    x, _ = synthetic.roundtrip_activation(b, s, d, planted=max(4, d // 100), gain=20.0, dtype=dtype, salt=d + bits)
    g = torch.Generator().manual_seed(d)
    w = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    bias = (0.05 * torch.randn(d, generator=g)).to(dtype) if kind == "ln" else None
    xd, wd, bd = x.cuda(), w.cuda(), None if bias is None else bias.cuda()
    y_r, thr, scale, codes_r, coo_r, mean_r, rstd_r = _reference_forward(kind, xd, wd, bd, 1e-5, bits, method, 0.01)

    p, y, rstd, mean = pk.compress_r(xd, thr, scale, bits, outlier_ratio=0.01,
                                     norm=dict(kind=kind, weight=wd, bias=bd, eps=1e-5))
    assert int(p.status.item()) == 0
    # norm output and statistics: floating point, different summation order
    assert ((y.float() - y_r.float()).abs() <= 1e-2 * y_r.float().abs() + 1e-3).all()
    assert torch.allclose(rstd, rstd_r, rtol=1e-4, atol=0)
    if kind == "ln":
        assert torch.allclose(mean, mean_r, rtol=1e-3, atol=1e-5)
    # packed codes and the outlier set: bit-exact
    assert torch.equal(p.codes.reshape(codes_r.shape).view(torch.uint8), codes_r.view(torch.uint8))
    coo = coo_r.coalesce()
    idx = coo.indices().cpu()
    want_flat = idx[0] * (s * d) + idx[1] * d + idx[2]
    order = torch.argsort(want_flat)
    flat, val = p.outlier_coo()
    assert torch.equal(flat, want_flat[order])
    assert torch.equal(val.view(torch.int16), coo.values().cpu()[order].to(torch.bfloat16).view(torch.int16))
