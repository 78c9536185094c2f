"""Pin the CPU oracle against the reference's own code, imported in place.

Skipped where the reference tree is absent; the committed fixtures under
tests/golden/ (made from the same imported code) carry the pin there."""
import itertools

import pytest
import torch

from oracle import hyc_oracle as oc
from oracle import ref_loader

ref = ref_loader.load()
pytestmark = pytest.mark.skipif(ref is None, reason="reference tree not present")


def _x(dtype, shape=(3, 32, 256), seed=0, gain=20.0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g)
    idx = torch.randperm(shape[-1], generator=g)[:4]
    x[..., idx] *= gain
    return x.to(dtype)


def _coo_equal(coo, c):
    coo = coo.coalesce()
    assert torch.equal(coo.indices(), c.out_index)
    assert torch.equal(coo.values(), c.out_value)


@pytest.mark.parametrize("dtype,bits,method,rank", list(itertools.product(
    [torch.bfloat16, torch.float32], [1, 2, 4, 8], ["per-tensor", "per-channel", "per-token"], [0, 2])))
def test_calibrate_compress_decompress_match_reference(dtype, bits, method, rank):
    cf = ref.compress_function
    x = _x(dtype, seed=bits * 10 + rank)
    with ref_loader.cpu_cuda_noop():
        torch.manual_seed(123)
        thr_r, L_r, R_r, sc_r = cf.get_statistics(x, 0, 0.01, 1.0, bits, method, rank)
        thr, L, R, sc = oc.r_calibrate(x, 0.01, 1.0, bits, method, rank, svd_seed=123)
        assert torch.equal(thr_r, thr) and torch.equal(L_r, L) and torch.equal(R_r, R)
        assert torch.equal(sc_r, sc) and sc.dtype == torch.bfloat16
        o_r, c_r, s_r = cf.true_divide_outlier_suboutlier_svd_compress(x, thr_r, sc_r, bits, 1.0, L_r, R_r)
        c = oc.r_compress(x, thr, sc, bits, 1.0, L, R)
        _coo_equal(o_r, c)
        assert c_r.dtype == c.codes.dtype and torch.equal(c_r, c.codes)
        xh_r = cf.true_divide_outlier_suboutlier_svd_decompress(o_r, c_r, bits, s_r, L=L_r, R=R_r)
        xh = oc.r_decompress(c, L, R)
        assert xh.dtype == torch.bfloat16 and torch.equal(xh_r, xh)


def test_head_layout_matches_reference():
    cf = ref.compress_function
    x = _x(torch.bfloat16, shape=(2, 4, 16, 64), seed=5)
    with ref_loader.cpu_cuda_noop():
        thr, L, R, sc = oc.r_calibrate(x, 0.02, 1.0, 4, "per-channel", 0)
        thr_r, L_r, R_r, sc_r = cf.get_statistics(x, 0, 0.02, 1.0, 4, "per-channel", 0)
        assert torch.equal(thr, thr_r) and torch.equal(sc, sc_r)
        o_r, c_r, s_r = cf.true_divide_outlier_suboutlier_svd_compress(x, thr, sc, 4, 1.0, L, R)
        c = oc.r_compress(x, thr, sc, 4, 1.0, L, R)
        _coo_equal(o_r, c)
        assert torch.equal(c_r, c.codes)
        xh_r = cf.true_divide_outlier_suboutlier_svd_decompress(o_r, c_r, 4, s_r, True, 4, L=L, R=R)
        assert torch.equal(xh_r, oc.r_decompress(c, L, R, num_heads=4))


def test_softmax_sparse_matches_reference():
    cf = ref.compress_function
    y = torch.softmax(_x(torch.float32, shape=(2, 3, 16, 16), seed=9, gain=3.0), dim=-1)
    thr_r = cf.get_statistics_softmax(y, 0, 0.05)
    thr = oc.r_softmax_threshold(y, 0.05)
    assert torch.equal(thr_r, thr)
    kept_r = cf.true_decompress_softmax(cf.true_compress_softmax(y, thr_r))
    assert torch.equal(kept_r, oc.r_softmax_keep(y, thr))


def _ref_fn_grads(fn_cls, args, grad_idx, g):
    ins = [a.clone().requires_grad_(True) if i in grad_idx else a for i, a in enumerate(args)]
    with ref_loader.cpu_cuda_noop():
        out = fn_cls.apply(*ins)
        out[0].backward(g)
    return out, [ins[i].grad for i in grad_idx]


@pytest.mark.parametrize("op", ["silu", "gelu"])
def test_activation_backward_matches_reference(op):
    x = _x(torch.bfloat16, seed=11, gain=5.0)
    g = torch.randn(x.shape, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    cls = ref.efficient_silu.EfficientMemorySiLUFunc if op == "silu" else ref.efficient_gelu.EfficientMemoryGELUFunc
    out, (dx_r,) = _ref_fn_grads(cls, [x, 0.01, 1.0, 8, "per-channel", 0, 0, [None] * 4], [0], g)
    thr, L, R, sc = oc.r_calibrate(x, 0.01, 1.0, 8, "per-channel", 0)
    xh = oc.r_decompress(oc.r_compress(x, thr, sc, 8, 1.0, L, R), L, R)
    dx = (oc.silu_backward if op == "silu" else oc.gelu_backward)(xh, g)
    # the reference evaluates the formula in bf16 op by op; the oracle in fp32
    assert dx.dtype == dx_r.dtype
    assert torch.nn.functional.cosine_similarity(dx.float().flatten(), dx_r.float().flatten(), dim=0) > 0.9999
    assert (dx.float() - dx_r.float()).abs().max() <= 0.05 * dx_r.float().abs().max()


def test_product_backward_matches_reference():
    x1 = _x(torch.bfloat16, seed=21, gain=5.0)
    x2 = _x(torch.bfloat16, seed=22, gain=5.0)
    g = torch.randn(x1.shape, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    cls = ref.efficient_hadamard.EfficientMemoryHadamardFunc
    out, (d1_r, d2_r) = _ref_fn_grads(cls, [x1, x2, 0.01, 1.0, 4, "per-token", 0.01, 1.0, 4, "per-token", 0, 0,
                                            [None] * 4, [None] * 4], [0, 1], g)
    hats = []
    for x in (x1, x2):
        thr, L, R, sc = oc.r_calibrate(x, 0.01, 1.0, 4, "per-token", 0)
        hats.append(oc.r_decompress(oc.r_compress(x, thr, sc, 4, 1.0, L, R), L, R))
    d1, d2 = oc.product_backward(hats[0], hats[1], g)
    assert torch.equal(d1, d1_r) and torch.equal(d2, d2_r)


def test_linear_backward_matches_reference():
    x = _x(torch.bfloat16, seed=31)
    g0 = torch.Generator().manual_seed(6)
    w = (0.02 * torch.randn(16, x.shape[-1], generator=g0)).to(torch.bfloat16)
    g = torch.randn(*x.shape[:2], 16, generator=g0).to(torch.bfloat16)
    cls = ref.efficient_linear.EfficientMemoryLinearFunc
    out, (dx_r, dw_r) = _ref_fn_grads(cls, [x, w, None, False, 0.01, 1.0, 4, "per-channel", 0, 0, [None] * 4], [0, 1], g)
    thr, L, R, sc = oc.r_calibrate(x, 0.01, 1.0, 4, "per-channel", 0)
    xh = oc.r_decompress(oc.r_compress(x, thr, sc, 4, 1.0, L, R), L, R)
    dx, dw = oc.linear_backward(xh, w, g)
    assert torch.equal(dx, dx_r)
    assert torch.allclose(dw.float(), dw_r.float(), rtol=2e-2, atol=2e-2)
    assert torch.nn.functional.cosine_similarity(dw.float().flatten(), dw_r.float().flatten(), dim=0) > 0.9999


def test_softmax_backward_matches_reference():
    x = _x(torch.float32, shape=(2, 3, 16, 16), seed=41, gain=3.0)
    g = torch.randn(x.shape, generator=torch.Generator().manual_seed(8))
    cls = ref.efficient_softmax.EfficientMemorySoftmaxFunc
    out, (dx_r,) = _ref_fn_grads(cls, [x, 0.05, 0, None], [0], g)
    y = torch.softmax(x, dim=-1)
    kept = oc.r_softmax_keep(y, oc.r_softmax_threshold(y, 0.05))
    assert torch.allclose(oc.softmax_backward(kept, g), dx_r, rtol=0, atol=0)
