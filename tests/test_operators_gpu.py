"""GPU tests of the drop-in operator modules: forward + backward of every
``EfficientMemory*`` module against the CPU oracle (reference arithmetic) and, in
channel mode, against the oracle's channel-mode functions."""
import pytest
import torch

from hyc_lora_b200 import synthetic
from oracle import hyc_oracle as oc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.float().cpu().flatten(), b.float().cpu().flatten(), dim=0).item()


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-20)).item()


def _act(b=3, s=37, d=768, dtype=torch.bfloat16, salt=0, gain=20.0):
    return synthetic.roundtrip_activation(b, s, d, planted=5, gain=gain, dtype=dtype, salt=salt)[0]


def _rand(shape, seed, dtype=torch.bfloat16):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)).to(dtype)


def _oracle_xhat(x, bits, method, ratio=0.01):
    thr, L, R, scale = oc.r_calibrate(x, ratio, 1.0, bits, method, 0)
    return oc.r_decompress(oc.r_compress(x, thr, scale, bits, 1.0)), thr, scale


# ------------------------------------------------------------------ reference mode

@pytest.mark.parametrize("dtype,bits,method", [(torch.bfloat16, 4, "per-channel"), (torch.float32, 4, "per-token"),
                                               (torch.bfloat16, 8, "per-tensor"), (torch.bfloat16, 2, "per-token")])
def test_linear_matches_reference_arithmetic(dtype, bits, method):
    from hyc_lora_b200.operators.efficient_linear import EfficientMemoryLinear
    x = _act(dtype=dtype, salt=bits)
    a = (0.02 * _rand((16, 768), 1, torch.float32)).to(dtype)
    g = _rand((3, 37, 16), 2, dtype)
    m = EfficientMemoryLinear(768, 16, bias=False, outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=bits,
                              sub_outlier_quantize_method=method, rank=0).to(DEV).to(dtype)
    m.weight.data.copy_(a)
    xd = x.to(DEV).requires_grad_(True)
    out = m(xd)
    out.backward(g.to(DEV))
    xh, thr, scale = _oracle_xhat(x, bits, method)
    assert torch.equal(m.static_value[0].cpu(), thr) and torch.equal(m.static_value[2].cpu(), scale)
    dx_o, dw_o = oc.linear_backward(xh, a, g)
    assert _rel(out, x @ a.T) < 2e-2
    assert _rel(xd.grad, dx_o) < 2e-2 and _cos(xd.grad, dx_o) > 0.9999
    assert _cos(m.weight.grad, dw_o) > 0.9995 and _rel(m.weight.grad, dw_o) < 2e-2


def test_calibration_protocol_running_mean_then_frozen():
    from hyc_lora_b200.operators.efficient_silu import EfficientMemorySiLU
    m = EfficientMemorySiLU(outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=8,
                            sub_outlier_quantize_method="per-channel", rank=0)
    xs = [_act(salt=10 + i, gain=5.0) for i in range(4)]
    stats = [oc.r_calibrate(x, 0.01, 1.0, 8, "per-channel", 0) for x in xs]
    for i, x in enumerate(xs):
        m(x.to(DEV))
        if i == 0:
            assert torch.equal(m.static_value[0].cpu(), stats[0][0])
        if i == 1:
            want_thr = (1 * stats[0][0] + stats[1][0]) / 2
            want_scale = (1 * stats[0][3] + stats[1][3]) / 2
            assert torch.equal(m.static_value[0].cpu(), want_thr)
            assert torch.equal(m.static_value[2].cpu(), want_scale)
            frozen = [None if t is None else t.clone() for t in m.static_value]
    assert m.iteration == 4
    for a, b in zip(m.static_value, frozen):
        assert torch.equal(a, b)


@pytest.mark.parametrize("kind,dtype,d", [("rms", torch.bfloat16, 4096), ("ln", torch.float32, 768),
                                          ("rms_gemma", torch.bfloat16, 1024)])
def test_norm_modules(kind, dtype, d):
    from hyc_lora_b200.operators.efficient_layernorm import EfficientMemoryLayerNorm
    from hyc_lora_b200.operators.efficient_rmsnorm import EfficientMemoryRMSNorm
    from hyc_lora_b200.operators.efficient_rmsnorm_gemma import EfficientMemoryRMSNormGemma
    cls = {"rms": EfficientMemoryRMSNorm, "ln": EfficientMemoryLayerNorm, "rms_gemma": EfficientMemoryRMSNormGemma}[kind]
    x = _act(2, 41, d, dtype=dtype, salt=d)
    m = cls(d, eps=1e-5, outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=4,
            sub_outlier_quantize_method="per-channel", rank=0).to(DEV)
    w = synthetic.norm_weight(d, 0.1, dtype=torch.float32)
    bvec = 0.05 * _rand((d,), 3, torch.float32)
    m.weight.data.copy_(w)
    m.bias.data.copy_(bvec)
    xd = x.to(DEV).requires_grad_(True)
    y = m(xd)
    dy = _rand(x.shape, 4, dtype)
    y.backward(dy.to(DEV))
    y_o, mean_o, rstd_o = oc.norm_forward(x, w, bvec, 1e-5, kind)
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-4
    assert y.dtype == x.dtype and ((y.float().cpu() - y_o.float()).abs() <= tol * y_o.float().abs() + 1e-3).all()
    xh, _, _ = _oracle_xhat(x, 4, "per-channel")
    dx_o, dw_o, _ = oc.norm_backward(xh, dy, w, mean_o, rstd_o, kind, ref_compat_c2=True)
    assert xd.grad.dtype == x.dtype
    assert _rel(xd.grad, dx_o) < 1e-2 and _cos(xd.grad, dx_o) > 0.9999
    assert _cos(m.weight.grad, dw_o) > 0.9999 and _rel(m.weight.grad, dw_o) < 1e-2
    assert m.bias.grad is None                      # the reference returns no bias gradient


def test_norm_with_frozen_weight_skips_weight_gradient():
    from hyc_lora_b200.operators.efficient_rmsnorm import EfficientMemoryRMSNorm
    m = EfficientMemoryRMSNorm(1024, sub_outlier_ratio=1.0, sub_outlier_bit=8, rank=0).to(DEV)
    m.weight.requires_grad_(False)
    x = _act(2, 16, 1024, salt=3).to(DEV).requires_grad_(True)
    m(x).sum().backward()
    assert m.weight.grad is None and x.grad is not None


@pytest.mark.parametrize("op", ["silu", "gelu"])
def test_activation_modules(op):
    from hyc_lora_b200.operators.efficient_gelu import EfficientMemoryGELU
    from hyc_lora_b200.operators.efficient_silu import EfficientMemorySiLU
    cls = EfficientMemorySiLU if op == "silu" else EfficientMemoryGELU
    x = _act(2, 19, 3072, salt=5, gain=4.0)
    m = cls(outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=8, sub_outlier_quantize_method="per-channel",
            rank=0)
    xd = x.to(DEV).requires_grad_(True)
    y = m(xd)
    g = _rand(x.shape, 6)
    y.backward(g.to(DEV))
    ref_y = torch.nn.functional.silu(x.float()) if op == "silu" else torch.nn.functional.gelu(x.float())
    assert _rel(y, ref_y) < 1e-2
    xh, _, _ = _oracle_xhat(x, 8, "per-channel")
    o = (oc.silu_backward if op == "silu" else oc.gelu_backward)(xh, g)
    assert ((xd.grad.float().cpu() - o.float()).abs() <= 1e-2 * o.float().abs() + 1e-4).all()


def test_product_module_and_mixed_formats():
    from hyc_lora_b200.operators.efficient_hadamard import EfficientMemoryHadamard
    x1, x2 = _act(2, 19, 1024, salt=7, gain=4.0), _act(2, 19, 1024, salt=8, gain=4.0)
    g = _rand(x1.shape, 9)
    for b1, b2 in ((4, 4), (8, 4)):
        m = EfficientMemoryHadamard(0.01, 1.0, b1, "per-token", 0.01, 1.0, b2, "per-token", rank=0)
        a1, a2 = x1.to(DEV).requires_grad_(True), x2.to(DEV).requires_grad_(True)
        m(a1, a2).backward(g.to(DEV))
        xh1, _, _ = _oracle_xhat(x1, b1, "per-token")
        xh2, _, _ = _oracle_xhat(x2, b2, "per-token")
        d1, d2 = oc.product_backward(xh1, xh2, g)
        assert torch.equal(a1.grad.cpu(), d1) and torch.equal(a2.grad.cpu(), d2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_module(dtype):
    from hyc_lora_b200.operators.efficient_softmax import EfficientMemorySoftmax
    x = (3.0 * _rand((2, 12, 40, 40), 11, torch.float32)).to(dtype)
    g = _rand(x.shape, 12, dtype)
    m = EfficientMemorySoftmax(outlier_ratio=0.05)
    xd = x.to(DEV).requires_grad_(True)
    y = m(xd)
    y.backward(g.to(DEV))
    y_gpu = y.detach().cpu()
    thr = oc.r_softmax_threshold(y_gpu, 0.05)
    assert torch.equal(m.static_value.cpu(), thr)
    kept = oc.r_softmax_keep(y_gpu, thr)
    want = oc.softmax_backward(kept.float(), g.float())
    assert xd.grad.dtype == dtype
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(xd.grad.float().cpu(), want, rtol=tol, atol=tol * want.abs().max().item())


def test_sparse_rows_roundtrip_and_overflow():
    from hyc_lora_b200 import packed
    y = torch.softmax(3.0 * _rand((4, 6, 33, 50), 13, torch.float32), dim=-1).to(DEV)
    thr = torch.tensor(0.05)
    s = packed.softmax_compact(y, thr.to(DEV), capacity_ratio=0.5)
    assert torch.equal(packed.softmax_expand(s).cpu(), oc.r_softmax_keep(y.cpu(), thr))
    assert not s.overflowed()
    tiny = packed.softmax_compact(y, thr.to(DEV), capacity_ratio=0.0)   # floor of 1/64 of the tensor
    dense = packed.softmax_expand(tiny).cpu()
    assert tiny.overflowed()
    full = oc.r_softmax_keep(y.cpu(), thr)
    rows_kept = dense.reshape(-1, 50).abs().sum(dim=1) > 0
    assert torch.equal(dense.reshape(-1, 50)[rows_kept], full.reshape(-1, 50)[rows_kept])


def test_attention_gemm_modules():
    from hyc_lora_b200.operators.efficient_gemm import EfficientMemoryGEMM, EfficientMemoryGEMMWithSoftmax
    b, h, s, hd = 2, 12, 24, 64
    q = _act(b, s, h * hd, salt=21, gain=6.0).reshape(b, s, h, hd).permute(0, 2, 1, 3)
    kmat = _act(b, s, h * hd, salt=22, gain=6.0).reshape(b, s, h, hd).permute(0, 2, 1, 3)
    v = _act(b, s, h * hd, salt=23, gain=6.0).reshape(b, s, h, hd).permute(0, 2, 1, 3)
    g1 = _rand((b, h, s, s), 24)
    gemm1 = EfficientMemoryGEMM(0.01, 1.0, 4, "per-channel", 0.01, 1.0, 4, "per-channel", rank=0)
    qd, kd = q.to(DEV).requires_grad_(True), kmat.to(DEV).transpose(-1, -2).requires_grad_(True)
    out = gemm1(qd, kd)
    out.backward(g1.to(DEV))
    qh, _, _ = _oracle_xhat(oc.heads_to_rows(q), 4, "per-channel")
    kh, _, _ = _oracle_xhat(oc.heads_to_rows(kmat), 4, "per-channel")
    qh, kh = oc.rows_to_heads(qh, h), oc.rows_to_heads(kh, h)
    want_q = g1.float() @ kh.float()
    want_kT = (qh.float().transpose(-1, -2) @ g1.float())
    assert _rel(qd.grad, want_q) < 2e-2 and _cos(qd.grad, want_q) > 0.9995
    assert _rel(kd.grad, want_kT) < 2e-2 and _cos(kd.grad, want_kT) > 0.9995
    # P @ V with the thresholded probabilities
    pmat = torch.softmax(_rand((b, h, s, s), 25, torch.float32), dim=-1).to(torch.bfloat16)
    g2 = _rand((b, h, s, hd), 26)
    gemm2 = EfficientMemoryGEMMWithSoftmax(0.05, 0.01, 1.0, 4, "per-channel", rank=0)
    pd, vd = pmat.to(DEV).requires_grad_(True), v.to(DEV).requires_grad_(True)
    gemm2(pd, vd).backward(g2.to(DEV))
    vh, _, _ = _oracle_xhat(oc.heads_to_rows(v), 4, "per-channel")
    vh = oc.rows_to_heads(vh, h)
    kept = oc.r_softmax_keep(pmat, oc.r_softmax_threshold(pmat, 0.05))
    want_p = g2.float() @ vh.float().transpose(-1, -2)
    want_v = kept.float().transpose(-1, -2) @ g2.float()
    assert _rel(pd.grad, want_p) < 2e-2 and _rel(vd.grad, want_v) < 2e-2


def test_dropout_module_is_identity_at_p0_and_regenerates_its_mask():
    from hyc_lora_b200.operators.efficient_dropout import EfficientMemoryDropout
    x = _rand((4, 256), 30).to(DEV).requires_grad_(True)
    m0 = EfficientMemoryDropout(0.0)
    assert torch.equal(m0(x), x)
    m = EfficientMemoryDropout(0.5).train()
    y = m(x)
    y.sum().backward()
    kept = y != 0
    assert 0.3 < kept.float().mean().item() < 0.7
    assert torch.equal(x.grad != 0, kept)


# ------------------------------------------------------------------ channel mode

def test_channel_mode_modules_match_oracle():
    from hyc_lora_b200.operators.efficient_linear import EfficientMemoryLinear
    from hyc_lora_b200.operators.efficient_rmsnorm import EfficientMemoryRMSNorm
    from hyc_lora_b200.operators.efficient_silu import EfficientMemorySiLU
    d, r = 4096, 64
    x = _act(2, 33, d, salt=40, gain=30.0)
    ch = oc.n_select_channels(oc.n_channel_scores(x), oc.n_outlier_count(d, 0.01))
    c = oc.n_compress(x.reshape(-1, d), ch, 4, 0, 256)
    xh = oc.n_decompress(c).reshape(x.shape)
    # linear
    a = (0.02 * _rand((r, d), 41, torch.float32)).to(torch.bfloat16)
    g = _rand((2, 33, r), 42)
    lin = EfficientMemoryLinear(d, r, bias=False, outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=4,
                                rank=0, outlier_mode="channel", rotate=256).to(DEV).to(torch.bfloat16)
    lin.weight.data.copy_(a)
    xd = x.to(DEV).requires_grad_(True)
    lin(xd).backward(g.to(DEV))
    _, dw_o = oc.linear_backward(xh, a, g)
    assert _cos(lin.weight.grad, dw_o) > 0.9995
    assert torch.equal(lin.site.calib.channels.cpu(), ch)
    # rmsnorm (true RMSNorm gradient this time)
    norm = EfficientMemoryRMSNorm(d, eps=1e-5, outlier_ratio=0.01, sub_outlier_bit=4, rank=0, outlier_mode="channel",
                                  rotate=256, ref_compat_c2=False).to(DEV)
    xd = x.to(DEV).requires_grad_(True)
    dy = _rand(x.shape, 43)
    y = norm(xd)
    y.backward(dy.to(DEV))
    w = torch.ones(d)
    y_o, _, rstd_o = oc.norm_forward(x, w, None, 1e-5, "rms")
    dx_o, _, _ = oc.norm_backward(xh, dy, w, None, rstd_o, "rms", ref_compat_c2=False)
    assert ((y.float().cpu() - y_o.float()).abs() <= 1e-2 * y_o.float().abs() + 1e-3).all()
    assert _rel(xd.grad, dx_o) < 1e-2
    # and against the exact (uncompressed) gradient: the compression error stays small
    xe = x.float().requires_grad_(True)
    (xe * torch.rsqrt(xe.pow(2).mean(-1, keepdim=True) + 1e-5)).backward(dy.float())
    assert _cos(xd.grad, xe.grad) > 0.99
    # silu
    act = EfficientMemorySiLU(outlier_ratio=0.01, sub_outlier_bit=4, rank=0, outlier_mode="channel", rotate=256)
    xd = x.to(DEV).requires_grad_(True)
    act(xd).backward(dy.to(DEV))
    o = oc.silu_backward(xh, dy)
    assert ((xd.grad.float().cpu() - o.float()).abs() <= 1e-2 * o.float().abs() + 1e-4).all()


def test_channel_mode_wide_site_uses_fitting_rotation_block():
    """11 008 channels at 4 bits: segments of 5 504 channels do not start on 256-block boundaries, so the
    site rotates in blocks of 64; the result is the oracle's for that block size."""
    from hyc_lora_b200.operators.efficient_silu import EfficientMemorySiLU
    d = 11008
    x = _act(2, 19, d, salt=60, gain=30.0)
    dy = _rand(x.shape, 61)
    ch = oc.n_select_channels(oc.n_channel_scores(x), oc.n_outlier_count(d, 0.01))
    act = EfficientMemorySiLU(outlier_ratio=0.01, sub_outlier_bit=4, rank=0, outlier_mode="channel", rotate=256)
    assert act.site.rotate_for(d, 4) == 64
    xd = x.to(DEV).requires_grad_(True)
    act(xd).backward(dy.to(DEV))
    xh = oc.n_decompress(oc.n_compress(x.reshape(-1, d), ch, 4, 0, 64)).reshape(x.shape)
    o = oc.silu_backward(xh, dy)
    assert ((xd.grad.float().cpu() - o.float()).abs() <= 1e-2 * o.float().abs() + 1e-4).all()


def test_sites_saving_the_same_tensor_share_one_record():
    """Three LoRA-A style linears fed the same tensor object compress it once (per call) and get the
    gradients they get when every site compresses for itself."""
    from hyc_lora_b200.operators import _common, compress_function as cf
    from hyc_lora_b200.operators.efficient_linear import EfficientMemoryLinear
    d, r = 1024, 16
    x = _act(2, 40, d, salt=70, gain=20.0)
    g = [_rand((2, 40, r), 71 + i) for i in range(3)]
    ws = [(0.02 * _rand((r, d), 75 + i, torch.float32)).to(torch.bfloat16) for i in range(3)]
    grads = {}
    for share in (True, False):
        _common.SHARE_SITES = share
        _common._shared.clear()
        lins = []
        for w in ws:
            lin = EfficientMemoryLinear(d, r, bias=False, outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=4,
                                        rank=0, outlier_mode="channel", rotate=64).to(DEV).to(torch.bfloat16)
            lin.weight.data.copy_(w)
            lins.append(lin)
        calls, real = [0], cf.channel_compress
        def counted(*a, **k):
            calls[0] += 1
            return real(*a, **k)
        cf.channel_compress = counted
        try:
            for it in range(3):                      # two calibration calls, one steady-state call
                for lin in lins:
                    lin.weight.grad = None
                xd = x.to(DEV).requires_grad_(True)
                sum((lin(xd) * gi.to(DEV)).sum() for lin, gi in zip(lins, g)).backward()
        finally:
            cf.channel_compress = real
        assert calls[0] == (3 if share else 9)
        grads[share] = [lin.weight.grad.clone() for lin in lins] + [xd.grad.clone()]
    _common.SHARE_SITES = True
    for a, b in zip(grads[True], grads[False]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("kind,rotate", [("rms", 0), ("ln", 0), ("rms", 256)])
def test_norm_emits_the_record_of_its_output_for_the_sites_behind_it(kind, rotate):
    """A norm followed by three LoRA-A style linears (the q/k/v arrangement), all in channel mode
    with and without rotation: from the first steady-state call on, one launch makes both the record of the
    norm input and the record the three linears save, and every gradient is what it is when each
    site compresses for itself."""
    from hyc_lora_b200 import _lib
    from hyc_lora_b200.operators import _common, compress_function as cf
    from hyc_lora_b200.operators.efficient_layernorm import EfficientMemoryLayerNorm
    from hyc_lora_b200.operators.efficient_linear import EfficientMemoryLinear
    from hyc_lora_b200.operators.efficient_rmsnorm import EfficientMemoryRMSNorm
    d, r = 1024, 16
    x = _act(2, 40, d, salt=80, gain=20.0)
    g = [_rand((2, 40, r), 81 + i) for i in range(3)]
    ws = [(0.02 * _rand((r, d), 85 + i, torch.float32)).to(torch.bfloat16) for i in range(3)]
    kw = dict(outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=4, rank=0, outlier_mode="channel", rotate=rotate)
    grads, calls = {}, {}
    for share in (True, False):
        _common.SHARE_SITES = share
        _common._shared.clear()
        _common._last_norm_output = None
        norm = (EfficientMemoryRMSNorm(d, bias=False, **kw) if kind == "rms" else EfficientMemoryLayerNorm(d, **kw))
        norm = norm.to(DEV).to(torch.bfloat16)
        norm.weight.data.copy_(1.0 + 0.1 * _rand((d,), 90, torch.float32))
        lins = []
        for w in ws:
            lin = EfficientMemoryLinear(d, r, bias=False, **kw).to(DEV).to(torch.bfloat16)
            lin.weight.data.copy_(w)
            lins.append(lin)
        count, real = [0], cf.channel_compress
        def counted(*a, **k):
            count[0] += 1
            return real(*a, **k)
        cf.channel_compress = counted
        per_call = []
        try:
            for it in range(4):                      # two calibration calls, two steady-state calls
                for m in lins + [norm]:
                    m.weight.grad = None
                xd = x.to(DEV).requires_grad_(True)
                before, l0 = count[0], _lib.lib.hyc_launch_count()
                h = norm(xd)
                out = sum((lin(h) * gi.to(DEV)).sum() for lin, gi in zip(lins, g))
                per_call.append((count[0] - before, _lib.lib.hyc_launch_count() - l0))
                out.backward()
        finally:
            cf.channel_compress = real
        calls[share] = per_call
        grads[share] = [lin.weight.grad.clone() for lin in lins] + [xd.grad.clone(), norm.weight.grad.clone()]
        if share:
            assert norm.site.output_format is not None and norm.site.output_format[3] is lins[0].site.calib
    _common.SHARE_SITES = True
    # compress calls per forward: norm + one shared while calibrating, the norm's alone afterwards; 4 without sharing
    assert [c for c, _ in calls[True]] == [2, 2, 1, 1]
    assert [c for c, _ in calls[False]] == [4, 4, 4, 4]
    # and in launches of the library: the steady-state forward is ONE launch
    assert calls[True][3][1] == 1 and calls[False][3][1] == 4
    for a, b in zip(grads[True], grads[False]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("rotate,act", [(0, "silu"), (64, "silu"), (0, "gelu")])
def test_gated_mlp_sites_make_every_record_in_two_passes(rotate, act):
    """activation -> product -> LoRA-A linear (the gated MLP), channel mode: from the first steady-state call
    on, one launch makes the activation, the record of its input and the record of its output, a second one the
    product, the record of the other operand and the record the linear saves; gradients are what they are
    when every site compresses for itself."""
    from hyc_lora_b200 import _lib
    from hyc_lora_b200.operators import _common
    from hyc_lora_b200.operators.efficient_gelu import EfficientMemoryGELU
    from hyc_lora_b200.operators.efficient_hadamard import EfficientMemoryHadamard
    from hyc_lora_b200.operators.efficient_linear import EfficientMemoryLinear
    from hyc_lora_b200.operators.efficient_silu import EfficientMemorySiLU
    d, r = 1024, 16
    gate = 0.2 * _act(2, 40, d, salt=90, gain=20.0)
    up = _act(2, 40, d, salt=91, gain=20.0)
    g = _rand((2, 40, r), 92)
    w = (0.02 * _rand((r, d), 93, torch.float32)).to(torch.bfloat16)
    kw = dict(outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=4, rank=0, outlier_mode="channel", rotate=rotate)
    kw2 = dict(outlier_ratio_1=0.01, sub_outlier_ratio_1=1.0, sub_outlier_bit_1=4, outlier_ratio_2=0.01,
               sub_outlier_ratio_2=1.0, sub_outlier_bit_2=4, rank=0, outlier_mode="channel", rotate=rotate)
    grads, launches = {}, {}
    for share in (True, False):
        _common.SHARE_SITES = share
        _common._shared.clear()
        _common._last_norm_output = None
        fn = (EfficientMemorySiLU if act == "silu" else EfficientMemoryGELU)(**kw)
        prod = EfficientMemoryHadamard(**kw2)
        lin = EfficientMemoryLinear(d, r, bias=False, **kw).to(DEV).to(torch.bfloat16)
        lin.weight.data.copy_(w)
        per_call = []
        for it in range(4):                      # two calibration calls, two steady-state calls
            lin.weight.grad = None
            gd, ud = gate.to(DEV).requires_grad_(True), up.to(DEV).requires_grad_(True)
            l0 = _lib.lib.hyc_launch_count()
            out = lin(prod(fn(gd), ud))
            per_call.append(_lib.lib.hyc_launch_count() - l0)
            (out * g.to(DEV)).sum().backward()
        launches[share] = per_call
        grads[share] = [lin.weight.grad.clone(), gd.grad.clone(), ud.grad.clone(), out.detach().clone()]
    _common.SHARE_SITES = True
    # steady state: activation + product with sharing; without it the activation's output and the product are
    # compressed again by the sites that save them
    assert launches[True][3] == 2 and launches[False][3] == 4
    for a, b in zip(grads[True], grads[False]):
        assert torch.equal(a, b)
    # the forward value against torch's own activation and product (bf16, one unit in the last place)
    ref = torch.nn.functional.linear((torch.nn.functional.silu if act == "silu" else torch.nn.functional.gelu)(gate.to(DEV))
                                     * up.to(DEV), w.to(DEV))
    assert _cos(grads[True][3], ref) > 0.9999


def test_low_rank_site_and_calibration_state_roundtrip():
    """rank > 0: the randomized SVD differs between devices, so the check is against the exact
    derivative; then a second module restored from the first one's calibration state reproduces
    its steady-state result bit for bit."""
    from hyc_lora_b200.operators._common import calibration_state_dict, load_calibration_state_dict
    from hyc_lora_b200.operators.efficient_silu import EfficientMemorySiLU
    kw = dict(outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=8, sub_outlier_quantize_method="per-channel",
              rank=2)
    m = EfficientMemorySiLU(**kw)
    x = _act(2, 32, 1024, salt=50, gain=4.0)
    g = _rand(x.shape, 51)
    for _ in range(3):
        xd = x.to(DEV).requires_grad_(True)
        m(xd).backward(g.to(DEV))
    xe = x.float().requires_grad_(True)
    torch.nn.functional.silu(xe).backward(g.float())
    assert _cos(xd.grad, xe.grad) > 0.999
    assert m.static_value[1].shape == (32, 2) and m.static_value[3].shape == (2, 1024)
    m2 = EfficientMemorySiLU(**kw)
    load_calibration_state_dict(m2, calibration_state_dict(m))
    assert m2.iteration == 3
    x2 = x.to(DEV).requires_grad_(True)
    m2(x2).backward(g.to(DEV))
    x3 = x.to(DEV).requires_grad_(True)
    m(x3).backward(g.to(DEV))
    assert torch.equal(x2.grad, x3.grad)


@pytest.mark.parametrize("extra", [{}, dict(outlier_mode="channel")])
def test_config1_adapter_with_zero_b_gives_zero_da_and_the_oracles_db(extra):
    """Configuration 1, check (ii): the full adapter ``base(x) + B(A(x)) * s`` with ``B = 0`` and an
    upstream gradient G ~ N(0,1) on its output.  The chain rule gives dA = s * (G B)^T X = 0 exactly
    (the weight-gradient kernel contracts an all-zero gradient with the packed input) and
    dB = s * G^T (A x), which does not depend on the compressed copy at all."""
    from hyc_lora_b200.hosts.lora import LoRALinear
    from hyc_lora_b200.hosts.replace import replace_module, uniform_config
    x, _ = synthetic.roundtrip_activation()
    a, _ = synthetic.lora_a_problem()
    g = _rand((8, 128, 768), 9, torch.float32)
    m = LoRALinear(768, 768, r=16, alpha=16.0, quant="bf16", device=DEV, dtype=torch.float32)
    m.base_layer.weight.data = m.base_layer.weight.data.float()
    m.lora_A.weight.data.copy_(a)
    assert replace_module(m, uniform_config(sub_outlier_bit=4, sub_outlier_quantize_method="per-token"), extra) == 1
    assert float(m.lora_B.weight.detach().abs().max()) == 0.0
    for _ in range(3):                                   # two calibration calls, then the steady state
        m.zero_grad(set_to_none=True)
        xd = x.to(DEV).requires_grad_(True)
        m(xd).backward(g.to(DEV))
    da, db = m.lora_A.weight.grad, m.lora_B.weight.grad
    assert da is not None and float(da.abs().max()) == 0.0
    db_o = m.scaling * torch.einsum("bso,bsr->or", g, x @ a.T)
    assert _cos(db, db_o) > 0.99999 and _rel(db, db_o) < 1e-3
    # dX has no adapter share either: it is the frozen base's alone
    assert _rel(xd.grad, g @ m.base_layer.weight.detach().cpu().float()) < 1e-3
