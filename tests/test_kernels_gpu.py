"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU
oracle and the committed golden fixtures.

Bars: packed codes, outlier indices/values, scales and reconstructions are
compared BIT-EXACTLY; norm outputs and gradients (floating point, different
summation order) within 1e-2 relative of the row scale; weight gradients by
cosine >= 0.999 as well."""
import itertools

import pytest
import torch

from hyc_lora_b200 import synthetic
from oracle import hyc_oracle as oc
from tests import golden_io

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def pk():
    from hyc_lora_b200 import packed
    return packed


def _rel_err(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-20)).item()


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.float().cpu().flatten(), b.float().cpu().flatten(), dim=0).item()


def _lowrank(case):
    if not case.rank:
        return None
    return (oc.fit_rows(case.L, case.x.shape[-2]) @ case.R).to(torch.bfloat16)


def _oracle_coo_flat(c: oc.RCompressed):
    b, s, d = c.shape
    return c.out_index[0] * (s * d) + c.out_index[1] * d + c.out_index[2], c.out_value


# ------------------------------------------------------------------ reference mode vs golden fixtures

@pytest.mark.parametrize("case", list(golden_io.small_cases()), ids=lambda c: c.name)
def test_r_mode_small_fixture(pk, case):
    lr = _lowrank(case)
    p = pk.compress_r(case.x.to(DEV), case.thr.to(DEV), case.scale.to(DEV), case.bits,
                      lowrank=None if lr is None else lr.to(DEV), outlier_ratio=0.02)
    codes = p.codes.cpu().reshape(case.codes.shape)
    assert torch.equal(codes.view(torch.uint8), case.codes.view(torch.uint8))
    flat, val = p.outlier_coo()
    b, s, d = case.x.shape
    gold_flat = case.coo_index[0] * (s * d) + case.coo_index[1] * d + case.coo_index[2]
    assert torch.equal(flat, gold_flat)
    assert torch.equal(val.view(torch.int16), case.coo_value.view(torch.int16))
    xh = pk.decompress(p).cpu()
    assert torch.equal(xh, case.xhat)
    assert not p.overflowed() and not p.wait_expired()


def test_config1_layernorm_compress_roundtrip_and_lora_grads(pk):
    g = golden_io.config1()
    x, _ = synthetic.roundtrip_activation()
    a, grad = synthetic.lora_a_problem()
    w, b = torch.ones(768), torch.zeros(768)
    p, y, rstd, mean = pk.compress_r(x.to(DEV), g.thr.to(DEV), g.scale.to(DEV), 4, outlier_ratio=0.01,
                                     norm=dict(kind="ln", weight=w.to(DEV), bias=b.to(DEV), eps=1e-5))
    y_o, mean_o, rstd_o = oc.norm_forward(x, w, b, 1e-5, "ln")
    assert _rel_err(y, y_o) < 1e-4 and _rel_err(mean, mean_o) < 1e-4 and _rel_err(rstd, rstd_o) < 1e-5
    assert torch.equal(p.codes.cpu().reshape(g.codes.shape), g.codes)
    flat, val = p.outlier_coo()
    assert torch.equal(flat.int(), g.coo_flat) and torch.equal(val, g.coo_value)
    xh = pk.decompress(p)
    assert golden_io.sha_bits(xh.cpu()) == g.xhat_sha256
    # LoRA-A gradients from the reconstructed input (library GEMM on the decompressed rows)
    dx = grad.to(DEV) @ a.to(DEV)
    # the reference casts the upstream gradient to the reconstruction's dtype (bf16) and its
    # batched GEMM returns bf16 (efficient_linear.py:66-67): compare at that precision
    da = torch.einsum("bsr,bsd->rd", grad.to(DEV).bfloat16().float(), xh.float())
    assert _rel_err(dx[0, :8], g.dX0) < 1e-5
    assert _cos(da, g.dA) > 0.9999 and _rel_err(da, g.dA) < 1e-2


@pytest.mark.parametrize("dtype,bits,method", list(itertools.product(
    [torch.bfloat16, torch.float32], [1, 2, 4, 8], ["per-tensor", "per-channel", "per-token"])))
def test_r_mode_against_oracle_ragged_rows(pk, dtype, bits, method):
    # 3*37 = 111 rows: not a multiple of anything; D = 768 is not a power of two
    x, _ = synthetic.roundtrip_activation(3, 37, 768, planted=5, gain=20.0, dtype=dtype, salt=bits)
    thr, L, R, scale = oc.r_calibrate(x, 0.01, 1.0, bits, method, 0)
    c = oc.r_compress(x, thr, scale, bits, 1.0)
    p = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), bits)
    assert torch.equal(p.codes.cpu().reshape(c.codes.shape).view(torch.uint8), c.codes.view(torch.uint8))
    flat, val = p.outlier_coo()
    o_flat, o_val = _oracle_coo_flat(c)
    assert torch.equal(flat, o_flat) and torch.equal(val, o_val)
    assert torch.equal(pk.decompress(p).cpu(), oc.r_decompress(c))


@pytest.mark.parametrize("cols,bits,method", [
    (11008, 4, "per-channel"), (11008, 8, "per-tensor"), (11008, 2, "per-channel"),
    (14336, 4, "per-channel"), (8192, 4, "per-token"), (5120, 4, "per-channel")])
def test_r_mode_wide_rows(pk, cols, bits, method):
    # FFN-wide rows take other thread counts and units per thread (and a helper warp) than 4096 channels
    x, _ = synthetic.roundtrip_activation(2, 150, cols, planted=7, gain=20.0, dtype=torch.bfloat16, salt=cols + bits)
    thr, L, R, scale = oc.r_calibrate(x, 0.01, 1.0, bits, method, 0)
    c = oc.r_compress(x, thr, scale, bits, 1.0)
    p = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), bits)
    assert int(p.status.item()) == 0
    assert torch.equal(p.codes.cpu().reshape(c.codes.shape).view(torch.uint8), c.codes.view(torch.uint8))
    flat, val = p.outlier_coo()
    o_flat, o_val = _oracle_coo_flat(c)
    assert torch.equal(flat, o_flat) and torch.equal(val, o_val)
    assert torch.equal(pk.decompress(p).cpu(), oc.r_decompress(c))


@pytest.mark.parametrize("bits,norm_kind", [(4, None), (8, None), (2, None), (4, "rms")])
def test_r_mode_scales_outside_the_reciprocal_shortcut(pk, bits, norm_kind):
    # channels with a tiny or a huge scale, and infinite inputs: the quotient from the rounded reciprocal is
    # not valid there and the unit is redone with a true division; codes must still match the reference
    x, _ = synthetic.roundtrip_activation(2, 40, 768, planted=5, gain=20.0, dtype=torch.bfloat16, salt=70 + bits)
    x[0, 3, 5] = float("inf")
    x[1, 7, 700] = float("-inf")
    thr, L, R, scale = oc.r_calibrate(x, 0.01, 1.0, bits, "per-channel", 0)
    scale = scale.clone()
    scale.view(-1)[[2, 130, 385]] = 1e-30
    scale.view(-1)[[9, 131, 767]] = 1e30
    scale.view(-1)[[64, 65]] = -0.37          # a negative scale flips the codes
    c = oc.r_compress(x, thr, scale, bits, 1.0)
    if norm_kind is None:
        p = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), bits)
    else:
        w = synthetic.norm_weight(768, 0.1).to(DEV)
        p = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), bits,
                          norm=dict(kind=norm_kind, weight=w, bias=None, eps=1e-5))[0]
    assert int(p.status.item()) == 0
    assert torch.equal(p.codes.cpu().reshape(c.codes.shape).view(torch.uint8), c.codes.view(torch.uint8))
    flat, val = p.outlier_coo()
    o_flat, o_val = _oracle_coo_flat(c)
    assert torch.equal(flat, o_flat) and torch.equal(val, o_val)


def test_r_mode_rows_with_more_outliers_than_the_shared_list(pk):
    """A threshold far inside the distribution gives rows with thousands of element outliers: more than the
    kernel's per-row shared list holds, so warp 0 regenerates the row's entries straight into the pool."""
    x, _ = synthetic.sweep_activation(40, 4096, 0.01, dtype=torch.bfloat16, salt=77)
    x = x.reshape(2, 20, 4096)
    _, _, _, scale = oc.r_calibrate(x, 0.01, 1.0, 4, "per-channel", 0)
    thr = torch.tensor(0.5)
    c = oc.r_compress(x, thr, scale, 4, 1.0)
    assert c.out_index.shape[1] > 40 * 600
    p = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), 4, pool_entries=40 * 4096)
    assert torch.equal(p.codes.cpu().reshape(c.codes.shape).view(torch.uint8), c.codes.view(torch.uint8))
    flat, val = p.outlier_coo()
    o_flat, o_val = _oracle_coo_flat(c)
    assert torch.equal(flat, o_flat) and torch.equal(val, o_val)
    assert torch.equal(pk.decompress(p).cpu(), oc.r_decompress(c))
    assert not p.overflowed() and not p.wait_expired()


@pytest.mark.parametrize("kind,bits,method,rank", [("rms", 4, "per-channel", 4), ("ln", 8, "per-token", 0),
                                                   ("rms", 2, "per-tensor", 0)])
def test_r_mode_fused_norm_many_rows_per_cta(pk, kind, bits, method, rank):
    """Reference mode with the norm fused, low-rank part staged with the row, several rows per CTA."""
    b, seq, d = 24, 128, 1024
    x, _ = synthetic.sweep_activation(b * seq, d, 0.01, dtype=torch.bfloat16, salt=bits + rank)
    x = x.reshape(b, seq, d)
    thr, L, R, scale = oc.r_calibrate(x, 0.01, 1.0, bits, method, rank, 0)
    lr = (oc.fit_rows(L, seq) @ R).to(torch.bfloat16) if rank else None
    w = synthetic.norm_weight(d, 0.1, dtype=torch.bfloat16)
    bias = (0.05 * torch.randn(d, generator=torch.Generator().manual_seed(1))).to(torch.bfloat16)
    c = oc.r_compress(x, thr, scale, bits, 1.0, L if rank else None, R if rank else None)
    p, y, rstd, mean = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), bits,
                                     lowrank=None if lr is None else lr.to(DEV), outlier_ratio=0.02,
                                     norm=dict(kind=kind, weight=w.to(DEV), bias=bias.to(DEV), eps=1e-5))
    assert torch.equal(p.codes.cpu().reshape(c.codes.shape).view(torch.uint8), c.codes.view(torch.uint8))
    flat, val = p.outlier_coo()
    o_flat, o_val = _oracle_coo_flat(c)
    assert torch.equal(flat, o_flat) and torch.equal(val, o_val)
    y_o, mean_o, rstd_o = oc.norm_forward(x, w, bias, 1e-5, kind)
    assert ((y.float().cpu() - y_o.float()).abs() <= 1e-2 * y_o.float().abs() + 1e-3).all()
    assert _rel_err(rstd, rstd_o) < 1e-5
    xh = oc.r_decompress(c, L if rank else None, R if rank else None)
    assert torch.equal(pk.decompress(p).cpu(), xh)
    # consumers on the same packed record
    dy = torch.randn(b, seq, d, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    dx_o, _, _ = oc.norm_backward(xh, dy, w.float(), mean_o, rstd_o, kind)
    dx, _, _ = pk.norm_bwd(p, dy.to(DEV), w.float().to(DEV), rstd_o.to(DEV),
                           None if mean_o is None else mean_o.to(DEV), kind)
    assert _rel_err(dx, dx_o) < 1e-2
    o = oc.silu_backward(xh, dy)
    got = pk.act_bwd("silu", p, dy.to(DEV))
    assert ((got.float().cpu() - o.float()).abs() <= 1e-2 * o.float().abs() + 1e-4).all()
    assert not p.overflowed() and not p.wait_expired()


def test_r_mode_head_layout(pk):
    x, _ = synthetic.roundtrip_activation(2, 24, 768, planted=4, dtype=torch.bfloat16, salt=3)
    heads = x.reshape(2, 24, 12, 64).permute(0, 2, 1, 3)        # [B,H,S,hd] view, as the attention code makes it
    thr, L, R, scale = oc.r_calibrate(heads, 0.02, 1.0, 4, "per-channel", 0)
    c = oc.r_compress(heads, thr, scale, 4, 1.0)
    view = x.to(DEV).reshape(2, 24, 12, 64).permute(0, 2, 1, 3)   # strided head view
    copy = view.contiguous()                                      # really transposed copy
    for h in (view, copy):
        p = pk.compress_r(h, thr.to(DEV), scale.to(DEV), 4, outlier_ratio=0.02)
        assert torch.equal(p.codes.cpu().reshape(c.codes.shape), c.codes)
        out = pk.decompress(p, num_heads=12)
        assert out.shape == (2, 12, 24, 64)
        assert torch.equal(out.cpu(), oc.r_decompress(c, num_heads=12))


def test_r_mode_pool_overflow_degrades_to_quantised_rows(pk):
    x, _ = synthetic.roundtrip_activation(2, 16, 256, planted=4, dtype=torch.bfloat16, salt=9)
    thr, L, R, scale = oc.r_calibrate(x, 0.05, 1.0, 8, "per-channel", 0)
    p = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), 8, pool_entries=7)
    assert p.overflowed()
    meta = p.row_meta.cpu()
    assert int(meta[:, 1].sum()) <= 7
    # rows that lost their pool slot were quantised whole: identical to compressing with thr = +inf
    c_inf = oc.r_compress(x, torch.tensor(float("inf")), scale, 8, 1.0)
    lost = (meta[:, 1] == 0)
    got = p.codes.cpu().reshape(32, 256).view(torch.int8)
    want = c_inf.codes.reshape(32, 256)
    c_thr = oc.r_compress(x, thr, scale, 8, 1.0).codes.reshape(32, 256)
    had_outliers = (c_thr != want).any(dim=1)
    sel = lost & had_outliers
    assert sel.any() and torch.equal(got[sel], want[sel])


# ------------------------------------------------------------------ north-star mode vs oracle

N_CASES = [
    # rows, D, dtype, bits, group, rotate, fraction
    (64, 1024, torch.bfloat16, 4, 0, 0, 0.01),
    (64, 1024, torch.bfloat16, 4, 128, 0, 0.01),
    (37, 768, torch.float32, 4, 0, 0, 0.01),
    (37, 768, torch.float32, 2, 128, 256, 0.02),
    (50, 4096, torch.bfloat16, 2, 0, 256, 0.02),
    (50, 4096, torch.bfloat16, 8, 128, 256, 0.005),
    (50, 4096, torch.bfloat16, 4, 0, 4096, 0.01),
    (33, 4096, torch.bfloat16, 4, 128, 1024, 0.01),
    (33, 1024, torch.bfloat16, 4, 0, 64, 0.01),
    (33, 1024, torch.float32, 8, 128, 16, 0.0),
    (20, 11008, torch.bfloat16, 4, 0, 256, 0.01),
    (20, 14336, torch.bfloat16, 2, 128, 0, 0.02),
    (1, 4096, torch.bfloat16, 4, 0, 0, 0.01),
    (2000, 4096, torch.bfloat16, 4, 0, 256, 0.01),
    # rotation in registers with a half-filled last warp (segments of 384 channels, blocks of 64)
    (37, 768, torch.bfloat16, 4, 0, 64, 0.01),
    (50, 4096, torch.bfloat16, 4, 128, 256, 0.01),
]


@pytest.mark.parametrize("rows,d,dtype,bits,group,rotate,frac", N_CASES)
def test_n_mode_against_oracle(pk, rows, d, dtype, bits, group, rotate, frac):
    x, _ = synthetic.sweep_activation(rows, d, max(frac, 0.005), dtype=dtype, salt=bits + group + rotate)
    k = oc.n_outlier_count(d, frac)
    xd = x.to(DEV)
    score = pk.channel_absmax(xd)
    assert torch.equal(score.cpu(), oc.n_channel_scores(x))
    ch = pk.select_channels(score, k) if k else None
    ch_o = oc.n_select_channels(oc.n_channel_scores(x), k)
    if k:
        assert torch.equal(ch.cpu(), ch_o)
    c = oc.n_compress(x, ch_o, bits, group, rotate)
    p = pk.compress_n(xd, ch, bits, group, rotate)
    assert torch.equal(p.scales.cpu(), c.scales)
    assert torch.equal(p.codes.cpu().view(torch.uint8), c.codes.view(torch.uint8))
    if k:
        assert torch.equal(p.out_value.cpu(), c.out_value)
    xh = pk.decompress(p).cpu().reshape(rows, d)
    assert torch.equal(xh, oc.n_decompress(c))
    assert not p.wait_expired()


def test_n_mode_ties_zero_rows_and_nonfinite_values(pk):
    x = torch.zeros(16, 512, dtype=torch.bfloat16)
    x[3, 5] = 2.0
    x[7, 5] = -2.0
    x[2, 100] = 2.0         # ties with channel 5
    x[2, 101] = 2.0         # ties again: the lower index wins the last place
    x[9, 300] = float("inf")
    x[10, 301] = float("nan")   # NaN never wins a max: the channel scores 0
    xd = x.to(DEV)
    score = pk.channel_absmax(xd)
    assert score.cpu()[301] == 0 and score.cpu()[300] == float("inf")
    ch = pk.select_channels(score, 3)
    assert ch.cpu().tolist() == [5, 100, 300]
    # codes of a row that holds a non-finite value outside the outlier channels are unspecified,
    # but the call must stay inside its buffers (every output is a view into one guarded allocation)
    # and leave every other row exact
    arena = _Arena(1 << 20)
    p = _packed_n_in(arena, pk, 16, 512, 4, 128, 0, ch)
    _compress_into(pk, xd, p)
    torch.cuda.synchronize()
    arena.check()
    xh = pk.decompress(p).cpu().reshape(16, 512)
    rows = [r for r in range(16) if r != 10]
    keep = [c for c in range(512) if c != 101]
    assert torch.equal(xh[rows][:, keep].float(), x[rows][:, keep].float())
    assert xh[2, 101] == 2.0
    assert torch.equal(p.scales.cpu()[0], torch.ones(4))
    assert not p.wait_expired()


# ------------------------------------------------------------------ fused norm forward

@pytest.mark.parametrize("kind,dtype,d,rotate,rows", [
    ("rms", torch.bfloat16, 4096, 0, 45), ("rms_gemma", torch.bfloat16, 1024, 0, 45),
    ("ln", torch.float32, 768, 0, 45), ("ln", torch.bfloat16, 3072, 0, 45),
    ("rms", torch.float32, 768, 0, 45), ("rms", torch.bfloat16, 11008, 0, 45),
    # rotation in registers (the norm output re-reads the staged row), several rows per CTA
    ("rms", torch.bfloat16, 4096, 256, 3001), ("ln", torch.bfloat16, 768, 64, 5003),
    # rotation through shared memory (segments not aligned to the block)
    ("rms", torch.bfloat16, 11008, 256, 45),
    # wide row, rotation in registers: needs three staging slots although shared memory is tight
    ("rms", torch.bfloat16, 11008, 64, 1500)])
def test_norm_forward_matches_oracle(pk, kind, dtype, d, rotate, rows):
    x, _ = synthetic.sweep_activation(rows, d, 0.01, dtype=dtype, salt=d)
    w = synthetic.norm_weight(d, 0.1, dtype=dtype)
    b = (0.05 * torch.randn(d, generator=torch.Generator().manual_seed(d))).to(dtype)
    k = oc.n_outlier_count(d, 0.01)
    ch = oc.n_select_channels(oc.n_channel_scores(x), k)
    p, y, rstd, mean = pk.compress_n(x.to(DEV), ch.to(DEV), 4, 0, rotate,
                                     norm=dict(kind=kind, weight=w.to(DEV), bias=b.to(DEV), eps=1e-5))
    y_o, mean_o, rstd_o = oc.norm_forward(x, w, b, 1e-5, kind)
    assert y.dtype == x.dtype and y.shape == x.shape
    # 1e-2 relative at bf16 (the output is rounded to bf16 once on both sides)
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-4
    assert ((y.float().cpu() - y_o.float()).abs() <= tol * y_o.float().abs() + 1e-3).all()
    assert _rel_err(rstd, rstd_o) < 1e-5
    if kind == "ln":
        assert (mean.cpu() - mean_o).abs().max() < 1e-4 * x.float().abs().max()
    # the compressed copy is of the norm INPUT and is bit-exact
    c = oc.n_compress(x, ch, 4, 0, rotate)
    assert torch.equal(p.codes.cpu(), c.codes) and torch.equal(p.scales.cpu(), c.scales)
    assert not p.wait_expired()


# ------------------------------------------------------------------ backward kernels

def _packed_pair(pk, x, mode, bits, group=0, rotate=0):
    """Compress on the GPU and with the oracle; returns (packed, oracle reconstruction)."""
    if mode == "N":
        d = x.shape[-1]
        ch = oc.n_select_channels(oc.n_channel_scores(x), oc.n_outlier_count(d, 0.01))
        p = pk.compress_n(x.to(DEV), ch.to(DEV), bits, group, rotate)
        xh = oc.n_decompress(oc.n_compress(x.reshape(-1, d), ch, bits, group, rotate)).reshape(x.shape)
    else:
        thr, L, R, scale = oc.r_calibrate(x, 0.01, 1.0, bits, "per-channel", 0)
        p = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), bits)
        xh = oc.r_decompress(oc.r_compress(x, thr, scale, bits, 1.0))
    return p, xh


@pytest.mark.parametrize("kind,mode,bits,gdtype,d,rotate", [
    ("rms", "N", 4, torch.bfloat16, 4096, 256), ("rms", "R", 4, torch.bfloat16, 4096, 0),
    ("rms_gemma", "N", 8, torch.bfloat16, 1024, 0), ("ln", "R", 4, torch.float32, 768, 0),
    ("ln", "N", 2, torch.bfloat16, 3072, 0), ("rms", "N", 4, torch.float32, 768, 256)])
def test_norm_backward_matches_oracle(pk, kind, mode, bits, gdtype, d, rotate):
    b, s = 3, 41
    x, _ = synthetic.roundtrip_activation(b, s, d, planted=6, gain=20.0, dtype=torch.bfloat16, salt=d + bits)
    w = synthetic.norm_weight(d, 0.1, dtype=torch.float32)
    dy = torch.randn(b, s, d, generator=torch.Generator().manual_seed(5)).to(gdtype)
    p, xh = _packed_pair(pk, x, mode, bits, 0, rotate)
    _, mean_o, rstd_o = oc.norm_forward(x, w, torch.zeros(d), 1e-5, kind)
    for compat in (True, False):
        dx_o, dw_o, db_o = oc.norm_backward(xh, dy, w, mean_o, rstd_o, kind, ref_compat_c2=compat)
        dx, dw, db = pk.norm_bwd(p, dy.to(DEV), w.to(DEV), rstd_o.to(DEV),
                                 None if mean_o is None else mean_o.to(DEV), kind, ref_compat_c2=compat,
                                 need_dweight=True, need_dbias=(kind == "ln"))
        assert dx.dtype == torch.bfloat16 and dx.shape == dy.shape
        assert _rel_err(dx, dx_o) < 1e-2 and _cos(dx, dx_o) > 0.9999
        assert _cos(dw, dw_o) > 0.9999 and _rel_err(dw, dw_o) < 1e-3
        if kind == "ln":
            assert _rel_err(db, db_o) < 1e-3
    dx2, dw2, _ = pk.norm_bwd(p, dy.to(DEV), w.to(DEV), rstd_o.to(DEV),
                              None if mean_o is None else mean_o.to(DEV), kind)
    assert dw2 is None and _rel_err(dx2, oc.norm_backward(xh, dy, w, mean_o, rstd_o, kind)[0]) < 1e-2


@pytest.mark.parametrize("kind,bits,method,d", [
    ("rms", 4, "per-channel", 4096), ("rms", 2, "per-channel", 2048), ("ln", 8, "per-channel", 1024),
    ("rms", 4, "per-token", 768), ("ln", 2, "per-token", 4096), ("rms_gemma", 8, "per-tensor", 768),
    ("ln", 4, "per-tensor", 3072)])
def test_reference_mode_norm_backward_one_warp_per_row(pk, kind, bits, method, d):
    """Frozen norm weight, bf16 gradient, reference-mode record without a low-rank part: the warp-per-row
    kernel (static scales per channel / token / tensor, the row's element outliers put right from the pool
    after each pass).  Checked element by element, the outlier positions on their own as well."""
    b, s = 5, 67
    x, _ = synthetic.roundtrip_activation(b, s, d, planted=6, gain=20.0, dtype=torch.bfloat16, salt=d + bits)
    w = synthetic.norm_weight(d, 0.1, dtype=torch.float32)
    dy = torch.randn(b, s, d, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
    thr, L, R, scale = oc.r_calibrate(x, 0.02, 1.0, bits, method, 0)
    c = oc.r_compress(x, thr, scale, bits, 1.0)
    xh = oc.r_decompress(c)
    p = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), bits, outlier_ratio=0.05)
    assert int(p.pool_used.item()) > 0 and not p.overflowed()
    _, mean_o, rstd_o = oc.norm_forward(x, w, torch.zeros(d), 1e-5, kind)
    for compat in (True, False):
        dx_o = oc.norm_backward(xh, dy, w, mean_o, rstd_o, kind, ref_compat_c2=compat)[0].float()
        dx = pk.norm_bwd(p, dy.to(DEV), w.to(DEV), rstd_o.to(DEV), None if mean_o is None else mean_o.to(DEV), kind,
                         ref_compat_c2=compat)[0].float().cpu()
        tol = 1.6e-2 * dx_o.abs() + 2e-3 * dx_o.abs().max()
        assert ((dx - dx_o).abs() <= tol).all()
        out = (x.float().abs() > thr.float()).reshape(dx.shape)          # the element outliers
        assert out.any() and ((dx - dx_o).abs()[out] <= tol[out]).all()
    assert not p.wait_expired()


@pytest.mark.parametrize("op,mode,bits,gdtype,d,rotate", [
    ("silu", "N", 4, torch.bfloat16, 11008, 256), ("silu", "R", 8, torch.bfloat16, 1024, 0),
    ("gelu", "R", 4, torch.float32, 3072, 0), ("gelu", "N", 4, torch.bfloat16, 3072, 0),
    ("product", "N", 4, torch.bfloat16, 11008, 0), ("product", "R", 4, torch.bfloat16, 1024, 0),
    ("product", "N", 2, torch.float32, 1024, 256),
    # bf16 gradients, rows of up to 4096 channels without rotation: the warp-per-row kernel (whole and ragged
    # rounds of units, channel-mode and reference-mode records)
    ("silu", "N", 4, torch.bfloat16, 4096, 0), ("silu", "N", 2, torch.bfloat16, 768, 0),
    ("gelu", "N", 8, torch.bfloat16, 2048, 0), ("silu", "R", 4, torch.bfloat16, 4096, 0),
    ("gelu", "R", 2, torch.bfloat16, 768, 0), ("silu", "R", 8, torch.bfloat16, 3072, 0)])
def test_activation_backward_matches_oracle(pk, op, mode, bits, gdtype, d, rotate):
    b, s = 2, 23
    x1, _ = synthetic.roundtrip_activation(b, s, d, planted=6, gain=4.0, dtype=torch.bfloat16, salt=d)
    g = torch.randn(b, s, d, generator=torch.Generator().manual_seed(6)).to(gdtype)
    p1, xh1 = _packed_pair(pk, x1, mode, bits, 0, rotate)
    if op == "product":
        x2, _ = synthetic.roundtrip_activation(b, s, d, planted=6, gain=4.0, dtype=torch.bfloat16, salt=d + 1)
        p2, xh2 = _packed_pair(pk, x2, mode, bits, 0, rotate)
        d1, d2 = pk.act_bwd("product", p1, g.to(DEV), p2)
        o1, o2 = oc.product_backward(xh1, xh2, g)
        assert d1.dtype == o1.dtype and torch.equal(d1.cpu(), o1) and torch.equal(d2.cpu(), o2)
    else:
        dx = pk.act_bwd(op, p1, g.to(DEV))
        o = (oc.silu_backward if op == "silu" else oc.gelu_backward)(xh1, g)
        assert dx.dtype == o.dtype
        assert ((dx.float().cpu() - o.float()).abs() <= 1e-2 * o.float().abs() + 1e-4).all()


# ------------------------------------------------------------------ tensor-core weight gradient

@pytest.mark.parametrize("rows,d,bits,group,rotate,rank,frac", [
    (512, 4096, 4, 0, 0, 64, 0.01), (2048, 4096, 4, 0, 256, 64, 0.01), (300, 768, 4, 0, 0, 16, 0.01),
    (1000, 4096, 2, 128, 0, 64, 0.01), (777, 4096, 8, 0, 256, 16, 0.01), (64, 11008, 4, 0, 0, 64, 0.01),
    (4096, 1024, 4, 128, 64, 32, 0.01), (70, 4096, 4, 0, 0, 8, 0.01),
    # more than 128 outlier channels (two outlier tiles), 8-bit codes (two outlier CTAs per token slice), no outliers
    (3000, 4096, 4, 0, 256, 64, 0.05), (5000, 4096, 8, 0, 0, 64, 0.04), (900, 2048, 2, 0, 0, 32, 0.0)])
def test_lora_weight_gradient_from_codes(pk, rows, d, bits, group, rotate, rank, frac):
    x, _ = synthetic.sweep_activation(rows, d, max(frac, 0.005), salt=rank + bits)
    g = torch.randn(rows, rank, generator=torch.Generator().manual_seed(rank)).to(torch.bfloat16)
    k = oc.n_outlier_count(d, frac)
    ch = oc.n_select_channels(oc.n_channel_scores(x), k)
    p = pk.compress_n(x.to(DEV), ch.to(DEV) if k else None, bits, group, rotate)
    assert pk.lora_wgrad_supported(p, rank)
    dw = pk.lora_wgrad(p, g.to(DEV))
    xh = oc.n_decompress(oc.n_compress(x, ch, bits, group, rotate))
    want = g.float().T @ xh.float()
    assert dw.shape == (rank, d) and dw.dtype == torch.float32
    assert _cos(dw, want) > 0.9999 and _rel_err(dw, want) < 1e-2
    lib_path = pk.lora_wgrad(p, g.to(DEV), force_library=True)
    assert _cos(dw, lib_path) > 0.9999
    # the result in the weight's dtype straight from the kernel that finishes the sums: the same sums, rounded once
    dwb = pk.lora_wgrad(p, g.to(DEV), out_dtype=torch.bfloat16)
    assert dwb.dtype == torch.bfloat16 and torch.equal(dwb, dw.to(torch.bfloat16))
    assert not p.wait_expired()


@pytest.mark.parametrize("b,s,d,bits,method,rank,lr_rank,dtype", [
    (4, 512, 4096, 4, "per-channel", 64, 0, torch.bfloat16), (3, 100, 768, 4, "per-token", 16, 0, torch.float32),
    (2, 700, 4096, 8, "per-channel", 64, 2, torch.bfloat16), (5, 64, 1024, 2, "per-tensor", 32, 0, torch.bfloat16),
    (2, 256, 11008, 4, "per-channel", 64, 0, torch.bfloat16), (2, 128, 2048, 8, "per-token", 8, 4, torch.bfloat16)])
def test_lora_weight_gradient_from_reference_mode_codes(pk, b, s, d, bits, method, rank, lr_rank, dtype):
    """The reference's own format through the tensor-core kernel: static per-channel / per-token / per-tensor
    scales, element outliers from the pool, optional low-rank part; against the oracle's LoRA-A weight gradient
    on the oracle's reconstruction (operators/efficient_linear.py:61-67)."""
    x, _ = synthetic.roundtrip_activation(b, s, d, planted=max(4, d // 100), gain=20.0, dtype=dtype, salt=d + bits + rank)
    g = torch.randn(b, s, rank, generator=torch.Generator().manual_seed(rank + d)).to(torch.bfloat16)
    torch.manual_seed(d)
    thr, L, R, scale = oc.r_calibrate(x, 0.01, 1.0, bits, method, lr_rank)
    c = oc.r_compress(x, thr, scale, bits, 1.0, L if lr_rank else None, R if lr_rank else None)
    xh = oc.r_decompress(c, L if lr_rank else None, R if lr_rank else None)
    lr = (oc.fit_rows(L, s) @ R).to(torch.bfloat16).to(DEV) if lr_rank else None
    p = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), bits, lowrank=lr, outlier_ratio=0.01)
    assert torch.equal(p.codes.cpu().reshape(c.codes.shape).view(torch.uint8), c.codes.view(torch.uint8))
    assert pk.lora_wgrad_supported(p, rank) and int(p.status.item()) == 0
    dw = pk.lora_wgrad(p, g.to(DEV), path="tensor")
    want = torch.einsum("bsr,bsd->rd", g.float(), xh.float())
    assert dw.shape == (rank, d) and dw.dtype == torch.float32
    assert _cos(dw, want) > 0.9999 and _rel_err(dw, want) < 1e-2
    assert _cos(dw, pk.lora_wgrad(p, g.to(DEV), path="library")) > 0.9999
    # what the operators get (the faster route for this kind of record)
    assert _cos(dw, pk.lora_wgrad(p, g.to(DEV))) > 0.9999
    assert not p.wait_expired()


# ------------------------------------------------------------------ full-size properties (configuration 5 shapes)

@pytest.mark.parametrize("bits,group,rotate,rows", [(4, 0, 0, 65536), (2, 128, 256, 16384), (8, 0, 256, 16384)])
def test_full_size_roundtrip_properties(pk, bits, group, rotate, rows):
    """Configuration 5 at its sizes (the first case is the benchmark's own [65536, 4096] tensor): exact outlier
    channels, row slices bit for bit against the oracle, and size-independent error bounds over the whole tensor."""
    d = 4096
    x = torch.cat([synthetic.sweep_activation(8192, d, 0.01, salt=40 + bits)[0] * (1.0 + 0.01 * i)
                   for i in range(rows // 8192)]).to(torch.bfloat16)
    planted = synthetic.sweep_activation(8192, d, 0.01, salt=40 + bits)[1]
    xd = x.to(DEV)
    ch = pk.select_channels(pk.channel_absmax(xd), oc.n_outlier_count(d, 0.01))
    assert set(planted.tolist()) == set(ch.cpu().tolist())
    w = synthetic.norm_weight(d, 0.1)
    p, y, rstd, _ = pk.compress_n(xd, ch, bits, group, rotate,
                                  norm=dict(kind="rms", weight=w.to(DEV), bias=None, eps=1e-5))
    xh = pk.decompress(p).reshape(rows, d)
    # outlier channels are carried exactly
    assert torch.equal(xh[:, ch.long()], xd[:, ch.long()])
    # slices of rows (first, middle, last) against the oracle, bit for bit
    for sl in (slice(0, 96), slice(rows // 2 + 8, rows // 2 + 264), slice(rows - 96, rows)):
        c = oc.n_compress(x[sl], ch.cpu(), bits, group, rotate)
        assert torch.equal(p.codes[sl].cpu().view(torch.uint8), c.codes.view(torch.uint8))
        assert torch.equal(xh[sl].cpu(), oc.n_decompress(c))
    sl = slice(rows // 2 + 8, rows // 2 + 264)
    # checksum of checksums over the whole tensor: recompressing the reconstruction
    # keeps the scales within one bf16 rounding and the error bounded by half a step
    body = xd.float()
    body[:, ch.long()] = 0
    err = (xh.float() - xd.float())
    err[:, ch.long()] = 0
    g = d if group == 0 else group
    if not rotate:
        step = p.scales.repeat_interleave(g, dim=1)
        assert bool((err.abs() <= 0.5 * step * 1.01 + 0.008 * body.abs()).all())
    # the rotation is orthogonal, so in either case the row error norm is bounded by
    # half a quantisation step per element plus the bf16 rounding of the output
    bound = (g * (0.5 * p.scales) ** 2).sum(dim=1).sqrt() * 1.01 + 0.008 * body.norm(dim=1) + 1e-3
    assert bool((err.norm(dim=1) <= bound).all())
    y_o, _, rstd_o = oc.norm_forward(x[sl], w, None, 1e-5, "rms")
    assert ((y[sl].float().cpu() - y_o.float()).abs() <= 1e-2 * y_o.float().abs() + 1e-3).all()
    assert _rel_err(rstd[sl], rstd_o) < 1e-5
    assert not p.wait_expired()


# ------------------------------------------------------------------ empty and refused inputs

def test_empty_batches_and_refused_arguments(pk):
    from hyc_lora_b200._lib import HycError
    d = 1024
    ch = torch.tensor([3, 77], dtype=torch.int32, device=DEV)
    empty = torch.empty(0, d, dtype=torch.bfloat16, device=DEV)
    p = pk.compress_n(empty, ch, 4, 0, 0)
    assert p.codes.shape == (0, d // 2) and pk.decompress(p).numel() == 0
    w = torch.ones(d, dtype=torch.bfloat16, device=DEV)
    p2, y, rstd, _ = pk.compress_n(empty, ch, 4, 0, 0, norm=dict(kind="rms", weight=w, bias=None, eps=1e-5))
    assert y.numel() == 0 and rstd.numel() == 0
    assert pk.act_bwd("silu", p, empty).numel() == 0
    # a single row, and a row count that is no multiple of anything
    for rows in (1, 7):
        x, _ = synthetic.sweep_activation(rows, d, 0.01, salt=rows)
        c = oc.n_compress(x, ch.cpu(), 4, 0, 0)
        q = pk.compress_n(x.to(DEV), ch, 4, 0, 0)
        assert torch.equal(q.codes.cpu().view(torch.uint8), c.codes.view(torch.uint8))
    # refused before anything is launched
    with pytest.raises(HycError):
        pk.compress_n(torch.zeros(4, 192, dtype=torch.bfloat16, device=DEV), None, 4, 0, 0)      # cols % 128 != 0
    with pytest.raises(HycError):
        pk.compress_n(torch.zeros(4, d, dtype=torch.bfloat16, device=DEV), None, 3, 0, 0)        # bit width
    with pytest.raises(HycError):
        pk.compress_n(torch.zeros(4, d, dtype=torch.bfloat16, device=DEV), None, 4, 0, 96)       # rotation block
    with pytest.raises((RuntimeError, ValueError)):
        pk.compress_n(torch.zeros(4, d, dtype=torch.bfloat16), None, 4, 0, 0)                    # CPU tensor: no fallback


# ------------------------------------------------------------------ guarded outputs


class _Arena:
    """One device allocation filled with a pattern.  Outputs are carved from its middle, 256-byte aligned
    and a guard band apart; ``check`` asserts that every byte outside the carved regions still holds the
    pattern, so a store that leaves its buffer on either side is seen."""
    BAND, FILL = 4096, 0x5A

    def __init__(self, nbytes):
        self.buf = torch.full((nbytes,), self.FILL, dtype=torch.uint8, device=DEV)
        self.pos, self.taken = self.BAND, []

    def take(self, shape, dtype, zero=False):
        n = 1
        for v in shape:
            n *= v
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = self.pos
        assert start + nbytes + self.BAND <= self.buf.numel(), "arena too small"
        self.pos = (start + nbytes + self.BAND + 255) // 256 * 256
        self.taken.append((start, start + nbytes))
        t = self.buf[start:start + nbytes].view(dtype).view(*shape)
        if zero:
            t.zero_()
        return t

    def check(self):
        mask = torch.ones(self.buf.numel(), dtype=torch.bool, device=DEV)
        for a, b in self.taken:
            mask[a:b] = False
        bad = (self.buf != self.FILL) & mask
        assert not bool(bad.any()), f"bytes written outside the outputs at {bad.nonzero()[:8].flatten().tolist()}"


def _packed_n_in(arena, pk, rows, d, bits, group, rotate, ch):
    k = 0 if ch is None else ch.numel()
    return pk.Packed(mode="N", bits=bits, rows=rows, cols=d, seq=rows, shape=(1, rows, d),
                     codes=arena.take((rows, d * bits // 8), torch.uint8), status=arena.take((1,), torch.int32, zero=True),
                     channels=ch, group=group, rotate=rotate,
                     out_value=arena.take((rows, k), torch.bfloat16) if k else None,
                     scales=arena.take((rows, d // group if group else 1), torch.float32))


def _packed_r_in(arena, pk, rows, d, bits, thr, scale, pool_entries):
    return pk.Packed(mode="R", bits=bits, rows=rows, cols=d, seq=rows, shape=(1, rows, d),
                     codes=arena.take((rows, d * bits // 8), torch.uint8), status=arena.take((1,), torch.int32, zero=True),
                     scale=scale.contiguous(), scale_kind=pk.scale_kind_of(scale), thr=thr.reshape(1).float(),
                     pool=arena.take((pool_entries,), torch.int32), pool_used=arena.take((1,), torch.int32),
                     row_meta=arena.take((rows, 2), torch.int32))


def _dense(t, d):
    from hyc_lora_b200 import _lib
    r = _lib.HycDense()
    r.base, r.dtype, r.chunks, r.row_stride = t.data_ptr(), (_lib.HYC_BF16 if t.dtype == torch.bfloat16 else _lib.HYC_F32), 1, d
    return r


def _compress_into(pk, x, p, norm=None):
    """hyc_compress / hyc_norm_compress with every output already placed by the caller."""
    import ctypes as C
    from hyc_lora_b200 import _lib
    rec, dn = p.record(), _dense(x, p.cols)
    if norm is None:
        _lib.check(_lib.lib.hyc_compress(C.byref(dn), C.byref(rec), pk._stream()), "hyc_compress")
        return
    n = _lib.HycNormFwd()
    n.kind, n.eps = pk._NORM_KIND[norm["kind"]], 1e-5
    n.weight, n.bias, n.param_dtype = norm["weight"].data_ptr(), None, _lib.HYC_BF16
    n.y, n.rstd, n.mean = norm["y"].data_ptr(), norm["rstd"].data_ptr(), None
    _lib.check(_lib.lib.hyc_norm_compress(C.byref(dn), C.byref(n), C.byref(rec), pk._stream()), "hyc_norm_compress")


@pytest.mark.parametrize("d,bits,rotate,mode", [(768, 4, 0, "N"), (768, 4, 64, "N"), (11008, 4, 0, "N"), (11008, 2, 256, "N"),
                                               (768, 4, 0, "R"), (11008, 4, 0, "R"), (4096, 8, 256, "N"),
                                               # unit counts per lane that are not a power of two (register groups beyond the row)
                                               (2816, 8, 256, "N"), (3072, 4, 256, "N"), (3072, 4, 0, "N"), (2816, 2, 0, "N")])
def test_kernels_write_nothing_outside_their_outputs(pk, d, bits, rotate, mode):
    """Compress (alone and fused with the norm), decompress and norm backward with every output a view
    into the middle of one guarded allocation: results equal the ordinary calls', both flanks of every
    output stay untouched.  Row counts are odd so that the last CTA's walk ends mid-grid."""
    import ctypes as C
    from hyc_lora_b200 import _lib
    rows = 301
    x, _ = synthetic.sweep_activation(rows, d, 0.01, salt=d + bits + rotate)
    xd = x.to(DEV)
    w = synthetic.norm_weight(d, 0.1).to(DEV)
    dy = torch.randn(rows, d, generator=torch.Generator().manual_seed(d)).to(torch.bfloat16).to(DEV)
    arena = _Arena(rows * d * 12 + (1 << 20))
    if mode == "N":
        ch = pk.select_channels(pk.channel_absmax(xd), oc.n_outlier_count(d, 0.01))
        make = lambda: _packed_n_in(arena, pk, rows, d, bits, 0, rotate, ch)
        plain = pk.compress_n(xd, ch, bits, 0, rotate)
    else:
        thr, _, _, scale = oc.r_calibrate(x.reshape(1, rows, d), 0.01, 1.0, bits, "per-channel", 0)
        thr, scale = thr.to(DEV), scale.to(DEV)
        entries = pk.default_pool_entries(rows, d, 0.01)
        make = lambda: _packed_r_in(arena, pk, rows, d, bits, thr, scale, entries)
        plain = pk.compress_r(xd.reshape(1, rows, d), thr, scale, bits)
    p1, p2 = make(), make()
    y, rstd = arena.take((rows, d), torch.bfloat16), arena.take((rows,), torch.float32)
    _compress_into(pk, xd, p1)
    _compress_into(pk, xd, p2, norm=dict(kind="rms", weight=w, y=y, rstd=rstd))
    for p in (p1, p2):
        assert torch.equal(p.codes, plain.codes) and int(p.status.item()) == 0
    # decompress and norm backward into guarded outputs
    xh = arena.take((rows, d), torch.bfloat16)
    rec, out = p1.record(), _dense(xh, d)
    _lib.check(_lib.lib.hyc_decompress(C.byref(rec), C.byref(out), pk._stream()), "hyc_decompress")
    assert torch.equal(xh.reshape(-1), pk.decompress(plain).reshape(-1))
    dx = arena.take((rows, d), torch.bfloat16)
    a = _lib.HycNormBwdArgs()
    a.kind, a.ref_compat_c2 = _lib.HYC_NORM_RMS, 1
    a.weight, a.param_dtype, a.dy, a.dy_dtype = w.data_ptr(), _lib.HYC_BF16, dy.data_ptr(), _lib.HYC_BF16
    a.rstd, a.mean, a.dx = rstd.data_ptr(), None, dx.data_ptr()
    _lib.check(_lib.lib.hyc_norm_bwd(C.byref(rec), C.byref(a), pk._stream()), "hyc_norm_bwd")
    want_dx, _, _ = pk.norm_bwd(plain, dy, w, rstd, None, "rms")
    assert torch.equal(dx, want_dx)
    torch.cuda.synchronize()
    arena.check()


@pytest.mark.parametrize("d,bits,group,rotate,kind,rows", [
    # the rotating kernel that gives a lane one chunk of every packed segment (segments of 32 chunks of 32, 64 or
    # 128 channels); few rows take its 8-warp build, many rows the 12-warp one
    (4096, 4, 0, 256, None, 300), (4096, 4, 0, 256, "rms", 4001), (4096, 4, 128, 256, "ln", 300),
    (4096, 4, 0, 16, "rms", 300), (4096, 4, 0, 1024, None, 4001), (4096, 4, 128, 1024, "rms", 4001),
    (2048, 4, 0, 256, "rms", 4001), (2048, 4, 128, 64, None, 300), (2048, 4, 0, 1024, "ln", 300),
    (4096, 2, 0, 256, "rms", 300), (4096, 2, 128, 1024, None, 4001), (4096, 2, 0, 64, "ln", 4001),
    (4096, 8, 0, 256, "rms", 4001), (4096, 8, 128, 4096, None, 300), (4096, 8, 128, 256, "ln", 300),
    (2048, 8, 0, 1024, "rms", 300), (1024, 8, 128, 256, None, 4001), (1024, 8, 0, 1024, "rms", 300)])
def test_rotating_forward_one_chunk_per_lane(pk, d, bits, group, rotate, kind, rows):
    """Codes, scales and outlier values equal the oracle's bit for bit; the norm output and the row
    statistics are the oracle's within the bf16 tolerance; nothing is written outside the outputs."""
    import ctypes as C
    from hyc_lora_b200 import _lib
    x, _ = synthetic.sweep_activation(rows, d, 0.01, dtype=torch.bfloat16, salt=d + bits + rotate)
    x[rows // 2] = 0                                  # a dead row: scale 1, codes of zero
    xd = x.to(DEV)
    k = oc.n_outlier_count(d, 0.01)
    ch = pk.select_channels(pk.channel_absmax(xd), k)
    c = oc.n_compress(x, ch.cpu(), bits, group, rotate)
    w = synthetic.norm_weight(d, 0.1, dtype=torch.bfloat16)
    b = (0.05 * torch.randn(d, generator=torch.Generator().manual_seed(d))).to(torch.bfloat16)
    arena = _Arena(rows * d * 4 + (1 << 20))
    p = _packed_n_in(arena, pk, rows, d, bits, group, rotate, ch)
    rec, dn = p.record(), _dense(xd, d)
    if kind is None:
        _lib.check(_lib.lib.hyc_compress(C.byref(dn), C.byref(rec), pk._stream()), "hyc_compress")
    else:
        y, rstd = arena.take((rows, d), torch.bfloat16), arena.take((rows,), torch.float32)
        mean = arena.take((rows,), torch.float32)
        wd, bd = w.to(DEV), b.to(DEV)
        n = _lib.HycNormFwd()
        n.kind, n.eps = pk._NORM_KIND[kind], 1e-5
        n.weight, n.bias, n.param_dtype = wd.data_ptr(), (bd.data_ptr() if kind == "ln" else None), _lib.HYC_BF16
        n.y, n.rstd, n.mean = y.data_ptr(), rstd.data_ptr(), (mean.data_ptr() if kind == "ln" else None)
        _lib.check(_lib.lib.hyc_norm_compress(C.byref(dn), C.byref(n), C.byref(rec), pk._stream()), "hyc_norm_compress")
        y_o, mean_o, rstd_o = oc.norm_forward(x, w, b, 1e-5, kind)
        assert ((y.float().cpu() - y_o.float()).abs() <= 1e-2 * y_o.float().abs() + 1e-3).all()
        assert _rel_err(rstd, rstd_o) < 1e-5
        if kind == "ln":
            assert (mean.cpu() - mean_o).abs().max() < 1e-4
    torch.cuda.synchronize()
    assert torch.equal(p.scales.cpu(), c.scales)
    assert torch.equal(p.codes.cpu().view(torch.uint8), c.codes.view(torch.uint8))
    assert torch.equal(p.out_value.cpu(), c.out_value)
    assert int(p.status.item()) == 0
    arena.check()


@pytest.mark.parametrize("d,bits,group,rotate,kind,rows", [
    (4096, 4, 0, 256, "rms", 300), (4096, 4, 128, 256, "ln", 4001), (4096, 4, 0, 16, "rms_gemma", 300),
    (4096, 4, 128, 1024, "rms", 300), (2048, 4, 0, 256, "ln", 300), (2048, 4, 128, 64, "rms", 4001),
    (4096, 2, 0, 256, "rms", 4001), (4096, 2, 128, 1024, "ln", 300), (4096, 8, 0, 256, "rms", 300),
    (4096, 8, 128, 4096, "ln", 300), (2048, 8, 0, 1024, "rms", 300), (1024, 8, 128, 256, "rms", 4001)])
def test_rotated_consumers_one_chunk_per_lane(pk, d, bits, group, rotate, kind, rows):
    """Decompress of a rotated record equals the oracle's bit for bit; decompress + norm backward (frozen
    weight, bf16 gradient) is the oracle's within the bf16 tolerance; both write inside their outputs only."""
    import ctypes as C
    from hyc_lora_b200 import _lib
    x, _ = synthetic.sweep_activation(rows, d, 0.01, dtype=torch.bfloat16, salt=d + bits + rotate + 5)
    x[rows // 2] = 0
    xd = x.to(DEV)
    k = oc.n_outlier_count(d, 0.01)
    ch = pk.select_channels(pk.channel_absmax(xd), k)
    c = oc.n_compress(x, ch.cpu(), bits, group, rotate)
    xh_o = oc.n_decompress(c)
    p = pk.compress_n(xd, ch, bits, group, rotate)
    w = synthetic.norm_weight(d, 0.1, dtype=torch.bfloat16)
    dy = torch.randn(rows, d, generator=torch.Generator().manual_seed(d + 1)).to(torch.bfloat16)
    _, mean_o, rstd_o = oc.norm_forward(x, w, torch.zeros(d), 1e-5, kind)
    arena = _Arena(rows * d * 4 + (1 << 20))
    xh, dx = arena.take((rows, d), torch.bfloat16), arena.take((rows, d), torch.bfloat16)
    rec, out = p.record(), _dense(xh, d)
    _lib.check(_lib.lib.hyc_decompress(C.byref(rec), C.byref(out), pk._stream()), "hyc_decompress")
    wd, dyd, rstd = w.to(DEV), dy.to(DEV), rstd_o.to(DEV)
    mean = mean_o.to(DEV) if kind == "ln" else None
    a = _lib.HycNormBwdArgs()
    a.kind, a.ref_compat_c2 = pk._NORM_KIND[kind], 1
    a.weight, a.param_dtype, a.dy, a.dy_dtype = wd.data_ptr(), _lib.HYC_BF16, dyd.data_ptr(), _lib.HYC_BF16
    a.rstd, a.mean, a.dx = rstd.data_ptr(), (mean.data_ptr() if mean is not None else None), dx.data_ptr()
    _lib.check(_lib.lib.hyc_norm_bwd(C.byref(rec), C.byref(a), pk._stream()), "hyc_norm_bwd")
    torch.cuda.synchronize()
    assert torch.equal(xh.cpu(), xh_o)
    dx_o, _, _ = oc.norm_backward(xh_o, dy, w, mean_o if kind == "ln" else None, rstd_o, kind)
    err = (dx.float().cpu() - dx_o.float()).abs().max() / dx_o.float().abs().max()
    assert err < 1e-2, f"norm backward differs from the oracle ({err:.3e})"
    assert ((dx.float().cpu() - dx_o.float()).abs() <= 2e-2 * dx_o.float().abs() + 2e-2 * dx_o.float().abs().mean()).all()
    assert int(p.status.item()) == 0
    arena.check()


@pytest.mark.parametrize("d,bits,group,rotate,rows,frac", [
    (11008, 4, 0, 64, 70, 0.01), (11008, 4, 128, 64, 2500, 0.02), (11008, 2, 0, 16, 70, 0.01), (11008, 8, 128, 64, 70, 0.01),
    (14336, 4, 0, 256, 70, 0.02), (14336, 2, 128, 16, 300, 0.02), (3072, 8, 128, 256, 70, 0.01), (8192, 4, 0, 256, 300, 0.01),
    (5120, 4, 128, 64, 70, 0.01), (4096, 4, 0, 256, 2500, 0.01), (4096, 4, 128, 1024, 300, 0.01), (16384, 4, 0, 1024, 70, 0.005)])
def test_rotated_activation_backward_wide_rows(pk, d, bits, group, rotate, rows, frac):
    """SiLU / GELU / product backward from rotated records of many widths with a bf16 gradient: the product's two
    results equal the oracle's bit for bit, the activations' are within the tolerance of the formulas; nothing
    is written outside the outputs."""
    import ctypes as C
    from hyc_lora_b200 import _lib
    x1, _ = synthetic.sweep_activation(rows, d, frac, dtype=torch.bfloat16, salt=d + bits + 11)
    x2, _ = synthetic.sweep_activation(rows, d, frac, dtype=torch.bfloat16, salt=d + bits + 12)
    x1 = 0.25 * x1
    g = torch.randn(rows, d, generator=torch.Generator().manual_seed(d)).to(torch.bfloat16)
    k = oc.n_outlier_count(d, frac)
    recs, xhs = [], []
    for x in (x1, x2):
        xd = x.to(DEV)
        ch = pk.select_channels(pk.channel_absmax(xd), k)
        recs.append(pk.compress_n(xd, ch, bits, group, rotate))
        xhs.append(oc.n_decompress(oc.n_compress(x, ch.cpu(), bits, group, rotate)))
    gd = g.to(DEV)
    arena = _Arena(rows * d * 10 + (1 << 20))
    outs = [arena.take((rows, d), torch.bfloat16) for _ in range(4)]
    r1, r2 = recs[0].record(), recs[1].record()
    for op, o1, o2 in ((_lib.HYC_ACT_SILU, outs[0], None), (_lib.HYC_ACT_GELU_TANH, outs[1], None),
                       (_lib.HYC_ACT_PRODUCT, outs[2], outs[3])):
        _lib.check(_lib.lib.hyc_act_bwd(op, C.byref(r1), C.byref(r2) if o2 is not None else None, gd.data_ptr(), _lib.HYC_BF16,
                                        o1.data_ptr(), o2.data_ptr() if o2 is not None else None, pk._stream()), "hyc_act_bwd")
    torch.cuda.synchronize()
    s_o, g_o = oc.silu_backward(xhs[0], g), oc.gelu_backward(xhs[0], g)
    assert ((outs[0].float().cpu() - s_o.float()).abs() <= 1e-2 * s_o.float().abs() + 1e-4).all()
    assert ((outs[1].float().cpu() - g_o.float()).abs() <= 1e-2 * g_o.float().abs() + 1e-4).all()
    p1_o, p2_o = oc.product_backward(xhs[0], xhs[1], g)
    assert torch.equal(outs[2].cpu(), p1_o) and torch.equal(outs[3].cpu(), p2_o)
    assert int(recs[0].status.item()) == 0 and int(recs[1].status.item()) == 0
    arena.check()


def test_chunk_and_wide_kernels_without_outlier_channels(pk):
    """No outlier channels at all (ratio 0): the rotating forward, its two-record variant, the rotated consumers
    and the one-pass activation / product sites."""
    rows, d, bits, rotate = 300, 4096, 4, 256
    x, _ = synthetic.sweep_activation(rows, d, 0.01, dtype=torch.bfloat16, salt=77)
    xd = x.to(DEV)
    w = synthetic.norm_weight(d, 0.1, dtype=torch.bfloat16).to(DEV)
    none = torch.empty(0, dtype=torch.int32)
    c = oc.n_compress(x, none, bits, 0, rotate)
    p = pk.compress_n(xd, None, bits, 0, rotate)
    assert torch.equal(p.codes.cpu(), c.codes) and torch.equal(p.scales.cpu(), c.scales)
    assert torch.equal(pk.decompress(p).cpu().reshape(rows, d), oc.n_decompress(c))
    norm = dict(kind="rms", weight=w, bias=None, eps=1e-5)
    px, y, rstd, _, py = pk.compress_n(xd, None, bits, 0, rotate, norm=norm, also_output=dict(channels=None, bits=bits, group=0, rotate=rotate))
    assert py is not None and torch.equal(px.codes, p.codes)
    assert torch.equal(py.codes.cpu(), oc.n_compress(y.cpu(), none, bits, 0, rotate).codes)
    dy = torch.randn(rows, d, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    dx, _, _ = pk.norm_bwd(p, dy.to(DEV), w, rstd, None, "rms")
    dx_o, _, _ = oc.norm_backward(oc.n_decompress(c), dy, w.cpu(), None, rstd.cpu(), "rms")
    assert (dx.float().cpu() - dx_o.float()).abs().max() / dx_o.float().abs().max() < 1e-2
    fmt = dict(channels=None, bits=bits, group=0, rotate=64)
    pg, act, pa = pk.act_compress_n("silu", xd, None, bits, 0, 64, also_output=fmt)
    assert torch.equal(pg.codes.cpu(), oc.n_compress(x, none, bits, 0, 64).codes)
    assert torch.equal(pa.codes.cpu(), oc.n_compress(act.cpu(), none, bits, 0, 64).codes)
    pu, prod, pp = pk.product_compress_n(act, xd, None, bits, 0, 64, also_output=fmt)
    assert torch.equal(prod, act * xd) and torch.equal(pp.codes.cpu(), oc.n_compress(prod.cpu(), none, bits, 0, 64).codes)


WIDE_CASES = [
    # d, bits, group, rotate, rows, outlier fraction
    (11008, 4, 0, 64, 70, 0.01), (11008, 4, 0, 0, 2500, 0.01), (11008, 4, 128, 64, 300, 0.02), (11008, 2, 0, 16, 70, 0.01),
    (11008, 8, 128, 64, 70, 0.01), (14336, 2, 128, 0, 300, 0.02), (14336, 4, 0, 256, 70, 0.01), (3072, 4, 0, 0, 300, 0.01),
    (3072, 8, 128, 256, 70, 0.01), (8192, 4, 0, 256, 300, 0.01), (5120, 4, 128, 64, 70, 0.01), (4096, 4, 0, 256, 2500, 0.01),
    (16384, 4, 0, 1024, 70, 0.005)]


def _same_record(got, want):
    assert torch.equal(got.codes, want.codes)
    assert torch.equal(got.scales, want.scales)
    if want.out_value is not None:
        assert torch.equal(got.out_value, want.out_value)
    assert int(got.status.item()) == 0


@pytest.mark.parametrize("d,bits,group,rotate,rows,frac", WIDE_CASES)
def test_wide_rows_compress_against_oracle(pk, d, bits, group, rotate, rows, frac):
    """Rows wider than one warp holds (up to four warps per row): the record equals the oracle's."""
    x, _ = synthetic.sweep_activation(rows, d, frac, dtype=torch.bfloat16, salt=d + bits)
    x[rows // 3] = 0
    xd = x.to(DEV)
    k = oc.n_outlier_count(d, frac)
    ch = pk.select_channels(pk.channel_absmax(xd), k)
    c = oc.n_compress(x, ch.cpu(), bits, group, rotate)
    p = pk.compress_n(xd, ch, bits, group, rotate)
    assert torch.equal(p.scales.cpu(), c.scales)
    assert torch.equal(p.codes.cpu().view(torch.uint8), c.codes.view(torch.uint8))
    assert torch.equal(p.out_value.cpu(), c.out_value)
    assert torch.equal(pk.decompress(p).cpu().reshape(rows, d), oc.n_decompress(c))


@pytest.mark.parametrize("d,bits,group,rotate,rows,frac", WIDE_CASES)
@pytest.mark.parametrize("op", ["silu", "gelu"])
def test_activation_and_both_records_in_one_pass(pk, op, d, bits, group, rotate, rows, frac):
    """``hyc_act_compress``: the output is torch's, the record of the input is that of ``hyc_compress``, and
    the record of the output is that of ``hyc_compress`` on the output."""
    x, _ = synthetic.sweep_activation(rows, d, frac, dtype=torch.bfloat16, salt=d + bits + 1)
    xd = (0.25 * x).to(DEV)
    k = oc.n_outlier_count(d, frac)
    ch_x = pk.select_channels(pk.channel_absmax(xd), k)
    want_y = torch.nn.functional.silu(xd) if op == "silu" else torch.nn.functional.gelu(xd)
    ch_y = pk.select_channels(pk.channel_absmax(want_y), k)
    got = pk.act_compress_n(op, xd, ch_x, bits, group, rotate, also_output=dict(channels=ch_y, bits=bits, group=group, rotate=rotate))
    assert got is not None, "the call was refused"
    px, y, py = got
    # one rounding to bf16 of an fp32 value on both sides; the two exponential / erf routines may differ in the
    # last place of the fp32 value
    assert ((y.float() - want_y.float()).abs() <= 2 ** -7 * want_y.float().abs() + 1e-30).all()
    _same_record(px, pk.compress_n(xd, ch_x, bits, group, rotate))
    _same_record(py, pk.compress_n(y, ch_y, bits, group, rotate))
    # without the second record
    px1, y1, none = pk.act_compress_n(op, xd, ch_x, bits, group, rotate)
    assert none is None and torch.equal(y1, y)
    _same_record(px1, px)


@pytest.mark.parametrize("d,bits,group,rotate,rows,frac", WIDE_CASES)
def test_product_and_both_records_in_one_pass(pk, d, bits, group, rotate, rows, frac):
    """``hyc_product_compress``: ``y = x1 * x2`` exactly, the record of ``x2`` and the record of ``y``."""
    x1, _ = synthetic.sweep_activation(rows, d, frac, dtype=torch.bfloat16, salt=d + bits + 2)
    x2, _ = synthetic.sweep_activation(rows, d, frac, dtype=torch.bfloat16, salt=d + bits + 3)
    x1d, x2d = (0.25 * x1).to(DEV), x2.to(DEV)
    k = oc.n_outlier_count(d, frac)
    ch2 = pk.select_channels(pk.channel_absmax(x2d), k)
    want_y = x1d * x2d
    ch_y = pk.select_channels(pk.channel_absmax(want_y), k)
    got = pk.product_compress_n(x1d, x2d, ch2, bits, group, rotate, also_output=dict(channels=ch_y, bits=bits, group=group, rotate=rotate))
    assert got is not None, "the call was refused"
    p2, y, py = got
    assert torch.equal(y, want_y)
    _same_record(p2, pk.compress_n(x2d, ch2, bits, group, rotate))
    _same_record(py, pk.compress_n(want_y, ch_y, bits, group, rotate))
    p2b, yb, none = pk.product_compress_n(x1d, x2d, ch2, bits, group, rotate)
    assert none is None and torch.equal(yb, want_y)
    _same_record(p2b, p2)


def test_wide_row_kernels_write_nothing_outside_their_outputs(pk):
    """The three one-pass calls with every output inside a guarded arena."""
    import ctypes as C
    from hyc_lora_b200 import _lib
    d, rows, bits = 11008, 131, 4
    x1, _ = synthetic.sweep_activation(rows, d, 0.01, dtype=torch.bfloat16, salt=5)
    x2, _ = synthetic.sweep_activation(rows, d, 0.01, dtype=torch.bfloat16, salt=6)
    x1d, x2d = x1.to(DEV), x2.to(DEV)
    ch = pk.select_channels(pk.channel_absmax(x2d), 111)
    arena = _Arena(rows * d * 12 + (1 << 20))
    for op in ("compress", "silu", "product"):
        pa = _packed_n_in(arena, pk, rows, d, bits, 0, 64, ch)
        pb = _packed_n_in(arena, pk, rows, d, bits, 0, 64, ch)
        y = arena.take((rows, d), torch.bfloat16)
        ra, rb = pa.record(), pb.record()
        d1, d2 = _dense(x1d, d), _dense(x2d, d)
        if op == "compress":
            _lib.check(_lib.lib.hyc_compress(C.byref(d2), C.byref(ra), pk._stream()), "hyc_compress")
        elif op == "silu":
            _lib.check(_lib.lib.hyc_act_compress(C.byref(d2), _lib.HYC_ACT_SILU, y.data_ptr(), C.byref(ra), C.byref(rb),
                                                 pk._stream()), "hyc_act_compress")
        else:
            _lib.check(_lib.lib.hyc_product_compress(C.byref(d1), C.byref(d2), y.data_ptr(), C.byref(ra), C.byref(rb),
                                                     pk._stream()), "hyc_product_compress")
        torch.cuda.synchronize()
        _same_record(pa, pk.compress_n(x2d, ch, bits, 0, 64))
    arena.check()


@pytest.mark.parametrize("kind,d,bits,group,rotate,rows", [
    ("rms", 4096, 4, 0, 0, 3001), ("rms", 4096, 2, 128, 0, 517), ("rms_gemma", 2048, 8, 0, 0, 700),
    ("ln", 768, 4, 0, 0, 5003), ("rms", 2816, 4, 128, 0, 333), ("ln", 3072, 2, 0, 0, 129), ("rms", 1024, 4, 0, 0, 1),
    # rotated codes (the kernel that keeps the rotated row in registers)
    ("rms", 4096, 4, 0, 256, 3001), ("rms", 4096, 2, 128, 256, 517), ("ln", 1024, 4, 0, 64, 5003),
    ("rms_gemma", 2048, 8, 0, 256, 700), ("rms", 3072, 4, 128, 16, 333), ("ln", 2048, 2, 0, 256, 129)])
def test_norm_output_record_from_the_same_pass(pk, kind, d, bits, group, rotate, rows):
    """``hyc_norm_compress2``: the record of the norm OUTPUT that the pass emits beside the record of its
    input is, bit for bit, the record a separate ``hyc_compress`` of that output makes; the input record,
    the output and the row statistics are those of ``hyc_norm_compress``; nothing else is written."""
    import ctypes as C
    from hyc_lora_b200 import _lib
    x, _ = synthetic.sweep_activation(rows, d, 0.01, dtype=torch.bfloat16, salt=d + bits)
    xd = x.to(DEV)
    w = synthetic.norm_weight(d, 0.1, dtype=torch.bfloat16).to(DEV)
    b = (0.05 * torch.randn(d, generator=torch.Generator().manual_seed(d))).to(torch.bfloat16).to(DEV)
    k = oc.n_outlier_count(d, 0.01)
    ch_x = pk.select_channels(pk.channel_absmax(xd), k)
    norm = dict(kind=kind, weight=w, bias=b, eps=1e-5)
    p1, y1, rstd1, mean1 = pk.compress_n(xd, ch_x, bits, group, rotate, norm=norm)
    # the consumer's outlier channels come from the norm output, not from its input
    ch_y = pk.select_channels(pk.channel_absmax(y1), k)
    want_y = pk.compress_n(y1, ch_y, bits, group, rotate)
    px, y, rstd, mean, py = pk.compress_n(xd, ch_x, bits, group, rotate, norm=norm,
                                          also_output=dict(channels=ch_y, bits=bits, group=group, rotate=rotate))
    assert py is not None, "the pair was refused"
    assert torch.equal(y, y1) and torch.equal(rstd, rstd1)
    if kind == "ln":
        assert torch.equal(mean, mean1)
    for got, want in ((px, p1), (py, want_y)):
        assert torch.equal(got.codes, want.codes)
        assert torch.equal(got.scales, want.scales)
        assert torch.equal(got.out_value, want.out_value)
        assert int(got.status.item()) == 0
    # against the CPU restatement, on the output the kernel wrote
    o = oc.n_compress(y.cpu(), ch_y.cpu(), bits, group, rotate)
    assert torch.equal(py.codes.cpu().view(torch.uint8), o.codes.view(torch.uint8))
    assert torch.equal(py.scales.cpu(), o.scales) and torch.equal(py.out_value.cpu(), o.out_value)
    # the same call with every output inside a guarded arena
    arena = _Arena(rows * d * 8 + (1 << 20))
    ax = _packed_n_in(arena, pk, rows, d, bits, group, rotate, ch_x)
    ay = _packed_n_in(arena, pk, rows, d, bits, group, rotate, ch_y)
    yy, rr = arena.take((rows, d), torch.bfloat16), arena.take((rows,), torch.float32)
    mm = arena.take((rows,), torch.float32)
    n = _lib.HycNormFwd()
    n.kind, n.eps = pk._NORM_KIND[kind], 1e-5
    n.weight, n.bias, n.param_dtype = w.data_ptr(), (b.data_ptr() if kind == "ln" else None), _lib.HYC_BF16
    n.y, n.rstd, n.mean = yy.data_ptr(), rr.data_ptr(), (mm.data_ptr() if kind == "ln" else None)
    rx, ry, dn = ax.record(), ay.record(), _dense(xd, d)
    _lib.check(_lib.lib.hyc_norm_compress2(C.byref(dn), C.byref(n), C.byref(rx), C.byref(ry), pk._stream()),
               "hyc_norm_compress2")
    torch.cuda.synchronize()
    assert torch.equal(ay.codes, want_y.codes) and torch.equal(ax.codes, p1.codes) and torch.equal(yy, y1)
    if kind != "ln":
        assert bool((mm.view(torch.uint8) == _Arena.FILL).all())
    arena.check()


def test_norm_output_record_is_refused_where_the_pair_is_not_built(pk):
    """Records of two formats (rotation block, bits, scale grouping): the call answers HYC_ERR_SHAPE
    and writes nothing; the wrapper then returns no second record and the first one as ever."""
    import ctypes as C
    from hyc_lora_b200 import _lib
    d, rows = 1024, 64
    x, _ = synthetic.sweep_activation(rows, d, 0.01, dtype=torch.bfloat16, salt=3)
    xd = x.to(DEV)
    w = synthetic.norm_weight(d, 0.1, dtype=torch.bfloat16).to(DEV)
    ch = pk.select_channels(pk.channel_absmax(xd), 10)
    norm = dict(kind="rms", weight=w, bias=None, eps=1e-5)
    p1, y1, _, _ = pk.compress_n(xd, ch, 4, 0, 256, norm=norm)
    px, y, _, _, py = pk.compress_n(xd, ch, 4, 0, 256, norm=norm, also_output=dict(channels=ch, bits=4, group=0, rotate=64))
    assert py is None and torch.equal(px.codes, p1.codes) and torch.equal(y, y1)
    px, y, _, _, py = pk.compress_n(xd, ch, 4, 0, 0, norm=norm, also_output=dict(channels=ch, bits=2, group=0, rotate=0))
    assert py is None
    for fmt_x, fmt_y in (((4, 0, 256), (4, 0, 64)), ((4, 0, 0), (2, 0, 0)), ((4, 0, 0), (4, 128, 0))):
        arena = _Arena(rows * d * 8 + (1 << 20))
        ax = _packed_n_in(arena, pk, rows, d, *fmt_x, ch)
        ay = _packed_n_in(arena, pk, rows, d, *fmt_y, ch)
        yy, rr = arena.take((rows, d), torch.bfloat16), arena.take((rows,), torch.float32)
        arena.taken.clear()                      # nothing may be written at all
        ax.status.view(torch.uint8).fill_(_Arena.FILL), ay.status.view(torch.uint8).fill_(_Arena.FILL)
        n = _lib.HycNormFwd()
        n.kind, n.eps = pk._NORM_KIND["rms"], 1e-5
        n.weight, n.bias, n.param_dtype = w.data_ptr(), None, _lib.HYC_BF16
        n.y, n.rstd, n.mean = yy.data_ptr(), rr.data_ptr(), None
        rx, ry, dn = ax.record(), ay.record(), _dense(xd, d)
        rc = _lib.lib.hyc_norm_compress2(C.byref(dn), C.byref(n), C.byref(rx), C.byref(ry), pk._stream())
        assert rc == _lib.HYC_ERR_SHAPE
        torch.cuda.synchronize()
        arena.check()


def test_config1_in_channel_mode_on_its_own_tensor(pk):
    """Configuration 1 as written: LayerNorm of the [8,128,768] fp32 activation, the top 1 % absmax
    channels (8 of 768 -- they must be the planted ones) kept in full precision, the rest INT4 with one
    absmax scale per token; then the LoRA-A gradients from the packed record against the oracle."""
    x, planted = synthetic.roundtrip_activation()
    a, grad = synthetic.lora_a_problem()
    w, b = torch.ones(768), torch.zeros(768)
    xd = x.to(DEV)
    k = oc.n_outlier_count(768, 0.01)
    assert k == 8
    ch = pk.select_channels(pk.channel_absmax(xd), k)
    assert torch.equal(ch.cpu().long(), planted)
    p, y, rstd, mean = pk.compress_n(xd, ch, 4, 0, 0, norm=dict(kind="ln", weight=w.to(DEV), bias=b.to(DEV), eps=1e-5))
    c = oc.n_compress(x.reshape(-1, 768), ch.cpu(), 4, 0, 0)
    assert torch.equal(p.codes.cpu().reshape(c.codes.shape).view(torch.uint8), c.codes.view(torch.uint8))
    assert torch.equal(p.scales.cpu(), c.scales) and torch.equal(p.out_value.cpu(), c.out_value)
    y_o, mean_o, rstd_o = oc.norm_forward(x, w, b, 1e-5, "ln")
    assert _rel_err(y, y_o) < 1e-4 and _rel_err(rstd, rstd_o) < 1e-5
    xh_o = oc.n_decompress(c).reshape(x.shape)
    assert torch.equal(pk.decompress(p).cpu(), xh_o)
    # check (i): an upstream gradient applied at the LoRA-A output
    dx_o, da_o = oc.linear_backward(xh_o, a.to(torch.bfloat16), grad)
    da = pk.lora_wgrad(p, grad.to(DEV))
    assert pk.lora_wgrad_supported(p, 16)
    assert _cos(da, da_o) > 0.9999 and _rel_err(da, da_o.float()) < 1e-2
    # LayerNorm backward from the packed record
    g = torch.randn(8, 128, 768, generator=torch.Generator().manual_seed(5))
    dxn, _, _ = pk.norm_bwd(p, g.to(DEV).reshape(-1, 768), w.to(DEV), rstd, mean, "ln")
    dxn_o, _, _ = oc.norm_backward(xh_o, g, w, mean_o, rstd_o, "ln")
    assert _rel_err(dxn.reshape(x.shape), dxn_o) < 1e-2


def test_status_poll_reports_a_pool_overflow_without_blocking(pk):
    """Nothing on the hot path reads a record's status word; the per-device accumulator does.  A pool that
    is far too small overflows: the first poll only starts the copy to the host (and reports what the poll
    before it fetched: nothing), the next one reports the overflow, warns and doubles the capacities."""
    pk.reset_status()
    x, _ = synthetic.roundtrip_activation(2, 64, 768, planted=5, gain=20.0, dtype=torch.bfloat16, salt=3)
    thr, _, _, scale = oc.r_calibrate(x, 0.01, 1.0, 4, "per-channel", 0)
    before = pk.default_pool_entries(128, 768, 0.01)
    p = pk.compress_r(x.to(DEV), thr.to(DEV), scale.to(DEV), 4, pool_entries=8)
    assert pk.poll_status() == 0
    torch.cuda.synchronize()
    with pytest.warns(UserWarning, match="POOL_OVERFLOW"):
        seen = pk.poll_status()
    assert seen & 1 and p.overflowed()
    assert pk.default_pool_entries(128, 768, 0.01) > before
    pk.reset_status()
    assert pk.default_pool_entries(128, 768, 0.01) == before and pk.poll_status(wait=True) == 0


def test_expired_wait_in_the_tensor_copy_kernels(pk):
    """The same give-up path in the kernels that stage rows by tensor copies (rotating forward, its consumers,
    the wide-row sites with one and with three warps per row, where the warps of a row decide together):
    every call returns 0, every record carries HYC_STATUS_WAIT_EXPIRED, nothing is written outside the
    outputs, and the next ordinary calls are exact."""
    import ctypes as C
    from hyc_lora_b200 import _lib
    rows = 96
    pk.reset_status()
    cases = []
    for d, rotate in ((4096, 256), (11008, 64)):
        x, _ = synthetic.sweep_activation(rows, d, 0.01, dtype=torch.bfloat16, salt=d)
        xd = (0.25 * x).to(DEV)
        ch = pk.select_channels(pk.channel_absmax(xd), oc.n_outlier_count(d, 0.01))
        cases.append((d, rotate, xd, ch))
    d0, r0, x0, ch0 = cases[0]
    w = synthetic.norm_weight(d0, 0.1, dtype=torch.bfloat16).to(DEV)
    good = pk.compress_n(x0, ch0, 4, 0, r0)
    want_dec = pk.decompress(good).reshape(rows, d0).clone()
    dy = torch.randn(rows, d0, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    rstd = torch.ones(rows, device=DEV)
    want_dx, _, _ = pk.norm_bwd(good, dy, w, rstd, None, "rms")
    arena = _Arena(rows * 11008 * 16 + (1 << 20))
    flagged = []
    assert _lib.lib.hyc_debug_wait(2_000_000, 16) == 0
    try:
        # rotating forward with the norm fused, and the norm backward of a rotated record
        pa = _packed_n_in(arena, pk, rows, d0, 4, 0, r0, ch0)
        y, rs_ = arena.take((rows, d0), torch.bfloat16), arena.take((rows,), torch.float32)
        n = _lib.HycNormFwd()
        n.kind, n.eps = pk._NORM_KIND["rms"], 1e-5
        n.weight, n.bias, n.param_dtype = w.data_ptr(), None, _lib.HYC_BF16
        n.y, n.rstd, n.mean = y.data_ptr(), rs_.data_ptr(), None
        ra, dn = pa.record(), _dense(x0, d0)
        rcs = [_lib.lib.hyc_norm_compress(C.byref(dn), C.byref(n), C.byref(ra), pk._stream())]
        flagged.append(pa)
        dx = arena.take((rows, d0), torch.bfloat16)
        a = _lib.HycNormBwdArgs()
        a.kind, a.ref_compat_c2 = _lib.HYC_NORM_RMS, 1
        a.weight, a.param_dtype, a.dy, a.dy_dtype = w.data_ptr(), _lib.HYC_BF16, dy.data_ptr(), _lib.HYC_BF16
        a.rstd, a.mean, a.dx = rstd.data_ptr(), None, dx.data_ptr()
        rg = good.record()
        rcs.append(_lib.lib.hyc_norm_bwd(C.byref(rg), C.byref(a), pk._stream()))
        flagged.append(good)
        # the one-pass sites, one warp per row and three warps per row
        for d, rotate, xd, ch in cases:
            px = _packed_n_in(arena, pk, rows, d, 4, 0, rotate, ch)
            py = _packed_n_in(arena, pk, rows, d, 4, 0, rotate, ch)
            out = arena.take((rows, d), torch.bfloat16)
            rx, ry, dd = px.record(), py.record(), _dense(xd, d)
            rcs.append(_lib.lib.hyc_act_compress(C.byref(dd), _lib.HYC_ACT_SILU, out.data_ptr(), C.byref(rx), C.byref(ry), pk._stream()))
            rcs.append(_lib.lib.hyc_product_compress(C.byref(dd), C.byref(dd), out.data_ptr(), C.byref(rx), C.byref(ry), pk._stream()))
            flagged.append(px)
        torch.cuda.synchronize()
    finally:
        assert _lib.lib.hyc_debug_wait(0, 0) == 0
    assert rcs == [0] * len(rcs)
    for p in flagged:
        assert p.wait_expired()
    arena.check()
    with pytest.raises(RuntimeError, match="WAIT_EXPIRED"):
        pk.poll_status(wait=True)
    good.status.zero_()
    pk.reset_status()
    again = pk.compress_n(x0, ch0, 4, 0, r0)
    assert torch.equal(again.codes, good.codes) and torch.equal(pk.decompress(good).reshape(rows, d0), want_dec)
    assert torch.equal(pk.norm_bwd(good, dy, w, rstd, None, "rms")[0], want_dx)
    assert pk.act_compress_n("silu", cases[1][2], cases[1][3], 4, 0, 64) is not None
    assert not good.wait_expired() and pk.poll_status(wait=True) == 0


def test_expired_wait_is_reported_and_leaves_the_device_usable(pk):
    """The give-up path of the bounded waits, made to run without any fault: through the test hook every
    staged row of the consumer kernels announces 16 bytes more than it copies and waits end after about a
    millisecond.  All copies land, no barrier ever completes, every CTA gives up: the call returns 0, the
    record's status word carries HYC_STATUS_WAIT_EXPIRED, nothing is written outside the outputs, the
    poll raises, and the very next ordinary call is exact."""
    import ctypes as C
    from hyc_lora_b200 import _lib
    rows, d = 64, 1024
    x, _ = synthetic.sweep_activation(rows, d, 0.01, salt=77)
    xd = x.to(DEV)
    ch = pk.select_channels(pk.channel_absmax(xd), oc.n_outlier_count(d, 0.01))
    pk.reset_status()
    p = pk.compress_n(xd, ch, 4, 0, 0)
    want = pk.decompress(p).reshape(rows, d).clone()
    dy = torch.randn(rows, d, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    arena = _Arena(rows * d * 8 + (1 << 18))
    xh, dx = arena.take((rows, d), torch.bfloat16), arena.take((rows, d), torch.bfloat16)
    assert _lib.lib.hyc_debug_wait(2_000_000, 16) == 0
    try:
        rec, out = p.record(), _dense(xh, d)
        rc1 = _lib.lib.hyc_decompress(C.byref(rec), C.byref(out), pk._stream())
        rc2 = _lib.lib.hyc_act_bwd(_lib.HYC_ACT_SILU, C.byref(rec), None, C.c_void_p(dy.data_ptr()), _lib.HYC_BF16,
                                   C.c_void_p(dx.data_ptr()), None, pk._stream())
        torch.cuda.synchronize()
    finally:
        assert _lib.lib.hyc_debug_wait(0, 0) == 0
    assert rc1 == 0 and rc2 == 0
    assert p.wait_expired()
    arena.check()
    with pytest.raises(RuntimeError, match="WAIT_EXPIRED"):
        pk.poll_status(wait=True)
    p.status.zero_()
    pk.reset_status()
    assert torch.equal(pk.decompress(p).reshape(rows, d), want)
    assert not p.wait_expired() and pk.poll_status(wait=True) == 0
    assert _lib.lib.hyc_debug_wait(-1, 0) == -2 and _lib.lib.hyc_debug_wait(0, 8) == -2


def test_weight_gradient_added_to_a_gradient_buffer(pk):
    """hyc_lora_wgrad_to with accumulate: what the buffer held plus the fp32 sums, rounded once (bf16 and fp32)."""
    rows, d, rank = 700, 4096, 16
    x, _ = synthetic.sweep_activation(rows, d, 0.01, salt=3)
    g = torch.randn(rows, rank, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    ch = oc.n_select_channels(oc.n_channel_scores(x), oc.n_outlier_count(d, 0.01))
    p = pk.compress_n(x.to(DEV), ch.to(DEV), 4, 0, 256)
    dw = pk.lora_wgrad(p, g)
    for dtype in (torch.bfloat16, torch.float32):
        base = torch.randn(rank, d, device=DEV).to(dtype)
        buf = base.clone()
        out = pk.lora_wgrad(p, g, accumulate_into=buf)
        assert out.data_ptr() == buf.data_ptr()
        assert torch.equal(buf, (base.float() + dw).to(dtype))
