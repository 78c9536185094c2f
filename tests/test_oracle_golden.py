"""The CPU oracle against the committed golden fixtures (made by the
reference's own code), and property tests of the north-star-mode oracle."""
import math

import pytest
import torch

from oracle import hyc_oracle as oc
from hyc_lora_b200 import synthetic
from tests import golden_io


@pytest.mark.parametrize("case", list(golden_io.small_cases()), ids=lambda c: c.name)
def test_small_fixture(case):
    left, right = (case.L, case.R) if case.rank else (None, None)
    c = oc.r_compress(case.x, case.thr, case.scale, case.bits, 1.0, left, right)
    assert torch.equal(c.codes, case.codes)
    assert torch.equal(c.out_index, case.coo_index)
    assert torch.equal(c.out_value, case.coo_value)
    assert torch.equal(oc.r_decompress(c, left, right), case.xhat)


def test_config1_fixture():
    g = golden_io.config1()
    x, planted = synthetic.roundtrip_activation()
    assert golden_io.sha_bits(x) == g.x_sha256
    assert torch.equal(planted, g.planted)
    thr, L, R, scale = oc.r_calibrate(x, 0.01, 1.0, 4, "per-token", 0)
    assert torch.equal(thr, g.thr) and torch.equal(scale, g.scale)
    c = oc.r_compress(x, thr, scale, 4, 1.0, L, R)
    assert torch.equal(c.codes, g.codes)
    flat = c.out_index[0] * (128 * 768) + c.out_index[1] * 768 + c.out_index[2]
    assert torch.equal(flat.int(), g.coo_flat) and torch.equal(c.out_value, g.coo_value)
    xh = oc.r_decompress(c, L, R)
    assert golden_io.sha_bits(xh) == g.xhat_sha256
    a, grad = synthetic.lora_a_problem()
    dx, da = oc.linear_backward(xh, a, grad)
    assert golden_io.sha_bits(dx) == g.dX_sha256
    assert torch.allclose(da, g.dA, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
def test_pack_unpack_identity(bits):
    g = torch.Generator().manual_seed(bits)
    lo, hi = (-128, 128) if bits == 8 else (0, 2 ** bits)
    u = torch.randint(lo, hi, (5, 7, 256), generator=g)
    packed = oc.pack_codes(u if bits == 8 else u.to(torch.uint8), bits)
    assert packed.shape[-1] == 256 * bits // 8
    assert torch.equal(oc.unpack_codes(packed, bits), u.int())


@pytest.mark.parametrize("n", oc.ROTATE_BLOCKS)
def test_fwht_is_orthogonal_involution(n):
    g = torch.Generator().manual_seed(n)
    x = torch.randn(3, 2 * n if n < 4096 else n, generator=g)
    y = oc.fwht_blocks(x, n)
    assert torch.allclose(oc.fwht_blocks(y, n), x, atol=1e-4)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
    # against the explicit Sylvester matrix on one block
    h = torch.ones(1, 1)
    while h.shape[0] < min(n, 64):
        h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
    if n <= 64:
        assert torch.allclose(y[:, :n], (x[:, :n] @ h) / math.sqrt(n), atol=1e-4)


def test_channel_selection_ties_and_order():
    score = torch.tensor([1.0, 5.0, 5.0, 0.5, 5.0, 2.0])
    assert oc.n_select_channels(score, 2).tolist() == [1, 2]
    assert oc.n_select_channels(score, 4).tolist() == [1, 2, 4, 5]
    assert oc.n_outlier_count(768, 0.01) == 8 and oc.n_outlier_count(4096, 0.01) == 41
    assert oc.n_outlier_count(4096, 0.005) == 21 and oc.n_outlier_count(4096, 0.02) == 82


@pytest.mark.parametrize("bits,group,rotate", [(4, 0, 0), (4, 128, 0), (2, 0, 256), (8, 128, 256), (4, 0, 1024)])
def test_n_mode_roundtrip_properties(bits, group, rotate):
    x, planted = synthetic.sweep_activation(64, 1024, 0.01, salt=bits)
    ch = oc.n_select_channels(oc.n_channel_scores(x), oc.n_outlier_count(1024, 0.01))
    assert set(planted.tolist()) <= set(ch.tolist()) or len(planted) > len(ch)
    c = oc.n_compress(x, ch, bits, group, rotate)
    assert c.codes.shape == (64, 1024 * bits // 8) and c.scales.shape == (64, 1 if group == 0 else 1024 // group)
    xh = oc.n_decompress(c)
    assert xh.dtype == torch.bfloat16
    # outlier channels are exact, the rest is within half a step per element (rotation: in norm)
    assert torch.equal(xh[:, ch.long()], x[:, ch.long()].to(torch.bfloat16))
    cos = torch.nn.functional.cosine_similarity(xh.float().flatten(), x.float().flatten(), dim=0)
    assert cos > {2: 0.85, 4: 0.985, 8: 0.9999}[bits]
    if not rotate:
        body = x.float().clone()
        body[:, ch.long()] = 0
        g = 1024 if group == 0 else group
        step = c.scales.repeat_interleave(g, dim=1)
        err = (xh.float() - x.float()).abs()
        err[:, ch.long()] = 0
        assert (err <= 0.5 * step * 1.01 + 0.01 * body.abs()).all()
    # idempotence: compressing the reconstruction reproduces the codes
    c2 = oc.n_compress(xh, ch, bits, group, rotate)
    if not rotate and bits >= 4:
        assert (c2.codes != c.codes).float().mean() < 0.02


def test_n_mode_zero_rows():
    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    c = oc.n_compress(x, torch.tensor([3, 9], dtype=torch.int32), 4, 128, 0)
    assert torch.equal(c.scales, torch.ones(4, 2))
    assert torch.equal(oc.n_decompress(c), x)
