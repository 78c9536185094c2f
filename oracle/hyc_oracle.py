"""CPU oracle for the HyC-LoRA activation compress / decompress+grad hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
it is the checker used by the tests, by the smoke entry and by the CPU leg of
the benchmark.  Everything here is plain PyTorch on CPU tensors.

Two semantic modes are restated:

* ``r_*`` functions ("reference mode") restate, operation by operation and
  with the same dtype promotion points, what the reference does in
  ``operators/compress_function.py``:
    - ``r_calibrate``      <- get_statistics            (compress_function.py:292-340)
    - ``r_compress``       <- true_divide_outlier_suboutlier_svd_compress (:136-200)
    - ``r_decompress``     <- true_divide_outlier_suboutlier_svd_decompress (:203-261)
    - ``r_softmax_*``      <- true_compress_softmax / true_decompress_softmax /
                              get_statistics_softmax   (:264-275, :343-347)
    - ``fit_rows``         <- pad_cut_L                 (:350-360)
  Parity of these against the imported reference is pinned by
  ``tests/test_oracle_pin.py`` (when the reference tree is present) and by the
  fixtures under ``tests/golden/`` (always).

* ``n_*`` functions ("north-star mode") define the channel-top-k / dynamic
  absmax / group-128 / Walsh-Hadamard variant, which has no counterpart in the
  reference.  Parity of that mode is therefore UNPINNED against the reference;
  it reuses the reference's rounding (half-to-even), clamp range
  ``[-2^(b-1), 2^(b-1)-1]``, offset-binary codes and segment packing
  (compress_function.py:170-197) so one pack/unpack routine serves both modes.

The norm / activation / linear gradient formulas restate
``operators/efficient_rmsnorm.py:40-60,92-108``,
``operators/efficient_layernorm.py:33-62,131-148``,
``operators/efficient_silu.py:50-51``, ``operators/efficient_gelu.py:49-62``,
``operators/efficient_hadamard.py:62-66``, ``operators/efficient_softmax.py:35-45``
and ``operators/efficient_linear.py:61-69``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

BF16 = torch.bfloat16

# --------------------------------------------------------------------------
# code packing shared by both modes
# --------------------------------------------------------------------------


def pack_codes(u: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack offset-binary codes ``u`` (integers in [0, 2^bits), last dim D)
    into bytes.  The row is cut into ``8/bits`` contiguous segments of
    ``D*bits/8`` channels; byte ``j`` holds channel ``j`` of every segment,
    segment ``s`` in bit field ``s*bits`` (compress_function.py:177-197).
    8-bit codes are stored as two's-complement int8 without offset (:176)."""
    if bits == 8:
        return u.to(torch.int8)
    nseg = 8 // bits
    d = u.shape[-1]
    assert d % nseg == 0
    seg = u.to(torch.int32).reshape(*u.shape[:-1], nseg, d // nseg)
    shifts = (torch.arange(nseg, dtype=torch.int32) * bits).reshape(nseg, 1)
    return (seg << shifts).sum(dim=-2).to(torch.uint8)


def unpack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Inverse of :func:`pack_codes`; returns int32 codes with last dim D
    (for 8 bits: the signed values themselves)."""
    if bits == 8:
        return codes.to(torch.int32)
    nseg = 8 // bits
    c = codes.to(torch.int32).unsqueeze(-2)
    shifts = (torch.arange(nseg, dtype=torch.int32) * bits).reshape(nseg, 1)
    seg = (c >> shifts) & ((1 << bits) - 1)
    return seg.reshape(*codes.shape[:-1], nseg * codes.shape[-1])


def heads_to_rows(x: torch.Tensor) -> torch.Tensor:
    """[B,H,S,hd] -> [B,S,H*hd] (compress_function.py:10-12)."""
    b, h, s, hd = x.shape
    return x.transpose(1, 2).reshape(b, s, h * hd)


def rows_to_heads(x: torch.Tensor, num_heads: int) -> torch.Tensor:
    """[B,S,D] -> [B,H,S,D/H] (compress_function.py:4-7)."""
    b, s, d = x.shape
    return x.reshape(b, s, num_heads, d // num_heads).transpose(1, 2)


def fit_rows(src: torch.Tensor, rows: int) -> torch.Tensor:
    """Zero-pad or truncate the leading dim of ``src`` to ``rows``
    (compress_function.py:350-360)."""
    n = src.shape[0]
    if n < rows:
        pad = torch.zeros(rows - n, src.shape[1], dtype=src.dtype)
        src = torch.cat([src, pad], dim=0)
    elif n > rows:
        src = src[:rows]
    return src.contiguous()


# --------------------------------------------------------------------------
# reference mode
# --------------------------------------------------------------------------


@dataclass
class RCompressed:
    """What the reference keeps for backward at one site."""
    out_index: torch.Tensor   # int64 [3, nnz] (b, s, d), row-major sorted
    out_value: torch.Tensor   # bf16 [nnz]
    codes: Optional[torch.Tensor]  # uint8 / int8 [B,S,D*bits/8], None if nothing quantised
    scale: torch.Tensor
    bits: int
    shape: tuple


@torch.no_grad()
def r_calibrate(x: torch.Tensor, outlier_ratio: float, sub_outlier_ratio: float,
                bits: int, method: str, rank: int, svd_seed: Optional[int] = None):
    """Statistics from batch element 0 (compress_function.py:292-340).

    Returns ``(thr fp32 0-dim, L bf16 [S,r], R bf16 [r,D], scale bf16)``.
    ``scale`` is 0-dim (per-tensor), [1,D] (per-channel) or [S,1] (per-token)
    and is the min-max range of the outlier-free residual divided by
    ``2^bits-1``.  The threshold is the SIGNED quantile of x[0] (:319) that is
    later compared against ``abs`` (:320)."""
    if x.dim() == 4:
        x = heads_to_rows(x)
    if rank > 0:
        if svd_seed is not None:
            torch.manual_seed(svd_seed)
        u, s, v = torch.svd_lowrank(x[0].float(), q=rank, niter=16)
        left = u.contiguous()
        right = (torch.diag(s) @ v.T).contiguous()
        x = x - left @ right
    else:
        left = torch.zeros(x.shape[-2], 16, dtype=x.dtype)
        right = torch.zeros(16, x.shape[-1], dtype=x.dtype)
    first = x[0]
    kth = int(first.numel() * (1 - outlier_ratio))
    thr = torch.kthvalue(first.flatten().float(), kth).values
    removed = (first * (first.abs() > thr)).to(BF16)
    x = x - removed
    if sub_outlier_ratio > 0 and bits != 16:
        body = x[0]
        levels = 2 ** bits - 1
        if method == "per-tensor":
            scale = (body.max() - body.min()) / levels
        elif method == "per-channel":
            scale = (body.max(dim=-2, keepdim=True).values - body.min(dim=-2, keepdim=True).values) / levels
        elif method == "per-token":
            scale = (body.max(dim=-1, keepdim=True).values - body.min(dim=-1, keepdim=True).values) / levels
        else:
            raise ValueError(f"unknown quantize method {method!r}")
    else:
        scale = torch.tensor(1.0)
    return thr, left.to(BF16), right.to(BF16), scale.to(BF16)


@torch.no_grad()
def r_compress(x: torch.Tensor, thr: torch.Tensor, scale: torch.Tensor, bits: int,
               sub_outlier_ratio: float = 1.0, left: Optional[torch.Tensor] = None,
               right: Optional[torch.Tensor] = None) -> RCompressed:
    """Low-rank subtract, threshold split, quantise and pack
    (compress_function.py:136-200).  All arithmetic runs in the dtype torch's
    promotion gives the reference: with bf16 ``x`` the subtraction, the
    threshold compare and the division round to bf16; with fp32 ``x`` they are
    fp32."""
    if x.dim() == 4:
        x = heads_to_rows(x)
    if left is not None:
        x = x - fit_rows(left, x.shape[-2]) @ right
    big = x.abs() > thr
    picked = x * big
    x = x - picked
    coo = picked.to(BF16).to_sparse().coalesce()
    codes = None
    if sub_outlier_ratio != 0.0:
        assert bits in (1, 2, 4, 8)
        half = 2 ** (bits - 1)
        q = torch.clamp(torch.round(x / scale), min=-half, max=half - 1)
        if bits == 8:
            codes = pack_codes(q, 8)
        else:
            codes = pack_codes((q + half).to(torch.uint8), bits)
    return RCompressed(coo.indices(), coo.values(), codes, scale, bits, tuple(x.shape))


@torch.no_grad()
def r_decompress(c: RCompressed, left: Optional[torch.Tensor] = None,
                 right: Optional[torch.Tensor] = None, num_heads: int = 0) -> torch.Tensor:
    """bf16 reconstruction (compress_function.py:203-261): low-rank base
    (bf16) + outliers (bf16 add) + dequantised codes (bf16 multiply, bf16
    add)."""
    b, s, d = c.shape
    dense = torch.zeros(c.shape, dtype=BF16)
    dense[c.out_index[0], c.out_index[1], c.out_index[2]] = c.out_value
    if left is not None:
        base = (fit_rows(left, s) @ right).to(BF16)
    else:
        base = torch.zeros(s, d, dtype=BF16)
    x = base + dense
    if c.codes is not None:
        u = unpack_codes(c.codes, c.bits)
        half = 0 if c.bits == 8 else 2 ** (c.bits - 1)
        x = x + (u.to(BF16) - half) * c.scale
    if num_heads:
        x = rows_to_heads(x, num_heads)
    return x


@torch.no_grad()
def r_softmax_threshold(y: torch.Tensor, outlier_ratio: float) -> torch.Tensor:
    """Quantile of the probabilities of batch element 0
    (compress_function.py:343-347)."""
    first = y[0].float().flatten()
    return torch.kthvalue(first, int(first.numel() * (1 - outlier_ratio))).values


@torch.no_grad()
def r_softmax_keep(y: torch.Tensor, thr: torch.Tensor) -> torch.Tensor:
    """Dense view of what the sparse softmax copy keeps: entries ``> thr``,
    zero elsewhere (compress_function.py:264-275)."""
    return y * (y > thr)


# --------------------------------------------------------------------------
# north-star mode (no reference counterpart: parity unpinned)
# --------------------------------------------------------------------------

ROTATE_BLOCKS = (16, 64, 256, 1024, 4096)  # even powers of two: 1/sqrt(n) is exact


def n_outlier_count(d: int, ratio: float) -> int:
    """Number of full-precision channels: ceil(ratio * D)."""
    return int(math.ceil(ratio * d - 1e-9)) if ratio > 0 else 0


@torch.no_grad()
def n_channel_scores(x: torch.Tensor) -> torch.Tensor:
    """fp32 column absmax over every row of ``x`` ([..., D])."""
    return x.reshape(-1, x.shape[-1]).float().abs().amax(dim=0)


@torch.no_grad()
def n_select_channels(score: torch.Tensor, k: int) -> torch.Tensor:
    """The ``k`` channels of largest score, ties to the lower index, returned
    as an ascending int32 list."""
    # a stable descending sort orders by (-score, index)
    idx = torch.sort(score.float(), descending=True, stable=True).indices[:k]
    return torch.sort(idx).values.to(torch.int32)


@torch.no_grad()
def fwht_blocks(x: torch.Tensor, n: int) -> torch.Tensor:
    """Normalised Walsh-Hadamard transform of every aligned block of ``n``
    channels, natural (Sylvester) order, fp32.  Butterflies run with strides
    1, 2, 4, ... ; at each stage the lower element becomes ``a+b`` and the
    upper ``a-b``; the result is multiplied once by the exact power of two
    ``1/sqrt(n)``.  The transform is its own inverse."""
    assert n in ROTATE_BLOCKS and x.shape[-1] % n == 0
    shp = x.shape
    v = x.float().reshape(-1, n)
    h = 1
    while h < n:
        v = v.reshape(-1, n // (2 * h), 2, h)
        a = v[:, :, 0, :]
        b = v[:, :, 1, :]
        v = torch.stack((a + b, a - b), dim=2).reshape(-1, n)
        h *= 2
    return (v * (1.0 / math.sqrt(n))).reshape(shp)


@dataclass
class NCompressed:
    codes: torch.Tensor      # uint8 (int8 for 8 bits) [T, D*bits/8]
    scales: torch.Tensor     # fp32 [T, G]
    out_value: torch.Tensor  # bf16 [T, k]
    channels: torch.Tensor   # int32 [k], ascending
    bits: int
    group: int               # 0 = one scale per row, else channels per group
    rotate: int              # 0 = off, else FWHT block size
    cols: int


@torch.no_grad()
def n_compress(x: torch.Tensor, channels: torch.Tensor, bits: int, group: int = 0,
               rotate: int = 0) -> NCompressed:
    """Channel-outlier split, optional rotation, dynamic absmax quantisation.

    ``x`` is [T, D] (fp32 or bf16).  Outlier channels are kept as bf16 and
    zeroed in place; the remainder is (optionally) rotated in fp32; the scale
    of a row / 128-channel group is ``absmax / qmax`` with
    ``qmax = 2^(bits-1) - 1`` and the code is
    ``clamp(rint(x * (qmax / absmax)))`` -- the reciprocal is one IEEE fp32
    division and the product is rounded to an integer once, from its exact
    value, so CPU and GPU agree bit for bit on finite inputs (codes of rows
    holding inf/NaN are unspecified).  A zero absmax gives scale 1 and codes 0."""
    assert bits in (2, 4, 8) and x.dim() == 2
    t, d = x.shape
    half = 2 ** (bits - 1)
    qmax = float(half - 1)
    idx = channels.long()
    out_value = x[:, idx].to(BF16)
    v = x.float().clone()
    v[:, idx] = 0.0
    if rotate:
        v = fwht_blocks(v, rotate)
    g = d if group == 0 else group
    assert d % g == 0
    vg = v.reshape(t, d // g, g)
    amax = vg.abs().amax(dim=-1)
    live = amax > 0
    one = torch.ones_like(amax)
    scales = torch.where(live, amax / qmax, one)
    inv = torch.where(live, torch.tensor(qmax) / amax, one)
    # the product is rounded ONCE, from its exact value (fp32 x fp32 is exact in fp64),
    # which is what a fused multiply-add against a rounding constant computes on the GPU
    prod = vg.double() * inv.unsqueeze(-1).double()
    q = torch.clamp(torch.round(prod), min=-half, max=half - 1).reshape(t, d)
    q = torch.nan_to_num(q, nan=0.0).float()
    if bits == 8:
        codes = pack_codes(q, 8)
    else:
        codes = pack_codes((q + half).to(torch.uint8), bits)
    return NCompressed(codes, scales.contiguous(), out_value.contiguous(),
                       channels.to(torch.int32), bits, group, rotate, d)


@torch.no_grad()
def n_decompress(c: NCompressed) -> torch.Tensor:
    """bf16 [T, D]: ``(code - offset) * scale`` in fp32, inverse rotation in
    fp32, one rounding to bf16, then the stored outlier channels."""
    u = unpack_codes(c.codes, c.bits)
    half = 0 if c.bits == 8 else 2 ** (c.bits - 1)
    t, d = u.shape
    g = d if c.group == 0 else c.group
    v = ((u - half).float().reshape(t, d // g, g) * c.scales.unsqueeze(-1)).reshape(t, d)
    if c.rotate:
        v = fwht_blocks(v, c.rotate)
    out = v.to(BF16)
    out[:, c.channels.long()] = c.out_value
    return out


# --------------------------------------------------------------------------
# norm forward / backward (restating the reference's Triton kernels)
# --------------------------------------------------------------------------


@torch.no_grad()
def norm_forward(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                 eps: float, kind: str):
    """``kind`` in {"rms", "rms_gemma", "ln"}.  fp32 math, output in x's dtype;
    returns ``(y, mean fp32 [M] or None, rstd fp32 [M])``
    (efficient_rmsnorm.py:40-60, efficient_rmsnorm_gemma.py:59,
    efficient_layernorm.py:33-62)."""
    xf = x.reshape(-1, x.shape[-1]).float()
    w = weight.float()
    if kind == "ln":
        mean = xf.mean(dim=-1)
        xc = xf - mean[:, None]
        rstd = 1.0 / torch.sqrt((xc * xc).mean(dim=-1) + eps)
        y = xc * rstd[:, None] * w + bias.float()
    else:
        mean = None
        rstd = 1.0 / torch.sqrt((xf * xf).mean(dim=-1) + eps)
        if kind == "rms_gemma":
            w = w + 1.0
        y = xf * rstd[:, None] * w
    return y.to(x.dtype).reshape(x.shape), mean, rstd


@torch.no_grad()
def norm_backward(x_hat_input: torch.Tensor, dy: torch.Tensor, weight: torch.Tensor,
                  mean: Optional[torch.Tensor], rstd: torch.Tensor, kind: str,
                  ref_compat_c2: bool = True):
    """dx (bf16) and dw (fp32 here) from the DECOMPRESSED input
    (efficient_rmsnorm.py:92-108, efficient_layernorm.py:131-148).  ``dy`` is
    cast to bf16 first (efficient_rmsnorm.py:216).  With ``ref_compat_c2`` the
    RMSNorm backward keeps the reference's mean(w*dy) term (:103-104), which a
    true RMSNorm gradient does not have.  The reference accumulates dw in bf16
    buffers in lock order; this oracle sums in fp32."""
    d = x_hat_input.shape[-1]
    xf = x_hat_input.reshape(-1, d).float()
    g = dy.to(BF16).reshape(-1, d).float()
    w = weight.float()
    if kind == "rms_gemma":
        w = w + 1.0
    if kind == "ln":
        xn = (xf - mean[:, None]) * rstd[:, None]
    else:
        xn = xf * rstd[:, None]
    wdy = w * g
    c1 = (xn * wdy).mean(dim=-1, keepdim=True)
    if kind == "ln" or ref_compat_c2:
        c2 = wdy.mean(dim=-1, keepdim=True)
    else:
        c2 = torch.zeros_like(c1)
    dx = (wdy - (xn * c1 + c2)) * rstd[:, None]
    dw = (g * xn).sum(dim=0)
    db = g.sum(dim=0)
    return dx.to(BF16).reshape(dy.shape), dw, db


# --------------------------------------------------------------------------
# activation / product / softmax / linear backward
# --------------------------------------------------------------------------

GELU_GAMMA = math.sqrt(2.0 / math.pi)
GELU_KAPPA = 0.044715


@torch.no_grad()
def silu_backward(x_hat: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """sigma(x)(1 + x - x sigma(x)) g  (efficient_silu.py:50-51), fp32 math,
    output dtype = promote(bf16, g.dtype)."""
    x = x_hat.float()
    s = torch.sigmoid(x)
    return (s * (1 + x - x * s) * g.float()).to(torch.promote_types(x_hat.dtype, g.dtype))


@torch.no_grad()
def gelu_backward(x_hat: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """tanh-approximation GELU derivative (efficient_gelu.py:49-62)."""
    x = x_hat.float()
    t = torch.tanh(GELU_GAMMA * (x + GELU_KAPPA * x ** 3))
    d = 0.5 * ((1 + t) + x * ((1 - t * t) * GELU_GAMMA * (1 + 3 * GELU_KAPPA * x * x)))
    return (d * g.float()).to(torch.promote_types(x_hat.dtype, g.dtype))


@torch.no_grad()
def product_backward(x1_hat: torch.Tensor, x2_hat: torch.Tensor, g: torch.Tensor):
    """(g*x2, x1*g) (efficient_hadamard.py:62-66)."""
    dt = torch.promote_types(x1_hat.dtype, g.dtype)
    return (g.float() * x2_hat.float()).to(dt), (x1_hat.float() * g.float()).to(dt)


@torch.no_grad()
def softmax_backward(y_kept: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """(g - sum(g*y)) * y on the thresholded probabilities
    (efficient_softmax.py:41)."""
    return (g - (g * y_kept).sum(dim=-1, keepdim=True)) * y_kept


@torch.no_grad()
def linear_backward(x_hat: torch.Tensor, w: torch.Tensor, dy: torch.Tensor):
    """dX = dY W ; dW = sum_b dY_b^T X_b  (efficient_linear.py:64-67 plus the
    autograd engine's reduction of the batched [B,r,D] result to [r,D])."""
    dx = dy.to(w.dtype) @ w
    g = dy.to(x_hat.dtype)
    dw = (g.transpose(-2, -1) @ x_hat)
    if dw.dim() == 3:
        dw = dw.sum(dim=0)
    return dx, dw.to(w.dtype)
