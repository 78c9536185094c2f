"""Host side of the compression core, with the reference's function names.

Mirrors ``operators/compress_function.py`` of the reference: the same callables
with the same argument meaning, so the operator modules read like the
reference's.  The work itself is done by the CUDA library through
:mod:`hyc_lora_b200.packed`; nothing here runs on CPU tensors.

  get_statistics                              <- compress_function.py:292-340
  true_divide_outlier_suboutlier_svd_compress <- :136-200
  true_divide_outlier_suboutlier_svd_decompress <- :203-261
  true_compress_softmax / true_decompress_softmax / get_statistics_softmax <- :264-275, :343-347
  pad_cut_L, head_to_hidden_shape, hidden_to_head_shape <- :350-360, :4-12

Differences a caller can see:
  * the first value returned by the compress call is a :class:`Packed` record
    (pooled element outliers or channel outliers) instead of a sparse COO tensor;
  * calibration (the first two calls of a site) uses torch ops on the device, as
    the reference does; steady-state calls launch one kernel and never
    synchronise with the host.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import packed as _pk
from ..packed import Packed

BF16 = torch.bfloat16


class StaticList(list):
    """``static_value`` of a module: the reference's four-slot list
    ``[threshold, L, scale, R]`` plus a cache for the low-rank product, which
    only changes while the site calibrates."""

    def __init__(self, values=(None, None, None, None)):
        super().__init__(values)
        self.cache = {}


def hidden_to_head_shape(x: torch.Tensor, num_heads: int):
    bsz, seq_len, hidden = x.shape
    return x.reshape(bsz, seq_len, num_heads, hidden // num_heads).transpose(1, 2)


def head_to_hidden_shape(x: torch.Tensor):
    bsz, num_heads, seq_len, head_dim = x.shape
    return x.transpose(1, 2).reshape(bsz, seq_len, -1)


@torch.no_grad()
def pad_cut_L(src_L: torch.Tensor, tgt_L) -> torch.Tensor:
    """Zero-pad or truncate the rows of ``src_L`` to the row count of ``tgt_L``
    (a tensor or an int)."""
    rows = tgt_L if isinstance(tgt_L, int) else tgt_L.shape[0]
    n, r = src_L.shape
    if n < rows:
        src_L = torch.cat((src_L, torch.zeros(rows - n, r, dtype=src_L.dtype, device=src_L.device)), dim=0)
    elif n > rows:
        src_L = src_L[:rows]
    return src_L.contiguous()


@torch.no_grad()
def get_statistics(x: torch.Tensor, iteration: int, outlier_ratio: float, sub_outlier_ratio: float,
                   sub_outlier_bit: int = 8, sub_outlier_quantize_method: str = "per-tensor", svd_rank: int = 16):
    """Calibration from batch element 0, the reference's procedure op for op:
    optional rank-``svd_rank`` randomized SVD (L = U, R = diag(S) V^T), the
    SIGNED ``1 - ratio`` quantile as threshold, the min-max range of the
    outlier-free residual over ``2^bits - 1`` as scale.  Returns
    ``(threshold fp32 0-dim, L bf16, R bf16, scale bf16)`` on x's device."""
    if x.dim() == 4:
        x = head_to_hidden_shape(x)
    if svd_rank > 0:
        u, s, v = torch.svd_lowrank(x[0].to(torch.float32), q=svd_rank, niter=16)
        left = u.contiguous()
        right = (torch.diag(s) @ v.T).contiguous()
        x = x - left @ right
    else:
        left = torch.zeros((x.shape[-2], 16), device=x.device, dtype=x.dtype)
        right = torch.zeros((16, x.shape[-1]), device=x.device, dtype=x.dtype)
    first = x[0]
    thr = torch.kthvalue(first.flatten().to(torch.float32), int(first.numel() * (1 - outlier_ratio))).values
    removed = (first * (first.abs() > thr)).to(BF16)
    x = x - removed
    if sub_outlier_ratio > 0 and sub_outlier_bit != 16:
        body = x[0]
        levels = 2 ** sub_outlier_bit - 1
        if sub_outlier_quantize_method == "per-tensor":
            scale = (body.max() - body.min()) / levels
        elif sub_outlier_quantize_method == "per-channel":
            scale = (body.max(dim=-2, keepdim=True).values - body.min(dim=-2, keepdim=True).values) / levels
        elif sub_outlier_quantize_method == "per-token":
            scale = (body.max(dim=-1, keepdim=True).values - body.min(dim=-1, keepdim=True).values) / levels
        else:
            raise ValueError(f"Unsupport Quantize Method {sub_outlier_quantize_method!r}")
    else:
        scale = torch.tensor(1.0, device=x.device)
    return thr, left.to(BF16), right.to(BF16), scale.to(BF16)


@torch.no_grad()
def lowrank_product(L: Optional[torch.Tensor], R: Optional[torch.Tensor], seq: int, rank, cache=None):
    """bf16 [seq, D] product ``pad_cut_L(L) @ R`` the kernels subtract / add, or
    None when the site has no low-rank part (``rank == 0``).  The product is a
    small library GEMM; it is cached while L and R are the same tensors."""
    if rank == 0 or L is None or R is None:
        return None
    # the entry is valid for these very tensor objects (held weakly: a new tensor that happens to reuse a freed
    # tensor's address never matches), unmodified since
    key = (L._version, R._version, seq)
    if cache is not None and cache.get("key") == key:
        refs = cache.get("refs")
        if refs is not None and refs[0]() is L and refs[1]() is R:
            return cache["value"]
    value = (pad_cut_L(L, seq) @ R).to(BF16).contiguous()
    if cache is not None:
        import weakref
        cache["key"], cache["value"], cache["refs"] = key, value, (weakref.ref(L), weakref.ref(R))
    return value


# a finite scale so large that every code is the zero code: used when a site keeps outliers only
_NOTHING_QUANTISED = 3.0e38


@torch.no_grad()
def true_divide_outlier_suboutlier_svd_compress(x: torch.Tensor, outlier, scale, sub_outlier_bit: int = 8,
                                                sub_outlier_ratio: float = 1.0, L: torch.Tensor = None,
                                                R: torch.Tensor = None, rank=None, cache=None,
                                                outlier_ratio: float = 0.01, norm: Optional[dict] = None):
    """Reference-mode compression of ``x`` ([B,S,D] or [B,H,S,hd]).  Returns
    ``(x_outlier_compressed, x_sub_outlier_compressed, scale)`` like the
    reference: here the first is the :class:`Packed` record and the second its
    packed-code tensor.  With ``norm`` the norm forward is fused and
    ``(y, rstd, mean)`` are appended."""
    assert sub_outlier_bit in [1, 2, 4, 8, 16], "Only support 1,2,4,8,16 bit quantization"
    if sub_outlier_bit == 16:
        raise NotImplementedError("16-bit sub-outliers leave the reference's result unbound "
                                  "(compress_function.py:167-168,200); use 1, 2, 4 or 8 bits")
    seq = x.shape[-2]
    lowrank = lowrank_product(L, R, seq, rank, cache)
    # Outlier-pool capacity.  With frozen statistics (``cache`` is the site's, i.e. from the third call on)
    # the site counts once how many elements its threshold actually selects and sizes its pool from that:
    # one host synchronisation per site (the reference synchronises on every call, in to_sparse).
    density = None
    if cache is not None:
        density = cache.get("pool_density")
        if density is None and not torch.cuda.is_current_stream_capturing():
            resid = head_to_hidden_shape(x) if x.dim() == 4 else x
            if lowrank is not None:
                resid = resid - lowrank
            density = float((resid.abs() > outlier).float().mean().item())
            cache["pool_density"] = density
    if sub_outlier_ratio == 0.0:
        use_scale = torch.full((), _NOTHING_QUANTISED, device=x.device, dtype=BF16)
        bits = 8 if sub_outlier_bit == 16 else sub_outlier_bit
        out_scale = torch.tensor(1.0, device=x.device)
    else:
        use_scale, bits, out_scale = scale, sub_outlier_bit, scale
    res = _pk.compress_r(x, outlier, use_scale, bits, lowrank=lowrank, outlier_ratio=outlier_ratio, norm=norm,
                         density=density)
    if norm is None:
        p = res
        return p, p.codes.view(p.shape[0], p.shape[1], -1), out_scale
    p, y, rstd, mean = res
    return p, p.codes.view(p.shape[0], p.shape[1], -1), out_scale, y, rstd, mean


@torch.no_grad()
def true_divide_outlier_suboutlier_svd_decompress(x_outlier_compressed: Packed, x_sub_outlier_compressed,
                                                  sub_outlier_bit, scale, is_head: bool = False, num_heads: int = 1,
                                                  L=None, R=None):
    """bf16 reconstruction ([B,S,D], or [B,H,S,hd] with ``is_head``).  The
    record already carries codes, scale and the low-rank product, so the other
    arguments are accepted for signature compatibility only."""
    return _pk.decompress(x_outlier_compressed, num_heads=num_heads if is_head else 0)


@torch.no_grad()
def get_statistics_softmax(x: torch.Tensor, iteration: int, outlier_ratio: float):
    first = x[0].float().flatten()
    return torch.kthvalue(first, int(first.numel() * (1 - outlier_ratio))).values


@torch.no_grad()
def true_compress_softmax(x: torch.Tensor, outlier, outlier_ratio: Optional[float] = None):
    """Keep the probabilities above the threshold as a compact per-row list.  The list's
    capacity is twice the calibrated fraction (plus slack); rows that do not fit keep
    nothing and raise the overflow flag of the record."""
    cap = 0.125 if outlier_ratio is None else min(1.0, 2.0 * outlier_ratio + 0.02)
    return _pk.softmax_compact(x, outlier, capacity_ratio=cap)


@torch.no_grad()
def true_decompress_softmax(x_sparse):
    """Dense tensor with zeros where nothing was kept."""
    return _pk.softmax_expand(x_sparse)


# ---------------------------------------------------------------------------
# channel mode (no counterpart in the reference)
# ---------------------------------------------------------------------------


def outlier_channel_count(cols: int, ratio: float) -> int:
    return int(math.ceil(ratio * cols - 1e-9)) if ratio > 0 else 0


class ChannelCalibration:
    """Calibration state of a channel-mode site, following the reference's
    protocol for its own statistics (running mean over the first two calls,
    frozen afterwards, efficient_linear.py:122-146): the statistic is the fp32
    column-absmax vector; calls 0 and 1 use the channels of the fresh vector,
    later calls the channels of the averaged one."""

    def __init__(self, outlier_ratio: float):
        self.outlier_ratio = outlier_ratio
        self.score = None
        self.channels = None

    @torch.no_grad()
    def channels_for(self, x: torch.Tensor, iteration: int) -> Optional[torch.Tensor]:
        cols = x.shape[-1] if x.dim() != 4 else x.shape[1] * x.shape[3]
        k = outlier_channel_count(cols, self.outlier_ratio)
        if k == 0:
            return None
        if iteration >= 2 and self.channels is not None:
            return self.channels
        fresh = _pk.channel_absmax(x)
        self.score = fresh if self.score is None else (iteration * self.score + fresh) / (iteration + 1)
        self.channels = _pk.select_channels(self.score, k)
        return _pk.select_channels(fresh, k) if iteration < 2 else self.channels


@torch.no_grad()
def channel_compress(x: torch.Tensor, channels, bits: int, group_size: int = 0, rotate: int = 0,
                     norm: Optional[dict] = None, also_output: Optional[dict] = None):
    """Channel-mode compression; see :func:`hyc_lora_b200.packed.compress_n`."""
    return _pk.compress_n(x, channels, bits, group_size, rotate, norm=norm, also_output=also_output)
