"""Pieces shared by the ``EfficientMemory*`` modules: the calibration running
mean of the reference, the options of the channel mode and the one helper that
compresses an activation for backward in either mode."""
from __future__ import annotations

import weakref
from typing import Optional

import torch

from . import compress_function as cf
from .compress_function import StaticList


class SiteOptions:
    """Options the reference does not have.  ``outlier_mode="element"`` (default)
    is the reference's arithmetic; ``"channel"`` keeps the top ``outlier_ratio``
    absmax channels in bf16, quantises the rest with a dynamic absmax scale per
    token (``group_size=0``) or per 128 channels, optionally after a block
    Walsh-Hadamard rotation (``rotate`` = block size).

    The rotation kernels keep the butterflies in registers when every packed
    segment (``cols / (8 / bits)`` channels) starts on a block boundary.  With
    ``fit_rotate`` (default) a site whose segments do not, e.g. 11 008 channels at
    4 bits with blocks of 256, uses the largest supported block that does (64
    there); ``fit_rotate=False`` keeps the requested block and the slower
    shared-memory hand-over."""

    BLOCKS = (4096, 1024, 256, 64, 16)

    def __init__(self, outlier_ratio: float, outlier_mode: str = "element", group_size: int = 0, rotate: int = 0,
                 fit_rotate: bool = True):
        if outlier_mode not in ("element", "channel"):
            raise ValueError("outlier_mode must be 'element' or 'channel'")
        if group_size not in (0, 128):
            raise ValueError("group_size must be 0 (per token) or 128")
        if rotate not in (0, 16, 64, 256, 1024, 4096):
            raise ValueError("rotate must be 0 or a block size in {16, 64, 256, 1024, 4096}")
        self.outlier_mode, self.group_size, self.rotate = outlier_mode, group_size, rotate
        self.fit_rotate = fit_rotate
        self.calib = cf.ChannelCalibration(outlier_ratio)
        self._dummy = None
        # norm sites only: the format and calibration of the site that saves this norm's OUTPUT (learnt
        # during calibration), and the record of that output the last forward call made beside its own
        self.output_format = None
        self.pending_output = None

    @property
    def channel(self) -> bool:
        return self.outlier_mode == "channel"

    def rotate_for(self, cols: int, bits: int) -> int:
        """Rotation block used for an activation of ``cols`` channels at ``bits`` bits."""
        if not self.rotate or not self.fit_rotate:
            return self.rotate
        segment = cols // (8 // bits)
        for block in self.BLOCKS:
            if block <= self.rotate and segment % block == 0:
                return block
        return self.rotate

    def dummy_stats(self, device):
        """Placeholders for the four statistic outputs of a Function in channel mode."""
        if self._dummy is None or self._dummy[0].device != device:
            z = torch.zeros((), device=device)
            self._dummy = (z, torch.zeros(1, 1, device=device, dtype=torch.bfloat16),
                           torch.zeros(1, 1, device=device, dtype=torch.bfloat16),
                           torch.ones((), device=device, dtype=torch.bfloat16))
        return self._dummy


def site_options(extra) -> Optional[SiteOptions]:
    return extra[0] if extra else None


# ---------------------------------------------------------------------------------------------
# One compressed copy for sites that save the same tensor (channel mode).  The q, k and v LoRA-A
# linears of a layer all save the layer's normalised input, gate and up save the same tensor too: the
# reference compresses it once per module.  Here a site that is handed the very tensor object the
# previous site compressed (same object, same version counter, same format) takes that site's
# record instead of making its own; during calibration it also adopts that site's channel
# statistics, so that afterwards "same record" can be decided by object identity, without a look at
# the device.  Records are read-only in backward, so sharing is invisible in the results.
# ---------------------------------------------------------------------------------------------
SHARE_SITES = True
_shared = []     # most recent first: (weakref to x, version, format key, record, calibration of the producer)


def _shared_lookup(x, key, opts, iteration):
    if not SHARE_SITES:
        return None
    for ref, version, k, rec, calib in _shared:
        if ref() is x and version == x._version and k == key:
            if iteration < 2:
                opts.calib.score, opts.calib.channels = calib.score, calib.channels
                return rec
            mine = opts.calib.channels
            if mine is not None and mine is calib.channels:
                return rec
            # calibrations restored from a checkpoint hold equal channel lists in separate tensors: compare
            # once (one read of the device per site) and adopt the producer's tensor when they agree
            if (mine is not None and calib.channels is not None and getattr(opts.calib, "_compared", None) is not
                    calib.channels):
                opts.calib._compared = calib.channels
                if mine.shape == calib.channels.shape and bool(torch.equal(mine, calib.channels)):
                    opts.calib.channels = calib.channels
                    return rec
    return None


def _shared_store(x, key, rec, calib):
    if not SHARE_SITES:
        return
    _shared.insert(0, (weakref.ref(x), x._version, key, rec, calib))
    del _shared[2:]


# ---------------------------------------------------------------------------------------------
# The record of a norm's OUTPUT from the norm's own pass (channel mode).  The LoRA-A linears behind a
# norm save the norm output; the fused norm kernel has that row in shared memory already and can emit
# its record beside the record of the norm input.  Nothing tells a norm module who reads its output, so
# it is learnt at run time: while a norm knows no reader, its module notes the tensor object it
# returned, and the first site that is handed that very object (and has to compress it) leaves its
# format and its calibration object with the norm's options.  From the first steady-state call on, the
# norm's forward passes that site's frozen channels to the kernel and publishes the second record
# through the table above, where the sites behind the norm find it.
# ---------------------------------------------------------------------------------------------
_last_norm_output = None     # (weakref to the tensor, version, options of the norm site)


def _offer_to_norm(x, bits, rotate, opts):
    """Called by a site that is about to compress ``x`` itself."""
    global _last_norm_output
    if _last_norm_output is None:
        return
    ref, version, norm_opts = _last_norm_output
    if ref() is x and version == x._version:
        norm_opts.output_format = (bits, opts.group_size, rotate, opts.calib)
        _last_norm_output = None


def norm_output_ready(result, opts, iteration):
    """Called by a norm module with the tensor its Function returned."""
    global _last_norm_output
    if not SHARE_SITES:
        return
    rec, opts.pending_output = opts.pending_output, None
    if rec is not None:
        bits, group, rotate, calib = opts.output_format
        _shared_store(result, (bits, group, rotate, calib.outlier_ratio, False), rec, calib)
    elif opts.output_format is None:
        _last_norm_output = (weakref.ref(result), result._version, opts)


def _output_request(opts, iteration):
    """What a norm site asks ``compress_n`` to emit for its output, or None."""
    if not SHARE_SITES or iteration < 2 or opts.output_format is None:
        return None
    bits, group, rotate, calib = opts.output_format
    if calib.channels is None:
        return None
    return dict(channels=calib.channels, bits=bits, group=group, rotate=rotate)


@torch.no_grad()
def fused_site(kind: str, x, bits: int, iteration: int, opts: Optional[SiteOptions], x1=None):
    """Channel mode, bf16 rows: the site's output AND the record of its saved input from one kernel --
    ``kind`` "silu" / "gelu": ``y = act(x)``; "product": ``y = x1 * x``, the record being that of ``x`` (the
    second operand; the first one's record comes from the site that produced it).  When a later site has
    registered as the reader of ``y`` (see ``norm_output_ready``), the kernel makes that record too and it is
    left in ``opts.pending_output``.  Returns ``(packed, y)``, or None where this path does not apply (the
    caller then computes ``y`` and calls ``compress_site``)."""
    if (opts is None or not opts.channel or not x.is_cuda or x.dtype != torch.bfloat16 or x.dim() == 4
            or (x1 is not None and (x1.dtype != torch.bfloat16 or x1.shape != x.shape))):
        return None
    cols = x.shape[-1]
    rotate = opts.rotate_for(cols, bits)
    channels = opts.calib.channels_for(x, iteration)
    also = _output_request(opts, iteration)
    if kind == "product":
        res = cf._pk.product_compress_n(x1, x, channels, bits, opts.group_size, rotate, also_output=also)
    else:
        res = cf._pk.act_compress_n(kind, x, channels, bits, opts.group_size, rotate, also_output=also)
    if res is None:
        # the library does not build this shape: the separate passes, with the channels chosen above
        y = x1 * x if kind == "product" else (torch.nn.functional.silu(x) if kind == "silu" else torch.nn.functional.gelu(x))
        opts.pending_output = None
        return cf.channel_compress(x, channels, bits, opts.group_size, rotate), y
    packed, y, opts.pending_output = res
    return packed, y.view(x.shape)


@torch.no_grad()
def compress_site(x, outlier_ratio, sub_outlier_ratio, sub_outlier_bit, method, rank, iteration, static_value,
                  opts: Optional[SiteOptions], norm: Optional[dict] = None):
    """Compress ``x`` for backward.  Returns ``(packed, (outlier, L, R, scale), norm_out)``
    where ``norm_out`` is ``(y, rstd, mean)`` when ``norm`` is given."""
    if not x.is_cuda:
        raise RuntimeError("hyc_lora_b200 operators run on CUDA tensors only (there is no CPU path)")
    if opts is not None and opts.channel:
        cols = x.shape[-1] if x.dim() != 4 else x.shape[1] * x.shape[3]
        rotate = opts.rotate_for(cols, sub_outlier_bit)
        stats = opts.dummy_stats(x.device)
        key = (sub_outlier_bit, opts.group_size, rotate, opts.calib.outlier_ratio, iteration < 2)
        if norm is None:
            shared = _shared_lookup(x, key, opts, iteration)
            if shared is not None:
                return shared, stats, None
            _offer_to_norm(x, sub_outlier_bit, rotate, opts)
        channels = opts.calib.channels_for(x, iteration)
        if norm is None:
            res = cf.channel_compress(x, channels, sub_outlier_bit, opts.group_size, rotate)
            _shared_store(x, key, res, opts.calib)
            return res, stats, None
        also = _output_request(opts, iteration)
        res = cf.channel_compress(x, channels, sub_outlier_bit, opts.group_size, rotate, norm=norm, also_output=also)
        opts.pending_output = res[4] if also is not None else None
        return res[0], stats, res[1:4]
    if iteration < 2:
        outlier, L, R, scale = cf.get_statistics(x, iteration, outlier_ratio, sub_outlier_ratio, sub_outlier_bit,
                                                 method, rank)
        cache = None
    else:
        outlier, L, scale, R = static_value[0], static_value[1], static_value[2], static_value[3]
        cache = static_value.cache if isinstance(static_value, StaticList) else None
    res = cf.true_divide_outlier_suboutlier_svd_compress(x, outlier, scale, sub_outlier_bit, sub_outlier_ratio, L, R,
                                                         rank=rank, cache=cache, outlier_ratio=outlier_ratio, norm=norm)
    packed, _codes, scale_out = res[0], res[1], res[2]
    return packed, (outlier, L, R, scale_out), (res[3:] if norm is not None else None)


def update_static(static_value, iteration, outlier, L, scale, R):
    """The reference's running mean over the first two calls (efficient_linear.py:122-146)."""
    if iteration >= 2:
        return
    n = iteration
    static_value[0] = outlier if static_value[0] is None else (n * static_value[0] + outlier) / (n + 1)
    static_value[1] = L if static_value[1] is None else (n * static_value[1] + cf.pad_cut_L(L, static_value[1])) / (n + 1)
    static_value[2] = scale if static_value[2] is None else (n * static_value[2] + scale) / (n + 1)
    static_value[3] = R if static_value[3] is None else (n * static_value[3] + R) / (n + 1)
    if isinstance(static_value, StaticList):
        static_value.cache.clear()


def calibration_state_dict(module) -> dict:
    """Calibration state of one ``EfficientMemory*`` module as plain tensors / numbers, so that a
    resumed run does not recalibrate (in the reference this state is Python attributes only and is
    lost on resume)."""
    out = {"iteration": module.iteration}
    for name in ("static_value", "static_value_1", "static_value_2"):
        if hasattr(module, name):
            v = getattr(module, name)
            out[name] = [None if t is None else t.detach().clone() for t in v] if isinstance(v, list) else (
                None if v is None else v.detach().clone())
    for name in ("site", "site_1", "site_2"):
        if hasattr(module, name):
            c = getattr(module, name).calib
            out[name] = {"score": None if c.score is None else c.score.clone(),
                         "channels": None if c.channels is None else c.channels.clone()}
    return out


def load_calibration_state_dict(module, state: dict) -> None:
    module.iteration = int(state["iteration"])
    for name in ("static_value", "static_value_1", "static_value_2"):
        if name in state:
            v = state[name]
            setattr(module, name, StaticList(v) if isinstance(v, list) else v)
    for name in ("site", "site_1", "site_2"):
        if name in state and hasattr(module, name):
            c = getattr(module, name).calib
            c.score, c.channels = state[name]["score"], state[name]["channels"]
