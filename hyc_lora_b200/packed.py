"""Packed activations and thin Python callers of the C ABI.

A :class:`Packed` owns the device buffers of one compressed activation (all
of them ordinary torch tensors, so PyTorch's caching allocator manages their
lifetime) and knows how to describe itself as the ``hyc_packed`` record the
kernels take.  The functions below allocate outputs, fill the records and
enqueue the kernel on the current CUDA stream; none of them synchronises.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from . import _lib
from ._lib import HycDense, HycNormBwdArgs, HycNormFwd, HycPacked, HycSparseRows, check, lib

_SCALE_KIND = {"per-tensor": _lib.HYC_SCALE_TENSOR, "per-channel": _lib.HYC_SCALE_CHANNEL,
               "per-token": _lib.HYC_SCALE_TOKEN}
_NORM_KIND = {"rms": _lib.HYC_NORM_RMS, "rms_gemma": _lib.HYC_NORM_RMS_GEMMA, "ln": _lib.HYC_NORM_LAYER}
_ACT_OP = {"silu": _lib.HYC_ACT_SILU, "gelu": _lib.HYC_ACT_GELU_TANH, "product": _lib.HYC_ACT_PRODUCT}


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.HYC_BF16
    if t.dtype == torch.float32:
        return _lib.HYC_F32
    raise TypeError(f"unsupported dtype {t.dtype}: the kernels take float32 or bfloat16")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("hyc_lora_b200 operators run on CUDA tensors only (there is no CPU path)")


@dataclass
class Packed:
    """One compressed activation (rows x cols, rows = batch * seq)."""
    mode: str                    # "R" or "N"
    bits: int
    rows: int
    cols: int
    seq: int
    codes: torch.Tensor          # uint8 [rows, cols*bits/8]
    status: torch.Tensor         # int32 [1]
    shape: tuple                 # logical [B, S, D] shape of the activation
    # reference mode
    scale: Optional[torch.Tensor] = None
    scale_kind: str = "per-tensor"
    thr: Optional[torch.Tensor] = None
    lowrank: Optional[torch.Tensor] = None   # bf16 [seq, cols]
    pool: Optional[torch.Tensor] = None      # int32 [capacity]
    pool_used: Optional[torch.Tensor] = None  # int32 [1]
    row_meta: Optional[torch.Tensor] = None  # int32 [rows, 2]
    # north-star mode
    channels: Optional[torch.Tensor] = None  # int32 [k]
    group: int = 0
    rotate: int = 0
    out_value: Optional[torch.Tensor] = None  # bf16 [rows, k]
    scales: Optional[torch.Tensor] = None     # f32 [rows, G]
    _keep: list = field(default_factory=list, repr=False)

    def record(self) -> HycPacked:
        r = HycPacked()
        r.mode = _lib.HYC_MODE_R if self.mode == "R" else _lib.HYC_MODE_N
        r.bits, r.rows, r.cols, r.seq = self.bits, self.rows, self.cols, self.seq
        r.codes = self.codes.data_ptr()
        r.status = self.status.data_ptr()
        if self.mode == "R":
            r.scale_kind = _SCALE_KIND[self.scale_kind]
            r.scale_dtype = _dtype_code(self.scale)
            r.scale = self.scale.data_ptr()
            r.thr = self.thr.data_ptr() if self.thr is not None else None
            r.lowrank = self.lowrank.data_ptr() if self.lowrank is not None else None
            r.pool = self.pool.data_ptr()
            r.pool_cap = self.pool.numel()
            r.pool_used = self.pool_used.data_ptr()
            r.row_meta = self.row_meta.data_ptr()
        else:
            k = 0 if self.channels is None else self.channels.numel()
            r.channels = self.channels.data_ptr() if k else None
            r.n_channels = k
            r.group, r.rotate = self.group, self.rotate
            r.out_value = self.out_value.data_ptr() if k else None
            r.scales = self.scales.data_ptr()
        return r

    def nbytes(self) -> int:
        """Bytes this activation keeps alive for backward."""
        n = self.codes.numel()
        if self.mode == "R":
            n += self.pool.numel() * 4 + self.row_meta.numel() * 4
        else:
            n += self.scales.numel() * 4 + (0 if self.out_value is None else self.out_value.numel() * 2)
        return n

    # ---- helpers for checks (synchronise; not used on the training path) ----
    def overflowed(self) -> bool:
        return bool(int(self.status.item()) & _lib.HYC_STATUS_POOL_OVERFLOW)

    def wait_expired(self) -> bool:
        return bool(int(self.status.item()) & _lib.HYC_STATUS_WAIT_EXPIRED)

    def outlier_coo(self):
        """Reference-mode outliers as (flat element index int64 [nnz] sorted, bf16 values) -- the
        content of the reference's sparse COO tensor, for parity checks."""
        meta = self.row_meta.cpu().long()
        pool = self.pool.cpu()
        first, cnt = meta[:, 0], meta[:, 1]
        rows = torch.repeat_interleave(torch.arange(self.rows), cnt)
        starts = torch.repeat_interleave(first, cnt)
        within = torch.arange(int(cnt.sum())) - torch.repeat_interleave(torch.cumsum(cnt, 0) - cnt, cnt)
        entry = pool[(starts + within)].long() & 0xFFFFFFFF
        col = entry & 0xFFFF
        hi = (entry >> 16) & 0xFFFF
        val = torch.where(hi >= 32768, hi - 65536, hi).to(torch.int16).view(torch.bfloat16)
        flat = rows * self.cols + col
        order = torch.argsort(flat)
        return flat[order], val[order]


def _dense_record(x: torch.Tensor, cols: int):
    """Describe ``x`` ([..., D] contiguous rows, or a [B,H,S,hd] head tensor that is
    seen as [B,S,H*hd]) as an hyc_dense.  Returns (record, rows, seq, logical_shape, keepalive)."""
    d = HycDense()
    d.dtype = _dtype_code(x)
    if x.dim() == 4:
        b, h, s, hd = x.shape
        if x.stride(3) != 1:
            x = x.contiguous()
        d.base = x.data_ptr()
        d.chunks = h
        d.batch_stride, d.chunk_stride, d.row_stride = x.stride(0), x.stride(1), x.stride(2)
        if h * hd != cols:
            raise ValueError("head tensor does not match cols")
        return d, b * s, s, (b, s, h * hd), x
    if x.shape[-1] != cols:
        raise ValueError("last dimension does not match cols")
    if not x.is_contiguous():
        x = x.contiguous()
    d.base = x.data_ptr()
    d.chunks = 1
    d.row_stride = cols
    rows = x.numel() // cols
    seq = x.shape[-2] if x.dim() >= 2 else 1
    shape = tuple(x.shape) if x.dim() == 3 else (1, rows, cols) if x.dim() <= 2 else (rows // seq, seq, cols)
    return d, rows, seq, shape, x


_pool_growth = 1.0      # doubled by poll_status() each time it sees an overflowed pool


def default_pool_entries(rows: int, cols: int, outlier_ratio: float, density: Optional[float] = None) -> int:
    """Capacity of the element-outlier pool (4 bytes per entry).

    Without a measurement: eight times ``outlier_ratio`` of the tensor -- four times the density the
    reference's calibration produces (its signed quantile keeps about ``2 * ratio`` of the elements).
    With ``density``, the fraction of elements above the frozen threshold that the site measured on its
    first steady-state call: twice that plus one percent.  Either way at least 1/64 of the tensor, and
    multiplied by the growth factor that :func:`poll_status` raises after an overflow."""
    frac = 8.0 * outlier_ratio if density is None else 2.0 * density + 0.01
    frac = min(max(frac, 1.0 / 64.0) * _pool_growth, 1.0)
    return min(int(math.ceil(rows * cols * frac)) + 1024, 2 ** 32 - 2)


# ---------------------------------------------------------------------------
# Status words.  Every record carries one device word into which kernels OR what only the device can
# see: an outlier pool (or sparse-probability list) that was too small, a bounded wait that ran out.
# Nothing on the hot path reads them.  fold_status() ORs every word handed out since the last fold into
# one accumulator per device (a few tiny kernels; capturable, so a recorded training step folds its own
# words), and poll_status() brings the accumulator to the host without blocking and reports the value
# of the previous poll -- one step late, no synchronisation.
# ---------------------------------------------------------------------------
_STATUS_CHUNK = 1024


class _StatusBoard:
    def __init__(self):
        self.chunks = {}        # device key -> [chunk, words used]                (outside stream capture)
        self.capture = {}       # device key -> [chunk, words used]                (inside the current capture)
        self.dirty = {}         # device key -> tensors holding words handed out since the last fold
        self.acc = {}           # device key -> int32[1] accumulator
        self.pending = {}       # device key -> (pinned int32[1], event) of the last poll
        self.reported = 0       # bits already warned about

    @staticmethod
    def key(device):
        device = torch.device(device)
        return (device.type, device.index if device.index is not None else torch.cuda.current_device())

    def new(self, device) -> torch.Tensor:
        key = self.key(device)
        capturing = torch.cuda.is_current_stream_capturing()
        book = self.capture if capturing else self.chunks
        if not capturing:
            self.capture.pop(key, None)      # a chunk made inside a graph's memory pool is never used outside it
        slot = book.get(key)
        if slot is None or slot[1] >= _STATUS_CHUNK:
            slot = [torch.zeros(_STATUS_CHUNK, dtype=torch.int32, device=device), 0]
            book[key] = slot
            self.dirty.setdefault(key, []).append(slot[0])
        word = slot[0][slot[1]:slot[1] + 1]
        slot[1] += 1
        return word

    def fold(self, device=None):
        keys = [self.key(device)] if device is not None else list(self.dirty)
        for key in keys:
            tensors = self.dirty.get(key, [])
            if not tensors:
                continue
            if key not in self.acc:
                if torch.cuda.is_current_stream_capturing():
                    raise RuntimeError("fold_status(): call it once outside stream capture before recording a graph")
                self.acc[key] = torch.zeros(1, dtype=torch.int32, device=tensors[0].device)
            acc = self.acc[key]
            for t in tensors:
                acc.bitwise_or_((t & 1).amax() | (t & 2).amax())
            if torch.cuda.is_current_stream_capturing():
                self.capture.pop(key, None)              # the next recorded step starts a fresh chunk
            # a partly used chunk stays under watch: its remaining words are still to be handed out
            live = self.chunks.get(key)
            self.dirty[key] = [live[0]] if live is not None and live[1] < _STATUS_CHUNK else []

    def poll(self, wait: bool = False) -> int:
        global _pool_growth
        if not torch.cuda.is_current_stream_capturing():
            self.fold()
        seen = 0
        for key, acc in self.acc.items():
            host, ev = self.pending.get(key, (None, None))
            if ev is not None:
                if wait:
                    ev.synchronize()
                if not ev.query():
                    continue                               # the previous copy is still in flight: look again next time
                seen |= int(host.item())
            if host is None:
                host = torch.zeros(1, dtype=torch.int32).pin_memory()
            with torch.cuda.device(acc.device):
                host.copy_(acc, non_blocking=True)         # stream-ordered after everything enqueued so far
                ev = torch.cuda.Event()
                ev.record()
            self.pending[key] = (host, ev)
            if wait:
                ev.synchronize()
                seen |= int(host.item())
        fresh = seen & ~self.reported
        if fresh & _lib.HYC_STATUS_WAIT_EXPIRED:
            self.reported |= _lib.HYC_STATUS_WAIT_EXPIRED
            raise RuntimeError("hyc_lora_b200: a kernel gave up waiting for its own staged copy "
                               "(HYC_STATUS_WAIT_EXPIRED); results of that call are not valid")
        if fresh & _lib.HYC_STATUS_POOL_OVERFLOW:
            self.reported |= _lib.HYC_STATUS_POOL_OVERFLOW
            _pool_growth *= 2.0
            import warnings
            warnings.warn("hyc_lora_b200: an outlier pool or sparse-probability list was too small "
                          "(HYC_STATUS_POOL_OVERFLOW): some rows were stored without their outliers. Capacities are "
                          "doubled from now on; a recorded CUDA graph keeps its old capacities until it is recorded again.")
        return seen

    def reset(self):
        """Forget everything flagged so far: words handed out earlier are no longer watched."""
        self.chunks.clear()
        self.capture.clear()
        self.dirty.clear()
        for acc in self.acc.values():
            acc.zero_()
        self.pending.clear()
        self.reported = 0


_board = _StatusBoard()


def _new_status(device) -> torch.Tensor:
    """A zeroed int32 status word, handed out from a chunk zeroed by one fill so that a compression call
    does not cost a fill kernel of its own; a word is never handed out twice.  Words asked for during
    stream capture come from a chunk that lives in that capture."""
    return _board.new(device)


def fold_status(device=None) -> None:
    """OR every status word handed out since the last call into the per-device accumulator.  Cheap and
    capturable: a training step calls it once, after backward (before recording a graph, call it once
    outside the capture so that the accumulator exists)."""
    _board.fold(device)


def poll_status(wait: bool = False) -> int:
    """Bring the accumulated status to the host.  Without ``wait`` nothing blocks: the call starts an
    asynchronous copy and returns the value the PREVIOUS call fetched (0 the first time).  Raises on an
    expired wait; on a pool overflow warns once and doubles the default capacities.  Returns the OR of
    the HYC_STATUS_* bits seen."""
    return _board.poll(wait)


def reset_status() -> None:
    """Clear the accumulated status and stop watching the words handed out so far (also restores the
    default pool capacities)."""
    global _pool_growth
    _pool_growth = 1.0
    _board.reset()


def _alloc_common(rows, cols, bits, device):
    codes = torch.empty((rows, cols * bits // 8), dtype=torch.uint8, device=device)
    return codes, _new_status(device)


def _new_r(x, rows, cols, seq, shape, thr, scale, scale_kind, bits, lowrank, pool_entries) -> Packed:
    dev = x.device
    codes, status = _alloc_common(rows, cols, bits, dev)
    return Packed(mode="R", bits=bits, rows=rows, cols=cols, seq=seq, codes=codes, status=status, shape=shape,
                  scale=scale.contiguous(), scale_kind=scale_kind,
                  thr=thr.reshape(1).to(device=dev, dtype=torch.float32), lowrank=lowrank,
                  pool=torch.empty(pool_entries, dtype=torch.int32, device=dev),
                  pool_used=torch.empty(1, dtype=torch.int32, device=dev),
                  row_meta=torch.empty((rows, 2), dtype=torch.int32, device=dev))


def _new_n(x, rows, cols, seq, shape, channels, bits, group, rotate) -> Packed:
    dev = x.device
    codes, status = _alloc_common(rows, cols, bits, dev)
    k = 0 if channels is None else channels.numel()
    g = 1 if group == 0 else cols // group
    return Packed(mode="N", bits=bits, rows=rows, cols=cols, seq=seq, codes=codes, status=status, shape=shape,
                  channels=channels, group=group, rotate=rotate,
                  out_value=torch.empty((rows, k), dtype=torch.bfloat16, device=dev) if k else None,
                  scales=torch.empty((rows, g), dtype=torch.float32, device=dev))


def scale_kind_of(scale: torch.Tensor) -> str:
    """The reference tells its three scale layouts apart by shape: 0-dim,
    [1, D] (per-channel) and [S, 1] (per-token)."""
    if scale.dim() == 0 or scale.numel() == 1 and scale.dim() < 2:
        return "per-tensor"
    if scale.dim() == 2 and scale.shape[0] == 1:
        return "per-channel" if scale.shape[1] > 1 else "per-tensor"
    return "per-token"


def compress_r(x: torch.Tensor, thr: torch.Tensor, scale: torch.Tensor, bits: int,
               lowrank: Optional[torch.Tensor] = None, pool_entries: Optional[int] = None,
               outlier_ratio: float = 0.01, norm: Optional[dict] = None, density: Optional[float] = None):
    """Reference-mode compression of ``x`` ([B,S,D] or [B,H,S,hd]).  With
    ``norm`` (keys kind, weight, bias, eps) the norm forward is fused and
    ``(packed, y, rstd, mean)`` is returned, else ``packed``."""
    _require_cuda(x, thr, scale)
    cols = x.shape[-1] if x.dim() != 4 else x.shape[1] * x.shape[3]
    d, rows, seq, shape, keep = _dense_record(x, cols)
    if scale.dtype != torch.bfloat16:
        scale = scale.to(torch.bfloat16)
    kind = scale_kind_of(scale)
    if kind == "per-token" and scale.numel() != seq:
        raise ValueError(f"per-token scale has {scale.numel()} positions, the activation has {seq}")
    if pool_entries is None:
        pool_entries = default_pool_entries(rows, cols, outlier_ratio, density)
    p = _new_r(keep, rows, cols, seq, shape, thr, scale, kind, bits, lowrank, pool_entries)
    return _run_fwd(d, keep, p, norm)


def compress_n(x: torch.Tensor, channels: Optional[torch.Tensor], bits: int, group: int = 0, rotate: int = 0,
               norm: Optional[dict] = None, also_output: Optional[dict] = None):
    """North-star-mode compression (channel outliers, dynamic absmax scales,
    optional block Hadamard rotation).

    ``also_output`` (with ``norm`` only; keys ``channels``, ``bits``, ``group``, ``rotate``): the norm OUTPUT is
    compressed in the same pass into a second record, for the sites behind the norm that save it.  Returns
    ``(packed, y, rstd, mean, packed_y)`` then; ``packed_y`` is None when the library does not take the pair
    (the caller compresses ``y`` with a call of its own)."""
    _require_cuda(x, channels)
    cols = x.shape[-1] if x.dim() != 4 else x.shape[1] * x.shape[3]
    d, rows, seq, shape, keep = _dense_record(x, cols)
    p = _new_n(keep, rows, cols, seq, shape, channels, bits, group, rotate)
    if also_output is None or norm is None:
        return _run_fwd(d, keep, p, norm)
    p2 = None
    o = also_output
    # the library builds the pair for bf16 rows of one format that a warp can hold (rotation blocks of at most 256
    # channels that tile a packed segment); anything else is not asked for
    fits = cols <= 4096 and (rotate == 0 or (rotate <= 256 and (cols // (8 // bits)) % 256 == 0))
    if (o["bits"] == bits and o.get("group", 0) == group and o.get("rotate", 0) == rotate and keep.dim() != 4
            and keep.dtype == torch.bfloat16 and fits):
        p2 = _new_n(keep, rows, cols, seq, shape, o["channels"], bits, group, rotate)
    if p2 is None:
        return (*_run_fwd(d, keep, p, norm), None)
    return _run_fwd(d, keep, p, norm, p2)


def _same_format(a: dict, bits, group, rotate) -> bool:
    return a["bits"] == bits and a.get("group", 0) == group and a.get("rotate", 0) == rotate


def act_compress_n(op: str, x: torch.Tensor, channels, bits: int, group: int = 0, rotate: int = 0,
                   also_output: Optional[dict] = None):
    """``y = silu(x)`` / ``gelu(x)`` and the channel-mode record of ``x`` in one pass; with ``also_output``
    (keys ``channels``, ``bits``, ``group``, ``rotate``) also the record of ``y``.  Returns ``(packed_x, y, packed_y)``,
    or None when the library does not build this combination (the caller then computes ``y`` and compresses with
    calls of its own)."""
    _require_cuda(x, channels)
    if x.dim() == 4 or x.dtype != torch.bfloat16:
        return None
    cols = x.shape[-1]
    d, rows, seq, shape, keep = _dense_record(x, cols)
    p = _new_n(keep, rows, cols, seq, shape, channels, bits, group, rotate)
    p2 = None
    if also_output is not None and _same_format(also_output, bits, group, rotate):
        p2 = _new_n(keep, rows, cols, seq, shape, also_output["channels"], bits, group, rotate)
    y = torch.empty_like(keep)
    rec = p.record()
    rec2 = p2.record() if p2 is not None else None
    rc = lib.hyc_act_compress(C.byref(d), _ACT_OP[op], y.data_ptr(), C.byref(rec), C.byref(rec2) if rec2 is not None else None,
                              _stream())
    if rc == _lib.HYC_ERR_SHAPE:
        return None
    check(rc, "hyc_act_compress")
    return p, y, p2


def product_compress_n(x1: torch.Tensor, x2: torch.Tensor, channels2, bits: int, group: int = 0, rotate: int = 0,
                       also_output: Optional[dict] = None):
    """``y = x1 * x2`` and the channel-mode record of ``x2`` in one pass; with ``also_output`` also the record
    of ``y``.  Returns ``(packed_x2, y, packed_y)`` or None (see :func:`act_compress_n`)."""
    _require_cuda(x1, x2, channels2)
    if x1.dim() == 4 or x1.dtype != torch.bfloat16 or x2.dtype != torch.bfloat16 or x1.shape != x2.shape:
        return None
    cols = x2.shape[-1]
    d1, _, _, _, keep1 = _dense_record(x1, cols)
    d2, rows, seq, shape, keep2 = _dense_record(x2, cols)
    p = _new_n(keep2, rows, cols, seq, shape, channels2, bits, group, rotate)
    p2 = None
    if also_output is not None and _same_format(also_output, bits, group, rotate):
        p2 = _new_n(keep2, rows, cols, seq, shape, also_output["channels"], bits, group, rotate)
    y = torch.empty_like(keep2)
    rec = p.record()
    rec2 = p2.record() if p2 is not None else None
    rc = lib.hyc_product_compress(C.byref(d1), C.byref(d2), y.data_ptr(), C.byref(rec),
                                  C.byref(rec2) if rec2 is not None else None, _stream())
    if rc == _lib.HYC_ERR_SHAPE:
        return None
    check(rc, "hyc_product_compress")
    return p, y, p2


def _run_fwd(d, x, p: Packed, norm, p2: Optional[Packed] = None):
    rec = p.record()
    if norm is None:
        check(lib.hyc_compress(C.byref(d), C.byref(rec), _stream()), "hyc_compress")
        return p
    kind = norm["kind"]
    w, b = norm["weight"], norm.get("bias")
    _require_cuda(w, b)
    if b is not None and b.dtype != w.dtype:
        b = b.to(w.dtype)
    n = HycNormFwd()
    n.kind = _NORM_KIND[kind]
    n.eps = float(norm["eps"])
    n.weight, n.bias = w.data_ptr(), (b.data_ptr() if (b is not None and kind == "ln") else None)
    n.param_dtype = _dtype_code(w)
    y = torch.empty_like(x)
    rstd = torch.empty(p.rows, dtype=torch.float32, device=x.device)
    mean = torch.empty(p.rows, dtype=torch.float32, device=x.device) if kind == "ln" else None
    n.y, n.rstd, n.mean = y.data_ptr(), rstd.data_ptr(), (mean.data_ptr() if mean is not None else None)
    if p2 is not None:
        rec2 = p2.record()
        rc = lib.hyc_norm_compress2(C.byref(d), C.byref(n), C.byref(rec), C.byref(rec2), _stream())
        if rc == 0:
            return p, y, rstd, mean, p2
        if rc != _lib.HYC_ERR_SHAPE:
            check(rc, "hyc_norm_compress2")
        # the pair is not taken (row too wide, rotation, ...): one record now, the caller makes the other
        check(lib.hyc_norm_compress(C.byref(d), C.byref(n), C.byref(rec), _stream()), "hyc_norm_compress")
        return p, y, rstd, mean, None
    check(lib.hyc_norm_compress(C.byref(d), C.byref(n), C.byref(rec), _stream()), "hyc_norm_compress")
    return p, y, rstd, mean


def decompress(p: Packed, num_heads: int = 0) -> torch.Tensor:
    """bf16 reconstruction, [B,S,D] or (``num_heads``) a [B,H,S,hd] view of it."""
    b, s, dcols = p.shape
    out = torch.empty((b, s, dcols), dtype=torch.bfloat16, device=p.codes.device)
    d = HycDense()
    d.base, d.dtype, d.chunks, d.row_stride = out.data_ptr(), _lib.HYC_BF16, 1, dcols
    rec = p.record()
    check(lib.hyc_decompress(C.byref(rec), C.byref(d), _stream()), "hyc_decompress")
    if num_heads:
        return out.reshape(b, s, num_heads, dcols // num_heads).transpose(1, 2)
    return out


def norm_bwd(p: Packed, dy: torch.Tensor, weight: torch.Tensor, rstd: torch.Tensor, mean: Optional[torch.Tensor],
             kind: str, ref_compat_c2: bool = True, need_dweight: bool = False, need_dbias: bool = False):
    """Returns ``(dx bf16, dweight fp32 | None, dbias fp32 | None)``."""
    _require_cuda(dy, weight, rstd)
    if not dy.is_contiguous():
        dy = dy.contiguous()
    dx = torch.empty(dy.shape, dtype=torch.bfloat16, device=dy.device)
    a = HycNormBwdArgs()
    a.kind, a.ref_compat_c2 = _NORM_KIND[kind], int(ref_compat_c2)
    a.weight, a.param_dtype = weight.data_ptr(), _dtype_code(weight)
    a.dy, a.dy_dtype = dy.data_ptr(), _dtype_code(dy)
    a.rstd, a.mean = rstd.data_ptr(), (mean.data_ptr() if mean is not None else None)
    a.dx = dx.data_ptr()
    dw = db = partials = None
    if need_dweight:
        nparts = lib.hyc_norm_bwd_partial_rows()
        dw = torch.empty(p.cols, dtype=torch.float32, device=dy.device)
        db = torch.empty(p.cols, dtype=torch.float32, device=dy.device) if need_dbias else None
        partials = torch.empty((2 if need_dbias else 1) * nparts * p.cols, dtype=torch.float32, device=dy.device)
        a.dweight, a.dbias, a.partials = dw.data_ptr(), (db.data_ptr() if db is not None else None), partials.data_ptr()
    rec = p.record()
    check(lib.hyc_norm_bwd(C.byref(rec), C.byref(a), _stream()), "hyc_norm_bwd")
    return dx, dw, db


def act_bwd(op: str, p1: Packed, g: torch.Tensor, p2: Optional[Packed] = None):
    """``op`` in {"silu", "gelu", "product"}; returns dx (and dx2 for product) in g's dtype."""
    _require_cuda(g)
    if not g.is_contiguous():
        g = g.contiguous()
    dx1 = torch.empty_like(g)
    dx2 = torch.empty_like(g) if op == "product" else None
    r1 = p1.record()
    r2 = p2.record() if p2 is not None else None
    check(lib.hyc_act_bwd(_ACT_OP[op], C.byref(r1), C.byref(r2) if r2 is not None else None, _ptr(g),
                          _dtype_code(g), _ptr(dx1), _ptr(dx2), _stream()), "hyc_act_bwd")
    return (dx1, dx2) if op == "product" else dx1


def channel_absmax(x: torch.Tensor, score: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 column absmax of ``x`` merged (max) into ``score`` [D]."""
    _require_cuda(x)
    cols = x.shape[-1] if x.dim() != 4 else x.shape[1] * x.shape[3]
    d, rows, seq, _, keep = _dense_record(x, cols)
    if score is None:
        score = torch.zeros(cols, dtype=torch.float32, device=x.device)
    check(lib.hyc_channel_absmax(C.byref(d), rows, cols, seq, _ptr(score), _stream()), "hyc_channel_absmax")
    return score


def select_channels(score: torch.Tensor, k: int) -> torch.Tensor:
    """Ascending int32 list of the k channels of largest score (ties to the lower index)."""
    _require_cuda(score)
    cols = score.numel()
    channels = torch.empty(k, dtype=torch.int32, device=score.device)
    scratch = torch.empty(cols, dtype=torch.int32, device=score.device)
    check(lib.hyc_select_channels(_ptr(score), cols, k, _ptr(channels), _ptr(scratch), _stream()),
          "hyc_select_channels")
    return channels


# ---------------------------------------------------------------------------
# LoRA-A weight gradient from a packed activation
# ---------------------------------------------------------------------------


def lora_wgrad_supported(p: Packed, rank: int) -> bool:
    """Formats the tensor-core weight-gradient kernel takes: channel-mode records, and reference-mode records
    with 2-, 4- or 8-bit codes."""
    return (p.bits in (2, 4, 8) and rank % 8 == 0 and 8 <= rank <= 64 and (p.cols * p.bits // 8) % 128 == 0
            and p.rows > 0)


def lora_wgrad(p: Packed, grad_output: torch.Tensor, force_library: bool = False, path: str = "auto",
               out_dtype: torch.dtype = torch.float32, accumulate_into: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dW[r, D] = sum_t G[t, r] * X_hat[t, d]`` from the packed input, summed in fp32 and returned in
    ``out_dtype`` (fp32, or bf16: the LoRA-A weight's dtype, rounded once by the kernel that finishes the sums).
    ``accumulate_into``: a contiguous fp32 / bf16 ``[r, D]`` tensor (a gradient buffer) that the result is added
    to -- by the finishing kernel where the tensor-core route runs, else by one add -- and that is returned.

    The packed codes go to the dequant-fused tcgen05 kernel (the reconstruction never touches HBM).  Channel
    mode: the outlier channels' columns, the skinny product ``G^T @ out_value``, come from extra thread blocks
    of the same launch.  Reference mode: static scales are folded into the gradient rows (per token / per
    tensor) or into the result's columns (per channel), the element outliers are added as a sparse side term
    by a second kernel, and a low-rank part adds ``(sum over the batch of G)^T @ lowrank`` here, one small
    library GEMM.  1-bit codes (and ranks the kernel does not take) are rebuilt by the decompress kernel and
    contracted by a library GEMM in bf16 with fp32 accumulation -- the arithmetic of the reference
    (efficient_linear.py:61-67) followed by the autograd engine's sum over the batch.

    ``path``: "tensor" (the tcgen05 kernel where it takes the record), "library" (decompress + GEMM), or "auto":
    the faster of the two as measured on a B200 -- the tensor-core kernel for channel-mode records (0.13 ms
    against 0.24 ms at 65 536 x 4 096, rank 64); decompress + GEMM for reference-mode records, whose
    element-outlier side term (one multiply-add per stored outlier and rank, through shared-memory atomics)
    costs 0.44 ms + 0.43 ms per million stored outliers against 0.26 ms for the dense route."""
    _require_cuda(grad_output)
    rank = grad_output.shape[-1]
    g = grad_output.reshape(p.rows, rank).to(torch.bfloat16).contiguous()
    if path == "auto":
        path = "library" if p.mode == "R" else "tensor"
    if force_library or path == "library" or not lora_wgrad_supported(p, rank):
        xh = decompress(p).reshape(p.rows, p.cols)
        if accumulate_into is not None:
            return accumulate_into.add_(g.t() @ xh)
        return (g.t() @ xh).to(out_dtype)
    rec = p.record()
    need = lib.hyc_lora_wgrad_scratch_floats(C.byref(rec), rank)
    if need < 0:
        check(int(need), "hyc_lora_wgrad_scratch_floats")
    # a low-rank part is added in fp32 below: the kernel's own result stays fp32 then
    lowrank = p.mode == "R" and p.lowrank is not None
    sink = accumulate_into if (accumulate_into is not None and not lowrank and accumulate_into.is_contiguous()
                               and accumulate_into.shape == (rank, p.cols) and accumulate_into.data_ptr() % 16 == 0
                               and accumulate_into.dtype in (torch.float32, torch.bfloat16)) else None
    direct = out_dtype == torch.bfloat16 and not lowrank
    out = sink if sink is not None else torch.empty((rank, p.cols), dtype=torch.bfloat16 if direct else torch.float32,
                                                    device=g.device)
    partials = torch.empty(need, dtype=torch.float32, device=g.device)
    check(lib.hyc_lora_wgrad_to(C.byref(rec), _ptr(g), rank, _ptr(out), _dtype_code(out), int(sink is not None),
                                _ptr(partials), _stream()), "hyc_lora_wgrad_to")
    if sink is not None:
        return sink
    if lowrank:
        # the low-rank rows repeat for every batch element: contract them with the batch sum of the gradient
        gsum = g.view(-1, p.seq, rank).sum(dim=0, dtype=torch.float32).to(torch.bfloat16)
        out.addmm_(gsum.t().float(), p.lowrank.float())
    if accumulate_into is not None:
        return accumulate_into.add_(out.view_as(accumulate_into))
    return out.to(out_dtype)


# ---------------------------------------------------------------------------
# thresholded copy of attention probabilities
# ---------------------------------------------------------------------------


@dataclass
class SparseRows:
    rows: int
    cols: int
    shape: tuple
    val: torch.Tensor        # [cap], dtype of the probabilities
    col: torch.Tensor        # int16 storage of uint16 columns [cap]
    used: torch.Tensor       # int32 [1]
    row_meta: torch.Tensor   # int32 [rows, 2]
    status: torch.Tensor     # int32 [1]

    def record(self) -> HycSparseRows:
        r = HycSparseRows()
        r.rows, r.cols, r.dtype = self.rows, self.cols, _dtype_code(self.val)
        r.val, r.col, r.cap = self.val.data_ptr(), self.col.data_ptr(), self.val.numel()
        r.used, r.row_meta, r.status = self.used.data_ptr(), self.row_meta.data_ptr(), self.status.data_ptr()
        return r

    def overflowed(self) -> bool:
        return bool(int(self.status.item()) & _lib.HYC_STATUS_POOL_OVERFLOW)


def softmax_compact(y: torch.Tensor, thr: torch.Tensor, capacity_ratio: float = 0.125) -> SparseRows:
    """Keep ``y > thr`` of a [..., C] probability tensor as per-row lists."""
    _require_cuda(y, thr)
    if not y.is_contiguous():
        y = y.contiguous()
    cols = y.shape[-1]
    rows = y.numel() // cols
    cap = min(int(math.ceil(rows * cols * min(max(capacity_ratio, 1.0 / 64.0), 1.0))) + 1024, 2 ** 32 - 2)
    dev = y.device
    s = SparseRows(rows=rows, cols=cols, shape=tuple(y.shape),
                   val=torch.empty(cap, dtype=y.dtype, device=dev), col=torch.empty(cap, dtype=torch.int16, device=dev),
                   used=torch.empty(1, dtype=torch.int32, device=dev),
                   row_meta=torch.empty((rows, 2), dtype=torch.int32, device=dev),
                   status=_new_status(dev))
    thr32 = thr.reshape(1).to(device=dev, dtype=torch.float32)
    rec = s.record()
    check(lib.hyc_softmax_compact(_ptr(y), _ptr(thr32), C.byref(rec), _stream()), "hyc_softmax_compact")
    return s


def softmax_expand(s: SparseRows) -> torch.Tensor:
    out = torch.empty(s.shape, dtype=s.val.dtype, device=s.val.device)
    rec = s.record()
    check(lib.hyc_softmax_expand(C.byref(rec), _ptr(out), _stream()), "hyc_softmax_expand")
    return out


def softmax_bwd(s: SparseRows, g: torch.Tensor) -> torch.Tensor:
    _require_cuda(g)
    if not g.is_contiguous():
        g = g.contiguous()
    out_dtype = torch.bfloat16 if (g.dtype == torch.bfloat16 and s.val.dtype == torch.bfloat16) else torch.float32
    dx = torch.empty(s.shape, dtype=out_dtype, device=g.device)
    rec = s.record()
    check(lib.hyc_softmax_bwd(C.byref(rec), _ptr(g), _dtype_code(g), _ptr(dx), _stream()), "hyc_softmax_bwd")
    return dx
