"""Data parallelism for the LoRA path: one process per GPU, the batch sharded across ranks,
and ONE exchange step -- the sum of the trainable (LoRA) gradients -- on NCCL.

The gradients of all trainable parameters live in a single flat fp32 buffer (each ``.grad`` is
a view into it), so the exchange is a few large all-reduces that NCCL can run through NVSwitch
(in-switch reduction when available) instead of hundreds of small ones.  With ``overlap=True`` the
buffer is cut into buckets (64 MB by default) and a bucket's all-reduce is enqueued, asynchronously,
the moment backward has accumulated the last gradient that lives in it, so the exchange of the later
layers' gradients runs under the backward pass of the earlier ones; ``comm_dtype=torch.bfloat16``
halves the bytes on the wire (the sum is then a bf16 sum).  With ``fused_accumulate=True`` every parameter carries a
``hyc_grad_sink`` callable: a producer that can add its gradient into ``param.grad`` itself (in a GEMM epilogue,
in the kernel that finishes the LoRA-A weight gradient) does so and calls the sink, which counts the parameter in
for its bucket exactly as the accumulation hook would.  Nothing else on the compression path
communicates: every kernel is rank-local and calibration state stays per rank, as in the reference
(its DDP comes implicitly from the HF Trainer)."""
from __future__ import annotations

from typing import Iterable, List

import torch
import torch.distributed as dist


class FlatGradSync:
    def __init__(self, params: Iterable[torch.nn.Parameter], average: bool = True, dtype=None, overlap: bool = False,
                 bucket_bytes: int = 64 << 20, comm_dtype=None, fused_accumulate: bool = False):
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters to synchronise")
        dev = self.params[0].device
        dtype = dtype or self.params[0].dtype
        total = sum(p.numel() for p in self.params)
        self.flat = torch.zeros(total, dtype=dtype, device=dev)
        self.average = average
        off = 0
        for p in self.params:
            n = p.numel()
            p.grad = self.flat[off:off + n].view_as(p) if dtype == p.dtype else None
            off += n
        self._views = dtype == self.params[0].dtype and all(p.dtype == dtype for p in self.params)
        self.comm_dtype = comm_dtype
        # buckets: runs of whole parameters, in parameter order, of at least bucket_bytes each
        self.buckets, self._bucket_of = [], []
        start = off = 0
        members = []
        for i, p in enumerate(self.params):
            members.append(i)
            off += p.numel()
            if (off - start) * self.flat.element_size() >= bucket_bytes or i == len(self.params) - 1:
                self.buckets.append((start, off, members))
                self._bucket_of += [len(self.buckets) - 1] * len(members)
                start, members = off, []
        self.overlap = bool(overlap) and self._views
        self._pending, self._works, self._launched = [], [], []
        self._seen = []
        if self.overlap:
            for i, p in enumerate(self.params):
                p.register_post_accumulate_grad_hook(lambda _p, i=i: self._ready(i))
        # fused_accumulate: producers that know how (the LoRA-A weight gradient kernel, the LoRA-B GEMM of the host's
        # adapter) add their gradient straight into the parameter's view of the flat buffer and call the sink
        # instead of handing the engine a tensor to add -- one elementwise kernel less per parameter and step
        if fused_accumulate and self._views:
            for i, p in enumerate(self.params):
                p.hyc_grad_sink = (lambda i=i: self._ready(i)) if self.overlap else (lambda: None)

    def _active(self) -> bool:
        return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1

    def begin(self):
        """Call before backward (overlap mode): every bucket waits for all of its gradients again."""
        self._pending = [len(m) for _, _, m in self.buckets]
        self._launched = [False] * len(self.buckets)
        self._seen = [False] * len(self.params)
        self._works = []

    def _ready(self, i: int):
        if not self._pending or not self._active():
            return
        # a parameter counts once per backward pass: the accumulation hook may fire for a parameter whose producer
        # has already reported through the sink (the engine runs the hook even when no gradient tensor arrives)
        if self._seen[i]:
            return
        self._seen[i] = True
        b = self._bucket_of[i]
        self._pending[b] -= 1
        if self._pending[b] == 0 and not self._launched[b]:
            self._launch(b)

    def _launch(self, b: int):
        s, e, _ = self.buckets[b]
        self._launched[b] = True
        piece = self.flat[s:e]
        if self.comm_dtype is not None and self.comm_dtype != piece.dtype:
            wire = piece.to(self.comm_dtype)
            self._works.append((dist.all_reduce(wire, op=dist.ReduceOp.SUM, async_op=True), piece, wire))
        else:
            self._works.append((dist.all_reduce(piece, op=dist.ReduceOp.SUM, async_op=True), None, None))

    def numel(self) -> int:
        return self.flat.numel()

    def zero(self):
        self.flat.zero_()

    def _gather_into_flat(self):
        off = 0
        for p in self.params:
            n = p.numel()
            if p.grad is not None and p.grad.data_ptr() != self.flat[off:off + n].data_ptr():
                self.flat[off:off + n].copy_(p.grad.reshape(-1))
            off += n

    def _scatter_from_flat(self):
        off = 0
        for p in self.params:
            n = p.numel()
            if p.grad is not None and p.grad.data_ptr() != self.flat[off:off + n].data_ptr():
                p.grad.copy_(self.flat[off:off + n].view_as(p))
            off += n

    def sync(self, async_op: bool = False):
        """All-reduce the flat gradient buffer (sum, then divide by the world size)."""
        if not self._active():
            return None
        if self.overlap and self._pending:
            # buckets whose parameters got no gradient this step have not been sent yet
            for b in range(len(self.buckets)):
                if not self._launched[b]:
                    self._launch(b)
            for work, piece, wire in self._works:
                work.wait()
                if wire is not None:
                    piece.copy_(wire)
            self._works, self._pending = [], []
            if self.average:
                self.flat.div_(dist.get_world_size())
            return None
        self._gather_into_flat()
        if self.average:
            self.flat.div_(dist.get_world_size())
        work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, async_op=async_op)
        if not async_op:
            self._scatter_from_flat()
        return work
