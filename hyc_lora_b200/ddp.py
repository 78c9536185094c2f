"""Data parallelism for the LoRA path: one process per GPU, the batch sharded across ranks,
and ONE exchange step -- the sum of the trainable (LoRA) gradients -- on NCCL.

The gradients of all trainable parameters live in a single flat fp32 buffer (each ``.grad`` is
a view into it), so the exchange is one large all-reduce that NCCL can run through NVSwitch
(in-switch reduction when available) instead of hundreds of small ones.  Nothing else on the
compression path communicates: every kernel is rank-local and calibration state stays per
rank, as in the reference (its DDP comes implicitly from the HF Trainer)."""
from __future__ import annotations

from typing import Iterable, List

import torch
import torch.distributed as dist


class FlatGradSync:
    def __init__(self, params: Iterable[torch.nn.Parameter], average: bool = True, dtype=None):
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
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            return None
        self._gather_into_flat()
        if self.average:
            self.flat.div_(dist.get_world_size())
        work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, async_op=async_op)
        if not async_op:
            self._scatter_from_flat()
        return work
