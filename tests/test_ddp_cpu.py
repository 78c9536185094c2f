"""world_size-2 gloo test (CPU) of the LoRA-gradient exchange: the batch is sharded across
ranks, each rank back-propagates its shard, one flat all-reduce averages the trainable
gradients, and the result equals the single-process gradient of the whole batch."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        g = torch.Generator().manual_seed(5)
        self.base = torch.nn.Parameter(torch.randn(24, 24, generator=g), requires_grad=False)
        self.lora_A = torch.nn.Parameter(0.1 * torch.randn(4, 24, generator=g))
        self.lora_B = torch.nn.Parameter(0.1 * torch.randn(24, 4, generator=g))

    def forward(self, x):
        return ((x @ self.base.t() + x @ self.lora_A.t() @ self.lora_B.t()) ** 2).mean()


class _SelfAccumulating(torch.autograd.Function):
    """h = x W^T whose backward adds the weight gradient into ``W.grad`` itself and reports through the sink --
    what the LoRA-A weight-gradient kernel and the adapter's LoRA-B GEMM do on the GPU."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return x @ w.t()

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        sink = getattr(w, "hyc_grad_sink", None)
        if sink is not None and w.grad is not None:
            w.grad.addmm_(g.t(), x)
            sink()
            return g @ w, None
        return g @ w, g.t() @ x


class _TinyFused(_Tiny):
    def forward(self, x):
        h = _SelfAccumulating.apply(_SelfAccumulating.apply(x, self.lora_A), self.lora_B)
        return ((x @ self.base.t() + h) ** 2).mean()


def _worker(rank, world, port, out, overlap=False, comm_dtype=None, fused=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hyc_lora_b200.ddp import FlatGradSync
    model = _TinyFused() if fused else _Tiny()
    # overlap: one bucket per parameter (the buckets go out from the gradient hooks, during backward)
    # (with the producers reporting themselves: one bucket for both parameters, which must not go out early)
    one_bucket = fused or not overlap
    sync = FlatGradSync(model.parameters(), overlap=overlap, bucket_bytes=64 << 20 if one_bucket else 64, comm_dtype=comm_dtype,
                        fused_accumulate=fused)
    assert sync.numel() == 4 * 24 * 2 and len(sync.buckets) == (1 if one_bucket else 2)
    reported = set()
    if fused:
        # a bucket may go out only when the producers of all its gradients have reported (checked where it is sent:
        # with an asynchronous all-reduce a bucket that left early could still come out right by timing)
        params = list(model.parameters())
        for i, p in enumerate([q for q in params if q.requires_grad]):
            inner = p.hyc_grad_sink
            p.hyc_grad_sink = lambda i=i, inner=inner: (reported.add(i), inner())[1]
        send = sync._launch

        def checked_send(b):
            assert all(i in reported for i in sync.buckets[b][2]), "bucket sent before its gradients were in"
            return send(b)
        sync._launch = checked_send
    x = torch.randn(8, 24, generator=torch.Generator().manual_seed(9))
    for step in range(2):                       # second step: the flat buffer is reused after zero()
        reported.clear()
        sync.zero()
        loss = model(x[rank * 4:(rank + 1) * 4])
        sync.begin()
        loss.backward()
        if overlap:
            assert all(sync._launched)          # every bucket was sent by a hook before sync()
        sync.sync()
    if rank == 0:
        out.put((model.lora_A.grad.clone(), model.lora_B.grad.clone()))
    dist.barrier()
    dist.destroy_process_group()


import pytest


# fused: the producers add their gradients into the flat buffer themselves and report through the sink; the
# accumulation hook of such a parameter may fire as well, and the parameter must still count once (one bucket holds
# both parameters in these cases: counted twice, it would go out before the second gradient is in)
@pytest.mark.parametrize("overlap,comm_dtype,atol,fused", [
    (False, None, 1e-6, False), (True, None, 1e-6, False), (True, torch.bfloat16, 2e-3, False),
    (True, None, 1e-6, True), (False, None, 1e-6, True)])
def test_flat_gradient_allreduce_matches_single_process(overlap, comm_dtype, atol, fused):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out, overlap, comm_dtype, fused)) for r in range(2)]
    for p in procs:
        p.start()
    ga, gb = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    ref = _Tiny()
    x = torch.randn(8, 24, generator=torch.Generator().manual_seed(9))
    # each rank's loss is the mean over ITS shard; averaging the ranks gives the mean over the batch
    (0.5 * ref(x[:4]) + 0.5 * ref(x[4:])).backward()
    assert torch.allclose(ga, ref.lora_A.grad, atol=atol) and torch.allclose(gb, ref.lora_B.grad, atol=atol)


def test_flat_buffer_views_and_single_process_noop():
    from hyc_lora_b200.ddp import FlatGradSync
    m = _Tiny()
    sync = FlatGradSync(m.parameters())
    m(torch.ones(2, 24)).backward()
    assert m.lora_A.grad.data_ptr() == sync.flat.data_ptr()          # gradients accumulate straight into the flat buffer
    assert sync.flat.abs().sum() > 0 and sync.sync() is None
