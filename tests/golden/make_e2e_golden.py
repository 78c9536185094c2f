"""Generate tests/golden/e2e_decoder.npz: LoRA gradients of a two-layer decoder host whose
compression operators are the REFERENCE's own classes, run on CPU in fp32.

    python tests/golden/make_e2e_golden.py          (needs the reference tree; imported in place)

Linear / SiLU / product sites use the reference's EfficientMemoryLinear / SiLU / Hadamard
unchanged.  Its RMSNorm needs Triton on a GPU, so that one site type is a CPU Function built
from the reference's compress / decompress calls around the restated norm formulas
(oracle/hyc_oracle.py: norm_forward, norm_backward).  The host is seeded from a CPU
generator, so the GPU test rebuilds the identical model and compares its gradients."""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import hyc_oracle as oc  # noqa: E402
from oracle import ref_loader  # noqa: E402
from hyc_lora_b200 import synthetic  # noqa: E402

CFG = dict(hidden=128, layers=2, heads=4, kv_heads=4, ffn=256, vocab=128, lora_r=8, base_quant="bf16",
           dtype=torch.float32)
SITE = dict(outlier_ratio=0.01, sub_outlier_ratio=1.0, sub_outlier_bit=4, sub_outlier_quantize_method="per-channel",
            rank=0)
SEED, B_SEED, BATCH, SEQ = 11, 12, 2, 32


def build_host(device="cpu"):
    from hyc_lora_b200.hosts.llama import DecoderConfig, DecoderLM
    model = DecoderLM(DecoderConfig(**CFG), device=device, seed=SEED, init_on_cpu=True)
    g = torch.Generator().manual_seed(B_SEED)
    for n, p in model.named_parameters():
        if "lora_B" in n:
            p.data.copy_(torch.empty(p.shape).normal_(0, 0.05, generator=g))
    return model


def inputs():
    return synthetic.token_ids(3, BATCH, SEQ, CFG["vocab"])


def main():
    ref = ref_loader.load()
    assert ref is not None, "reference tree not found"
    cf = ref.compress_function

    class RefRMSNormFunc(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, weight, eps):
            y, _, rstd = oc.norm_forward(x, weight, None, eps, "rms")
            thr, L, R, scale = cf.get_statistics(x, 0, SITE["outlier_ratio"], 1.0, SITE["sub_outlier_bit"],
                                                 SITE["sub_outlier_quantize_method"], 0)
            coo, codes, scale = cf.true_divide_outlier_suboutlier_svd_compress(x, thr, scale, SITE["sub_outlier_bit"],
                                                                               1.0, L, R)
            ctx.saved = (coo, codes, scale, L, R, weight, rstd)
            return y

        @staticmethod
        def backward(ctx, dy):
            coo, codes, scale, L, R, weight, rstd = ctx.saved
            xh = cf.true_divide_outlier_suboutlier_svd_decompress(coo, codes, SITE["sub_outlier_bit"], scale, L=L, R=R)
            dx, _, _ = oc.norm_backward(xh, dy, weight, None, rstd, "rms", ref_compat_c2=True)
            return dx.to(dy.dtype), None, None

    class RefRMSNorm(torch.nn.Module):
        def __init__(self, weight, eps):
            super().__init__()
            self.weight, self.eps = weight, eps

        def forward(self, x):
            return RefRMSNormFunc.apply(x, self.weight, self.eps)

    def install(module):
        for name, child in module.named_children():
            cls = child.__class__.__name__
            new = None
            if isinstance(child, torch.nn.Linear) and child.weight.requires_grad and child.in_features > 100:
                new = ref.efficient_linear.EfficientMemoryLinear(child.in_features, child.out_features, bias=False, **SITE)
                new.weight.data = child.weight.data
            elif "SiLU" in cls:
                new = ref.efficient_silu.EfficientMemorySiLU(**SITE)
            elif "RMSNorm" in cls:
                new = RefRMSNorm(child.weight, child.variance_epsilon)
            elif "Hadamard" in cls:
                kw = {f"{k}_{i}": v for k, v in SITE.items() if k != "rank" for i in (1, 2)}
                new = ref.efficient_hadamard.EfficientMemoryHadamard(rank=0, **kw)
                new.forward = _no_empty_cache(new)
            if new is not None:
                setattr(module, name, new)
            else:
                install(child)

    def _no_empty_cache(mod):
        fwd = mod.forward

        def wrapped(x1, x2):
            saved = torch.cuda.empty_cache
            torch.cuda.empty_cache = lambda: None
            try:
                return fwd(x1, x2)
            finally:
                torch.cuda.empty_cache = saved
        return wrapped

    model = build_host()
    install(model)
    ids = inputs()
    with ref_loader.cpu_cuda_noop():
        loss = model(ids)
        loss.backward()
    out = {"loss": np.array(loss.item(), dtype=np.float64)}
    for n, p in model.named_parameters():
        if p.requires_grad:
            out["grad/" + n] = p.grad.detach().float().numpy()
    path = os.path.join(HERE, "e2e_decoder.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes;", len(out) - 1, "gradients; loss", loss.item())


if __name__ == "__main__":
    main()
