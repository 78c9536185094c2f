"""Generate the end-to-end gradient fixtures tests/golden/e2e_*.npz: LoRA gradients of small host
models whose compression operators are the REFERENCE's own classes, run on CPU.

    python tests/golden/make_e2e_golden.py [case ...]      (needs the reference tree; imported in place)

Linear / SiLU / GELU / product / softmax / attention-GEMM sites use the reference's
EfficientMemoryLinear / SiLU / GELU / Hadamard / Softmax / GEMM / GEMMWithSoftmax unchanged.  Its
RMSNorm and LayerNorm need Triton on a GPU, so those two site types are CPU modules that keep the
reference's calibration protocol (fresh statistics on calls 0 and 1, their running mean from call 2
on, operators/efficient_rmsnorm.py:296-339) and call the reference's own get_statistics / compress /
decompress around the restated norm formulas (oracle/hyc_oracle.py: norm_forward, norm_backward).
The hosts are seeded from a CPU generator, so the GPU test rebuilds the identical model and compares
its gradients.

Cases (``CASES``): the decoder in fp32 and in bf16 at 1 024 channels, at INT2 with 2 % outliers, and
with a rank-2 low-rank part at the reference's own preset (8 bits, 0.5 % outliers); the encoder with
every operator of the eager-attention path.  A case with ``calibrate`` runs two calibration steps
first and stores every site's frozen statistics, which the GPU test loads instead of recalibrating
(the randomized SVD does not reproduce across devices)."""
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


def _site(ratio=0.01, bits=4, method="per-channel", rank=0):
    return dict(outlier_ratio=ratio, sub_outlier_ratio=1.0, sub_outlier_bit=bits, sub_outlier_quantize_method=method,
                rank=rank)


CASES = {
    # name: host kind, host config, site settings, seeds, batch, seq, calibration steps before the recorded one
    "decoder": dict(kind="decoder", cfg=dict(hidden=128, layers=2, heads=4, kv_heads=4, ffn=256, vocab=128, lora_r=8,
                                             base_quant="bf16", dtype=torch.float32),
                    site=_site(), seed=11, b_seed=12, batch=2, seq=32, calibrate=0),
    "decoder_bf16": dict(kind="decoder", cfg=dict(hidden=1024, layers=2, heads=8, kv_heads=2, ffn=1536, vocab=256,
                                                  lora_r=8, base_quant="bf16", dtype=torch.bfloat16),
                         site=_site(), seed=21, b_seed=22, batch=2, seq=64, calibrate=0),
    "decoder_int2": dict(kind="decoder", cfg=dict(hidden=256, layers=2, heads=4, kv_heads=2, ffn=512, vocab=128,
                                                  lora_r=8, base_quant="bf16", dtype=torch.float32),
                         site=_site(ratio=0.02, bits=2), seed=31, b_seed=32, batch=2, seq=32, calibrate=0),
    "decoder_rank2": dict(kind="decoder", cfg=dict(hidden=256, layers=2, heads=4, kv_heads=4, ffn=512, vocab=128,
                                                   lora_r=8, base_quant="bf16", dtype=torch.float32),
                          site=_site(ratio=0.005, bits=8, rank=2), seed=41, b_seed=42, batch=2, seq=32, calibrate=2),
    "encoder": dict(kind="encoder", cfg=dict(hidden=768, layers=2, heads=12, ffn=3072, vocab=1000, max_pos=140,
                                             lora_r=16, dtype=torch.float32),
                    site=_site(), softmax_ratio=0.05, seed=51, b_seed=52, batch=2, seq=128, calibrate=0),
}
# kept for callers of the first fixture
CFG, SITE = CASES["decoder"]["cfg"], CASES["decoder"]["site"]


def build_host(device="cpu", case="decoder"):
    c = CASES[case]
    if c["kind"] == "decoder":
        from hyc_lora_b200.hosts.llama import DecoderConfig, DecoderLM
        model = DecoderLM(DecoderConfig(**c["cfg"]), device=device, seed=c["seed"], init_on_cpu=True)
    else:
        from hyc_lora_b200.hosts.roberta import EncoderClassifier, EncoderConfig
        model = EncoderClassifier(EncoderConfig(**c["cfg"]), device=device, seed=c["seed"], init_on_cpu=True)
    g = torch.Generator().manual_seed(c["b_seed"])
    for n, p in model.named_parameters():
        if "lora_B" in n:
            p.data.copy_(torch.empty(p.shape).normal_(0, 0.05, generator=g))
    return model


def inputs(case="decoder"):
    """Positional arguments of the host's forward: (ids,) for the decoder, (ids, labels) for the encoder."""
    c = CASES[case]
    ids = synthetic.token_ids(3 if c["kind"] == "decoder" else 2, c["batch"], c["seq"], c["cfg"]["vocab"])
    if c["kind"] == "decoder":
        return (ids,)
    labels = torch.randint(0, 2, (c["batch"],), generator=torch.Generator().manual_seed(c["b_seed"]))
    return (ids, labels)


STATE_NAMES = ("static_value", "static_value_1", "static_value_2")


def export_calibration(model):
    """{'calib/<module path>/<attribute>[/<slot>]': array} for every module that carries calibration state."""
    out = {}
    for path, m in model.named_modules():
        if not hasattr(m, "iteration"):
            continue
        for name in STATE_NAMES:
            if not hasattr(m, name):
                continue
            v = getattr(m, name)
            if isinstance(v, list):
                for i, t in enumerate(v):
                    out[f"calib/{path}/{name}/{i}"] = t.detach().float().numpy()
            elif v is not None:
                out[f"calib/{path}/{name}"] = v.detach().float().numpy()
    return out


def load_calibration(model, fix, device):
    """Give every operator module of ``model`` the frozen statistics of the fixture (threshold fp32, the rest
    bf16, as the reference holds them) and mark it calibrated."""
    from hyc_lora_b200.operators._common import load_calibration_state_dict
    n = 0
    for path, m in model.named_modules():
        if not hasattr(m, "iteration"):
            continue
        state = {"iteration": 2}
        for name in STATE_NAMES:
            if f"calib/{path}/{name}" in fix:
                state[name] = torch.from_numpy(fix[f"calib/{path}/{name}"]).to(device)
            elif f"calib/{path}/{name}/0" in fix:
                vals = [torch.from_numpy(fix[f"calib/{path}/{name}/{i}"]) for i in range(4)]
                state[name] = [vals[0].to(device)] + [v.to(device=device, dtype=torch.bfloat16) for v in vals[1:]]
        if len(state) > 1:
            load_calibration_state_dict(m, state)
            n += 1
    return n


def _install_reference(model, case):
    ref = ref_loader.load()
    assert ref is not None, "reference tree not found"
    cf = ref.compress_function
    c = CASES[case]
    site = c["site"]

    class RefNormFunc(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, weight, bias, eps, kind, iteration, static_value):
            y, mean, rstd = oc.norm_forward(x, weight, bias, eps, kind)
            if iteration < 2:
                thr, L, R, scale = cf.get_statistics(x, iteration, site["outlier_ratio"], 1.0, site["sub_outlier_bit"],
                                                     site["sub_outlier_quantize_method"], site["rank"])
            else:
                thr, L, scale, R = static_value
            coo, codes, scale = cf.true_divide_outlier_suboutlier_svd_compress(x, thr, scale, site["sub_outlier_bit"],
                                                                               1.0, L, R)
            ctx.saved = (coo, codes, scale, L, R, weight, mean, rstd, kind)
            ctx.mark_non_differentiable(thr, L, R, scale)
            return y, thr, L, R, scale

        @staticmethod
        def backward(ctx, dy, *_):
            coo, codes, scale, L, R, weight, mean, rstd, kind = ctx.saved
            xh = cf.true_divide_outlier_suboutlier_svd_decompress(coo, codes, site["sub_outlier_bit"], scale, L=L, R=R)
            dx, _, _ = oc.norm_backward(xh, dy, weight, mean, rstd, kind, ref_compat_c2=True)
            return dx.to(dy.dtype), None, None, None, None, None, None

    class RefNorm(torch.nn.Module):
        def __init__(self, weight, bias, eps, kind):
            super().__init__()
            self.weight, self.bias, self.eps, self.kind = weight, bias, eps, kind
            self.iteration, self.static_value = 0, [None, None, None, None]

        def forward(self, x):
            y, thr, L, R, scale = RefNormFunc.apply(x, self.weight, self.bias, self.eps, self.kind, self.iteration,
                                                    self.static_value)
            if self.iteration < 2:
                n, s = self.iteration, self.static_value
                s[0] = thr if s[0] is None else (n * s[0] + thr) / (n + 1)
                s[1] = L if s[1] is None else (n * s[1] + cf.pad_cut_L(L, s[1])) / (n + 1)
                s[2] = scale if s[2] is None else (n * s[2] + scale) / (n + 1)
                s[3] = R if s[3] is None else (n * s[3] + R) / (n + 1)
            self.iteration += 1
            return y

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

    double = {f"{k}_{i}": v for k, v in site.items() if k != "rank" for i in (1, 2)}

    def install(module):
        for name, child in module.named_children():
            cls = child.__class__.__name__
            new = None
            if (isinstance(child, torch.nn.Linear) and child.weight.requires_grad and child.in_features > 100
                    and name not in ("lm_head", "class_intermediate", "out_proj", "classifier")):
                new = ref.efficient_linear.EfficientMemoryLinear(child.in_features, child.out_features, bias=False, **site)
                new = new.to(child.weight.dtype)
                new.weight.data = child.weight.data
            elif "SiLU" in cls:
                new = ref.efficient_silu.EfficientMemorySiLU(**site)
            elif "GELU" in cls:
                new = ref.efficient_gelu.EfficientMemoryGELU(**site)
            elif "RMSNorm" in cls:
                new = RefNorm(child.weight, None, child.variance_epsilon, "rms")
            elif "LayerNorm" in cls:
                new = RefNorm(child.weight, child.bias, 1e-5, "ln")      # the reference does not forward eps here
            elif isinstance(child, torch.nn.Softmax):
                new = ref.efficient_softmax.EfficientMemorySoftmax(c["softmax_ratio"])
            elif isinstance(child, torch.nn.Dropout):
                new = torch.nn.Identity()                                 # the reference installs dropout with p = 0
            elif "Hadamard" in cls:
                new = ref.efficient_hadamard.EfficientMemoryHadamard(rank=site["rank"], **double)
                new.forward = _no_empty_cache(new)
            elif "GEMM" in cls:
                if "gemm1" in name:
                    new = ref.efficient_gemm.EfficientMemoryGEMM(rank=site["rank"], **double)
                else:
                    new = ref.efficient_gemm.EfficientMemoryGEMMWithSoftmax(
                        outlier_ratio_1=c["softmax_ratio"], outlier_ratio_2=site["outlier_ratio"],
                        sub_outlier_ratio_2=1.0, sub_outlier_bit_2=site["sub_outlier_bit"],
                        sub_outlier_quantize_method_2=site["sub_outlier_quantize_method"], rank=site["rank"])
            if new is not None:
                setattr(module, name, new)
            else:
                install(child)

    install(model)


def make(case):
    c = CASES[case]
    torch.manual_seed(c["seed"])                      # the randomized SVD of the calibration draws from the global generator
    model = build_host(case=case)
    _install_reference(model, case)
    args = inputs(case)
    out = {}
    with ref_loader.cpu_cuda_noop():
        for _ in range(c["calibrate"]):
            model.zero_grad(set_to_none=True)
            model(*args).backward()
        if c["calibrate"]:
            out.update(export_calibration(model))
        model.zero_grad(set_to_none=True)
        loss = model(*args)
        loss.backward()
    out["loss"] = np.array(loss.item(), dtype=np.float64)
    n = 0
    for name, p in model.named_parameters():
        if p.requires_grad and (c["kind"] == "decoder" or "lora" in name):
            out["grad/" + name] = p.grad.detach().float().numpy()
            n += 1
    path = os.path.join(HERE, f"e2e_{case}.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes;", n, "gradients; loss", loss.item())


def main():
    for case in (sys.argv[1:] or list(CASES)):
        make(case)


if __name__ == "__main__":
    main()
