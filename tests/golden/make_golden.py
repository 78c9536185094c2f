"""Generate the golden fixtures in this directory from the reference's own code.

Run on a machine that has the reference tree (read-only, imported in place):

    python tests/golden/make_golden.py

Outputs (committed):
  r_mode_small.npz   compress/decompress of small seeded tensors for every
                     (dtype, bits, scale method) and a few low-rank cases
  c1_roundtrip.npz   configuration 1 ([8,128,768] fp32, LayerNorm input, INT4
                     per-token): statistics, codes, outlier COO, reconstruction
                     (batch element 0 plus a SHA-256 of the whole tensor) and the
                     LoRA-A dA / dX of the reference's linear operator
bf16 tensors are stored as their int16 bit patterns (suffix ``_bf16``).
"""
import hashlib
import itertools
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ref_loader  # noqa: E402
from hyc_lora_b200 import synthetic  # noqa: E402


def bits_of(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.contiguous().numpy()


def small_input(dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(2, 16, 128, generator=g)
    idx = torch.randperm(128, generator=g)[:3]
    x[..., idx] *= 25.0
    return x.to(dtype)


def main():
    ref = ref_loader.load()
    assert ref is not None, "reference tree not found"
    cf = ref.compress_function
    out = {}
    names = []
    cases = [(dt, b, m, 0) for dt, b, m in itertools.product(
        ["bf16", "fp32"], [1, 2, 4, 8], ["per-tensor", "per-channel", "per-token"])]
    cases += [("bf16", 4, "per-channel", 2), ("fp32", 4, "per-token", 2), ("bf16", 8, "per-tensor", 2),
              ("bf16", 2, "per-channel", 2)]
    with ref_loader.cpu_cuda_noop():
        for i, (dt, bits, method, rank) in enumerate(cases):
            dtype = torch.bfloat16 if dt == "bf16" else torch.float32
            x = small_input(dtype, 500 + i)
            torch.manual_seed(77 + i)
            thr, L, R, scale = cf.get_statistics(x, 0, 0.02, 1.0, bits, method, rank)
            coo, codes, _ = cf.true_divide_outlier_suboutlier_svd_compress(x, thr, scale, bits, 1.0, L, R)
            xh = cf.true_divide_outlier_suboutlier_svd_decompress(coo, codes, bits, scale, L=L, R=R)
            coo = coo.coalesce()
            name = f"{dt}_b{bits}_{method}_r{rank}"
            names.append(name)
            key = "x_bf16" if dt == "bf16" else "x"
            out[f"{name}/{key}"] = bits_of(x)
            out[f"{name}/thr"] = thr.numpy()
            out[f"{name}/scale_bf16"] = bits_of(scale)
            out[f"{name}/L_bf16"] = bits_of(L)
            out[f"{name}/R_bf16"] = bits_of(R)
            out[f"{name}/codes"] = codes.numpy()
            out[f"{name}/coo_index"] = coo.indices().numpy().astype(np.int32)
            out[f"{name}/coo_value_bf16"] = bits_of(coo.values())
            out[f"{name}/xhat_bf16"] = bits_of(xh)
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "r_mode_small.npz"), **out)

    # configuration 1
    x, planted = synthetic.roundtrip_activation()
    a, grad = synthetic.lora_a_problem()
    c1 = {"x_sha256": np.array(hashlib.sha256(x.numpy().tobytes()).hexdigest()),
          "planted": planted.numpy()}
    with ref_loader.cpu_cuda_noop():
        thr, L, R, scale = cf.get_statistics(x, 0, 0.01, 1.0, 4, "per-token", 0)
        coo, codes, _ = cf.true_divide_outlier_suboutlier_svd_compress(x, thr, scale, 4, 1.0, L, R)
        xh = cf.true_divide_outlier_suboutlier_svd_decompress(coo, codes, 4, scale, L=L, R=R)
        coo = coo.coalesce()
        xin = x.clone().requires_grad_(True)
        w = a.clone().requires_grad_(True)
        res = ref.efficient_linear.EfficientMemoryLinearFunc.apply(
            xin, w, None, False, 0.01, 1.0, 4, "per-token", 0, 0, [None] * 4)
        res[0].backward(grad)
    c1.update({
        "thr": thr.numpy(), "scale_bf16": bits_of(scale), "codes": codes.numpy(),
        "coo_flat": (coo.indices()[0] * (128 * 768) + coo.indices()[1] * 768 + coo.indices()[2]).numpy().astype(np.int32),
        "coo_value_bf16": bits_of(coo.values()),
        "xhat_sha256": np.array(hashlib.sha256(bits_of(xh).tobytes()).hexdigest()),
        "xhat0_bf16": bits_of(xh[0]),
        "dX_sha256": np.array(hashlib.sha256(xin.grad.numpy().tobytes()).hexdigest()),
        "dX0": xin.grad[0, :8].numpy(), "dA": w.grad.numpy(),
    })
    np.savez_compressed(os.path.join(HERE, "c1_roundtrip.npz"), **c1)
    for f in ("r_mode_small.npz", "c1_roundtrip.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
