"""Readers for the fixtures under tests/golden/ (see make_golden.py there)."""
import hashlib
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _t(a, bf16=False):
    t = torch.from_numpy(np.array(a, copy=True))  # keeps 0-dim shapes
    return t.view(torch.bfloat16) if bf16 else t


class Case(dict):
    __getattr__ = dict.__getitem__


def small_cases():
    z = np.load(os.path.join(GOLDEN, "r_mode_small.npz"))
    for name in z["names"]:
        name = str(name)
        dt, b, method, r = name.split("_")
        c = Case(name=name, dtype=dt, bits=int(b[1:]), method=method, rank=int(r[1:]))
        c["x"] = _t(z[f"{name}/x_bf16"], True) if dt == "bf16" else _t(z[f"{name}/x"])
        c["thr"] = _t(z[f"{name}/thr"])
        c["scale"] = _t(z[f"{name}/scale_bf16"], True)
        c["L"] = _t(z[f"{name}/L_bf16"], True)
        c["R"] = _t(z[f"{name}/R_bf16"], True)
        c["codes"] = _t(z[f"{name}/codes"])
        c["coo_index"] = _t(z[f"{name}/coo_index"]).long()
        c["coo_value"] = _t(z[f"{name}/coo_value_bf16"], True)
        c["xhat"] = _t(z[f"{name}/xhat_bf16"], True)
        yield c


def config1():
    z = np.load(os.path.join(GOLDEN, "c1_roundtrip.npz"))
    c = Case()
    for k in ("thr", "codes", "coo_flat", "planted", "dA", "dX0"):
        c[k] = _t(z[k])
    for k in ("scale", "coo_value", "xhat0"):
        c[k] = _t(z[k + "_bf16"], True)
    for k in ("x_sha256", "xhat_sha256", "dX_sha256"):
        c[k] = str(z[k])
    return c


def sha_bits(t: torch.Tensor) -> str:
    a = t.contiguous().view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.contiguous().numpy()
    return hashlib.sha256(a.tobytes()).hexdigest()
