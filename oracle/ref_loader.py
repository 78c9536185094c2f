"""Import the reference's own ``operators`` package for pinning the oracle.

TEST INFRASTRUCTURE ONLY.  The modules are imported, unmodified, from the
reference checkout when this machine has one, else from the staged copy that
``oracle/make_ref.py`` leaves under ``oracle/_ref`` (not under version control);
``load()`` returns ``None`` when neither exists, and callers skip.

Two unused imports of the reference need stand-ins to import on a CPU box:
``bitsandbytes.functional`` (operators/efficient_linear.py:2) and the
``.cuda()`` calls on sentinel scalars (operators/compress_function.py:161-163,
338), which are made no-ops while the reference runs on CPU tensors.
"""
from __future__ import annotations

import contextlib
import os
import sys
import types

# the reference checkout: HYC_REFERENCE_ROOT, else a directory named "reference" next to this repository,
# else the staged copy under oracle/_ref
_HERE = os.path.dirname(os.path.abspath(__file__))
_REPO = os.path.dirname(_HERE)
REFERENCE_ROOT = os.environ.get("HYC_REFERENCE_ROOT", os.path.join(os.path.dirname(_REPO), "reference"))
if not os.path.isdir(os.path.join(REFERENCE_ROOT, "operators")) and os.path.isdir(os.path.join(_HERE, "_ref", "operators")):
    REFERENCE_ROOT = os.path.join(_HERE, "_ref")

_cached = None


def available() -> bool:
    return os.path.isdir(os.path.join(REFERENCE_ROOT, "operators"))


def load():
    """Return the reference ``operators`` package, or None if absent."""
    global _cached
    if _cached is not None:
        return _cached
    if not available():
        return None
    for name in ("bitsandbytes", "bitsandbytes.functional"):
        if name not in sys.modules:
            sys.modules[name] = types.ModuleType(name)
    sys.modules["bitsandbytes"].functional = sys.modules["bitsandbytes.functional"]
    # the reference's ``operators`` directory has no __init__.py: register it
    # as a package under a private name so its relative imports resolve
    pkg = types.ModuleType("hyc_reference_operators")
    pkg.__path__ = [os.path.join(REFERENCE_ROOT, "operators")]
    sys.modules["hyc_reference_operators"] = pkg
    import importlib

    for sub in ("compress_function", "efficient_linear", "efficient_silu", "efficient_gelu",
                "efficient_hadamard", "efficient_softmax", "efficient_gemm"):
        setattr(pkg, sub, importlib.import_module(f"hyc_reference_operators.{sub}"))
    _cached = pkg
    return pkg


def load_norms():
    """The reference's three norm modules (Triton kernels inside; importing them needs no GPU, running
    them does), or None when the reference or Triton is absent."""
    pkg = load()
    if pkg is None:
        return None
    import importlib
    try:
        for sub in ("efficient_rmsnorm", "efficient_rmsnorm_gemma", "efficient_layernorm"):
            if not hasattr(pkg, sub):
                setattr(pkg, sub, importlib.import_module(f"hyc_reference_operators.{sub}"))
    except ImportError:
        return None
    return pkg


@contextlib.contextmanager
def cpu_cuda_noop():
    """While active, ``Tensor.cuda()`` returns the tensor itself so the
    reference's sentinel ``torch.tensor(1.).cuda()`` works without a GPU."""
    import torch

    saved = torch.Tensor.cuda
    torch.Tensor.cuda = lambda self, *a, **k: self
    try:
        yield
    finally:
        torch.Tensor.cuda = saved
