"""B200-native activation compress / decompress+grad kernels behind the
HyC-LoRA operator interface.

Sub-modules:
  build       compile the CUDA library in-tree (no GPU needed)
  _lib        ctypes binding of the C ABI (include/hyc_b200.h); raises if the library is missing
  packed      packed-activation records and Python callers of the C ABI
  operators   drop-in ``EfficientMemory*`` modules / autograd Functions
  synthetic   seeded synthetic inputs shaped like the benchmark configurations

Importing the package itself loads nothing heavy, so ``python -m
hyc_lora_b200.build`` works before the library exists.
"""
__version__ = "0.1.0"


OPERATOR_MODULES = ("compress_function", "efficient_linear", "efficient_rmsnorm", "efficient_rmsnorm_gemma",
                    "efficient_layernorm", "efficient_silu", "efficient_gelu", "efficient_hadamard",
                    "efficient_softmax", "efficient_gemm", "efficient_dropout")


def install_as_operators(name: str = "operators"):
    """Register this package's operator modules under the top-level name the reference's
    drivers import from (``from operators.efficient_linear import EfficientMemoryLinear``,
    train_gsm8k.py:18-27), so those import lines work unchanged.  Returns the package."""
    import importlib
    import sys

    pkg = importlib.import_module(__name__ + ".operators")
    sys.modules[name] = pkg
    for sub in OPERATOR_MODULES:
        sys.modules[f"{name}.{sub}"] = importlib.import_module(f"{__name__}.operators.{sub}")
    return pkg
