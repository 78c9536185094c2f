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
