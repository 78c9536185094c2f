"""ctypes binding of libhyc_b200.so (the C ABI declared in include/hyc_b200.h).

The library is built in-tree by ``python -m hyc_lora_b200.build``.  There is no
fallback: if the shared object is missing or a symbol is absent, importing
this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhyc_b200.so")

HYC_OK = 0
HYC_ERR_SHAPE = -2
HYC_F32, HYC_BF16 = 0, 1
HYC_MODE_R, HYC_MODE_N = 0, 1
HYC_SCALE_TENSOR, HYC_SCALE_CHANNEL, HYC_SCALE_TOKEN = 0, 1, 2
HYC_NORM_RMS, HYC_NORM_RMS_GEMMA, HYC_NORM_LAYER = 0, 1, 2
HYC_ACT_SILU, HYC_ACT_GELU_TANH, HYC_ACT_PRODUCT = 0, 1, 2
HYC_STATUS_POOL_OVERFLOW, HYC_STATUS_WAIT_EXPIRED = 1, 2


class HycPacked(C.Structure):
    _fields_ = [
        ("mode", C.c_int32), ("bits", C.c_int32),
        ("rows", C.c_int64),
        ("cols", C.c_int32), ("seq", C.c_int32),
        ("codes", C.c_void_p),
        ("status", C.c_void_p),
        ("scale_kind", C.c_int32), ("scale_dtype", C.c_int32),
        ("scale", C.c_void_p),
        ("thr", C.c_void_p),
        ("lowrank", C.c_void_p),
        ("pool", C.c_void_p),
        ("pool_cap", C.c_uint32),
        ("pool_used", C.c_void_p),
        ("row_meta", C.c_void_p),
        ("channels", C.c_void_p),
        ("n_channels", C.c_int32), ("group", C.c_int32), ("rotate", C.c_int32), ("_pad", C.c_int32),
        ("out_value", C.c_void_p),
        ("scales", C.c_void_p),
    ]


class HycDense(C.Structure):
    _fields_ = [
        ("base", C.c_void_p),
        ("dtype", C.c_int32), ("chunks", C.c_int32),
        ("row_stride", C.c_int64), ("batch_stride", C.c_int64), ("chunk_stride", C.c_int64),
    ]


class HycNormFwd(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("eps", C.c_float),
        ("weight", C.c_void_p), ("bias", C.c_void_p),
        ("param_dtype", C.c_int32), ("_pad", C.c_int32),
        ("y", C.c_void_p), ("rstd", C.c_void_p), ("mean", C.c_void_p),
    ]


class HycNormBwdArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("ref_compat_c2", C.c_int32),
        ("weight", C.c_void_p),
        ("param_dtype", C.c_int32), ("dy_dtype", C.c_int32),
        ("dy", C.c_void_p), ("rstd", C.c_void_p), ("mean", C.c_void_p),
        ("dx", C.c_void_p), ("dweight", C.c_void_p), ("dbias", C.c_void_p), ("partials", C.c_void_p),
    ]


class HycSparseRows(C.Structure):
    _fields_ = [
        ("rows", C.c_int64), ("cols", C.c_int32), ("dtype", C.c_int32),
        ("val", C.c_void_p), ("col", C.c_void_p),
        ("cap", C.c_uint32), ("_pad", C.c_uint32),
        ("used", C.c_void_p), ("row_meta", C.c_void_p), ("status", C.c_void_p),
    ]


# every symbol include/hyc_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "hyc_strerror": (C.c_char_p, [C.c_int]),
    "hyc_last_cuda_error": (C.c_char_p, []),
    "hyc_version": (C.c_int, []),
    "hyc_launch_count": (C.c_uint64, []),
    "hyc_set_tuning": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "hyc_debug_wait": (C.c_int, [C.c_int64, C.c_uint32]),
    "hyc_compress": (C.c_int, [C.POINTER(HycDense), C.POINTER(HycPacked), C.c_void_p]),
    "hyc_decompress": (C.c_int, [C.POINTER(HycPacked), C.POINTER(HycDense), C.c_void_p]),
    "hyc_norm_compress": (C.c_int, [C.POINTER(HycDense), C.POINTER(HycNormFwd), C.POINTER(HycPacked), C.c_void_p]),
    "hyc_norm_compress2": (C.c_int, [C.POINTER(HycDense), C.POINTER(HycNormFwd), C.POINTER(HycPacked), C.POINTER(HycPacked),
                                     C.c_void_p]),
    "hyc_act_compress": (C.c_int, [C.POINTER(HycDense), C.c_int, C.c_void_p, C.POINTER(HycPacked), C.POINTER(HycPacked),
                                   C.c_void_p]),
    "hyc_product_compress": (C.c_int, [C.POINTER(HycDense), C.POINTER(HycDense), C.c_void_p, C.POINTER(HycPacked),
                                       C.POINTER(HycPacked), C.c_void_p]),
    "hyc_norm_bwd_partial_rows": (C.c_int, []),
    "hyc_norm_bwd": (C.c_int, [C.POINTER(HycPacked), C.POINTER(HycNormBwdArgs), C.c_void_p]),
    "hyc_act_bwd": (C.c_int, [C.c_int, C.POINTER(HycPacked), C.POINTER(HycPacked), C.c_void_p, C.c_int,
                              C.c_void_p, C.c_void_p, C.c_void_p]),
    "hyc_channel_absmax": (C.c_int, [C.POINTER(HycDense), C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "hyc_select_channels": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hyc_lora_wgrad_scratch_floats": (C.c_int64, [C.POINTER(HycPacked), C.c_int32]),
    "hyc_lora_wgrad": (C.c_int, [C.POINTER(HycPacked), C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hyc_lora_wgrad_to": (C.c_int, [C.POINTER(HycPacked), C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
                                    C.c_void_p, C.c_void_p]),
    "hyc_softmax_compact": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(HycSparseRows), C.c_void_p]),
    "hyc_softmax_expand": (C.c_int, [C.POINTER(HycSparseRows), C.c_void_p, C.c_void_p]),
    "hyc_softmax_bwd": (C.c_int, [C.POINTER(HycSparseRows), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "hyc_nf4_dequant": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "hyc_rope": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                           C.c_int32, C.c_void_p]),
    "hyc_select_channels_static_max_cols": (C.c_int, []),
    "hyc_select_channels_noalloc": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
}


class HycError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m hyc_lora_b200.build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(code: int, what: str) -> None:
    if code != HYC_OK:
        msg = lib.hyc_strerror(code).decode()
        if code == -8:
            msg += ": " + lib.hyc_last_cuda_error().decode()
        raise HycError(f"{what} failed ({code}): {msg}")
