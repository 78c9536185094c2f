"""No-GPU checks of the C-ABI library: it loads, exports every symbol the header
declares, and rejects bad arguments with error codes before touching CUDA."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "hyc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hyc_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from hyc_lora_b200 import build
    build.build()
    from hyc_lora_b200 import _lib
    return _lib


def test_header_symbols_are_exported_and_bound(lib):
    declared = _declared_symbols()
    assert len(declared) >= 12
    raw = C.CDLL(lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), f"{name} declared in include/hyc_b200.h but not exported"
        assert name in lib.SYMBOLS, f"{name} has no ctypes signature in _lib.SYMBOLS"
    assert sorted(lib.SYMBOLS) == declared


def test_error_strings(lib):
    assert lib.lib.hyc_strerror(0) == b"ok"
    for code in range(-9, 0):
        assert lib.lib.hyc_strerror(code) != b"unknown error code"
    assert lib.lib.hyc_strerror(-99) == b"unknown error code"
    assert lib.lib.hyc_version() >= 100
    assert lib.lib.hyc_norm_bwd_partial_rows() > 0


def test_tuning_validation(lib):
    assert lib.lib.hyc_set_tuning(0, 0, 0) == 0
    assert lib.lib.hyc_set_tuning(48, 0, 0) == -2
    assert lib.lib.hyc_set_tuning(128, 9, 0) == -2
    assert lib.lib.hyc_set_tuning(0, 0, 0) == 0


def _packed(lib, **kw):
    p = lib.HycPacked()
    p.mode, p.bits, p.rows, p.cols, p.seq = lib.HYC_MODE_N, 4, 4, 256, 4
    p.codes = 0x1000
    p.scales = 0x2000
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def _dense(lib, **kw):
    d = lib.HycDense()
    d.base, d.dtype, d.chunks, d.row_stride = 0x4000, lib.HYC_BF16, 1, 256
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_argument_errors_come_back_as_codes(lib):
    f = lib.lib.hyc_compress
    ok_d = _dense(lib)
    assert f(None, C.byref(_packed(lib)), None) == -1 or f(None, C.byref(_packed(lib)), None) < 0
    assert f(C.byref(ok_d), C.byref(_packed(lib, codes=None)), None) == -1
    assert f(C.byref(ok_d), C.byref(_packed(lib, cols=200)), None) == -2
    assert f(C.byref(ok_d), C.byref(_packed(lib, bits=3)), None) == -3
    assert f(C.byref(ok_d), C.byref(_packed(lib, bits=1)), None) == -3      # 1 bit is reference-mode only
    assert f(C.byref(ok_d), C.byref(_packed(lib, mode=7)), None) == -5
    assert f(C.byref(ok_d), C.byref(_packed(lib, codes=0x1004)), None) == -6
    assert f(C.byref(ok_d), C.byref(_packed(lib, group=64)), None) == -2
    assert f(C.byref(ok_d), C.byref(_packed(lib, rotate=512)), None) == -2
    assert f(C.byref(ok_d), C.byref(_packed(lib, rotate=1024)), None) == -2  # does not divide 256
    assert f(C.byref(_dense(lib, dtype=5)), C.byref(_packed(lib)), None) == -4
    assert f(C.byref(_dense(lib, base=0x4008)), C.byref(_packed(lib)), None) == -6
    assert f(C.byref(_dense(lib, chunks=3)), C.byref(_packed(lib)), None) == -2
    r = _packed(lib, mode=lib.HYC_MODE_R, scale_dtype=lib.HYC_BF16)
    assert f(C.byref(ok_d), C.byref(r), None) == -1                          # no scale / pool
    assert lib.lib.hyc_norm_compress(C.byref(ok_d), None, C.byref(_packed(lib)), None) == -1
    assert lib.lib.hyc_act_bwd(9, C.byref(_packed(lib)), None, 0x10, 1, 0x10, None, None) == -5
    assert lib.lib.hyc_decompress(C.byref(_packed(lib)), C.byref(_dense(lib, dtype=lib.HYC_F32)), None) == -4
    assert lib.lib.hyc_select_channels(0x10, 256, 300, 0x10, 0x10, None) == -2


def test_zero_rows_is_a_no_op(lib):
    # rows == 0 returns before any CUDA call, so it is safe without a device
    assert lib.lib.hyc_compress(C.byref(_dense(lib)), C.byref(_packed(lib, rows=0)), None) == 0
    assert lib.lib.hyc_decompress(C.byref(_packed(lib, rows=0)), C.byref(_dense(lib)), None) == 0


def test_python_callers_refuse_cpu_tensors(lib):
    import torch
    from hyc_lora_b200 import packed
    with pytest.raises(RuntimeError, match="no CPU path"):
        packed.compress_n(torch.zeros(4, 256, dtype=torch.bfloat16), None, 4)
