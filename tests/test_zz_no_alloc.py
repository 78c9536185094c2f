"""The allocation-free channel selection against the ordinary one, through the C ABI.

Some hosts of this library cannot allocate device memory when they call it (a binding
from another language that is only handed raw pointers, or a runtime that froze its
memory plan after start-up).  For them ``hyc_select_channels_noalloc`` keeps its rank
scratch in a fixed array inside the library.  Every call shares that array, so the test
runs the entry point twice in a row, with different inputs, and checks both results
against ``hyc_select_channels``, which takes its scratch from the caller.  This file is
named to be collected last: if it fails under ``-x`` every other test has already run.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _select(lib, score, k, noalloc):
    cols = score.numel()
    out = torch.full((k,), -1, dtype=torch.int32, device=score.device)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if noalloc:
        rc = lib.hyc_select_channels_noalloc(C.c_void_p(score.data_ptr()), cols, k, C.c_void_p(out.data_ptr()), stream)
    else:
        scratch = torch.empty(cols, dtype=torch.int32, device=score.device)
        rc = lib.hyc_select_channels(C.c_void_p(score.data_ptr()), cols, k, C.c_void_p(out.data_ptr()),
                                     C.c_void_p(scratch.data_ptr()), stream)
    torch.cuda.synchronize()
    return rc, out


def test_noalloc_selection_matches_the_allocating_entry_point_twice():
    from hyc_lora_b200 import _lib
    lib = _lib.lib
    gen = torch.Generator().manual_seed(11)
    # the first call on the device also does the one-time address look-up
    # small then large, then large then small (the array still holds the larger call's ranks
    # beyond the smaller call's columns: they must not be read), then exactly the limit
    for cols, k in ((4096, 41), (14336, 287), (4096, 82), (16384, 164)):
        score = torch.rand(cols, generator=gen)
        score[torch.randperm(cols, generator=gen)[:50]] = 2.0      # ties: the lower index must win
        score = score.cuda()
        rc_a, want = _select(lib, score, k, noalloc=False)
        rc_b, got = _select(lib, score, k, noalloc=True)
        assert rc_a == 0 and rc_b == 0
        assert torch.equal(got, want)                                # integer output: exact
        assert bool((got[1:] > got[:-1]).all())                     # ascending, as documented


def test_noalloc_selection_refuses_sizes_beyond_its_fixed_scratch():
    from hyc_lora_b200 import _lib
    lib = _lib.lib
    limit = lib.hyc_select_channels_static_max_cols()
    assert limit == 16384
    score = torch.zeros(limit + 128, device="cuda")
    out = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = lib.hyc_select_channels_noalloc(C.c_void_p(score.data_ptr()), limit + 128, 4, C.c_void_p(out.data_ptr()), None)
    assert rc == -7 and lib.hyc_strerror(rc) == b"size exceeds a stated maximum"


def test_selection_with_nan_and_infinite_scores_writes_exactly_k_entries():
    """A raw caller may hand over any bits.  Every NaN orders above +inf, so the ranks stay a
    total order and the k-entry list is filled exactly, never overrun: the list sits in the
    middle of one allocation whose flanks must come back untouched."""
    from hyc_lora_b200 import _lib
    lib = _lib.lib
    cols, k, flank = 1024, 8, 64
    score = torch.rand(cols)
    score[[0, 5, 17, 300, 301, 700, 701, 702, 900, 1023]] = float("nan")    # more NaNs than k
    score[[1, 2]] = float("inf")
    score[3] = -float("inf")
    score[4] = -0.0
    want = torch.sort(torch.sort(score, descending=True, stable=True).indices[:k]).values.to(torch.int32)
    sd = score.cuda()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for noalloc in (False, True):
        buf = torch.full((flank + k + flank,), -7, dtype=torch.int32, device="cuda")
        out = buf[flank:flank + k]
        if noalloc:
            rc = lib.hyc_select_channels_noalloc(C.c_void_p(sd.data_ptr()), cols, k, C.c_void_p(out.data_ptr()), stream)
        else:
            scratch = torch.empty(cols, dtype=torch.int32, device="cuda")
            rc = lib.hyc_select_channels(C.c_void_p(sd.data_ptr()), cols, k, C.c_void_p(out.data_ptr()),
                                         C.c_void_p(scratch.data_ptr()), stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.equal(out.cpu(), want)
        assert bool((buf[:flank] == -7).all()) and bool((buf[flank + k:] == -7).all())
