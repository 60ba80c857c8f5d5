"""``al_std_tiles_static``: the per-tile standard deviation for callers that cannot allocate.

Some users of the library live inside a host that gives them a fixed slice of device memory
at start-up and forbids ``cudaMalloc`` afterwards (it would synchronise the device under the
host's other streams), others are hooks with no allocator at all.  For them the library keeps
the scratch of this one reduction in a built-in device array.  The test drives the new entry
point through the C ABI with torch used only to hold the input and output, and compares with
``al_std_tiles`` (caller-supplied scratch) twice in a row: the second call finds the first
call's partials still in the shared array and must not be disturbed by them.

The file name sorts last on purpose, so that a run that stops at the first failure has
already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ends(sizes):
    acc, out = 0, []
    for s in sizes:
        acc += s
        out.append(acc)
    return (ctypes.c_int32 * len(out))(*out)


def _both(lib, a, sizes, dtype_code):
    rows, k = a.shape
    t = len(sizes)
    ends = _ends(sizes)
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.empty(t, device="cuda", dtype=torch.float32)
    scratch = torch.empty(lib.al_std_scratch_floats(rows, t), device="cuda", dtype=torch.float32)
    assert lib.al_std_tiles(dtype_code, a.data_ptr(), rows, k, ends, t, want.data_ptr(),
                            scratch.data_ptr(), stream) == 0
    got = torch.full((t,), -1.0, device="cuda", dtype=torch.float32)
    status = lib.al_std_tiles_static(dtype_code, a.data_ptr(), rows, k, ends, t, got.data_ptr(), stream)
    assert status == 0, lib.al_last_error()
    torch.cuda.synchronize()
    return got.cpu(), want.cpu()


def test_static_scratch_variant_matches_twice_in_a_row():
    from aihwkit_lightning_b200 import _lib

    lib = _lib.load()
    torch.manual_seed(3)
    # first call: a larger problem that fills many slots of the shared array
    a1 = (torch.randn(4096, 1024, device="cuda") * 2.0 + 0.5).bfloat16()
    got, want = _both(lib, a1, [256] * 4, _lib.AL_BF16)
    assert torch.equal(got, want)
    # second call, different shape and dtype: stale partials of call one are still in the array
    a2 = torch.randn(300, 130, device="cuda") * 0.3
    got, want = _both(lib, a2, [44, 43, 43], _lib.AL_F32)
    assert torch.equal(got, want)
    ref = torch.stack([a2[:, :44].std(), a2[:, 44:87].std(), a2[:, 87:].std()]).cpu()
    assert torch.allclose(got, ref, rtol=1e-5, atol=0)


def test_static_scratch_variant_rejects_oversize():
    from aihwkit_lightning_b200 import _lib

    lib = _lib.load()
    rows = _lib.AL_STD_STATIC_MAX_SEGMENTS // 2 + 1
    a = torch.zeros(rows, 4, device="cuda")
    out = torch.empty(2, device="cuda")
    status = lib.al_std_tiles_static(_lib.AL_F32, a.data_ptr(), rows, 4, _ends([2, 2]), 2, out.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
    assert status == _lib.AL_ERR_TOO_LARGE
    assert b"exceeds the built-in scratch" in lib.al_last_error()
    with pytest.raises(Exception):
        _lib.check(status)
