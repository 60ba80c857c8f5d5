"""The C-ABI library loads and exports every symbol ``include/analog_b200.h`` declares
(no compute calls: this runs without a GPU)."""
import ctypes
import os
import re

import pytest

from aihwkit_lightning_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "analog_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(al_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_functions() == sorted(_lib.SYMBOLS)


def test_library_exports_every_symbol():
    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("library not built (python aihwkit-lightning_b200/build.py)")
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), name
    lib.al_version.restype = ctypes.c_int32
    assert lib.al_version() >= 1
    lib.al_status_str.restype = ctypes.c_char_p
    assert lib.al_status_str(0) == b"ok"
    assert b"timed out" in lib.al_status_str(4)


def test_struct_sizes_match_the_header():
    """AlDesc mixes int32 and double fields: the ctypes mirror must agree with the C layout."""
    import subprocess
    import tempfile

    src = '#include "analog_b200.h"\n#include <stdio.h>\nint main(){printf("%zu %zu %zu\\n", sizeof(AlDesc), sizeof(AlForwardArgs), sizeof(AlBackwardArgs));return 0;}\n'
    with tempfile.TemporaryDirectory() as tmp:
        c_file = os.path.join(tmp, "s.c")
        open(c_file, "w").write(src)
        exe = os.path.join(tmp, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c_file, "-o", exe])
        sizes = [int(v) for v in subprocess.check_output([exe]).split()]
    assert sizes == [ctypes.sizeof(_lib.AlDesc), ctypes.sizeof(_lib.AlForwardArgs),
                     ctypes.sizeof(_lib.AlBackwardArgs)]


def test_bad_arguments_are_rejected_without_a_gpu():
    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("library not built")
    lib = _lib.load()
    assert lib.al_forward(None, None, None) == _lib.AL_ERR_BAD_ARGUMENT
    desc = _lib.AlDesc()
    desc.M, desc.K, desc.N, desc.T = 4, 8, 4, 1
    desc.dtype = 7
    args = _lib.AlForwardArgs()
    assert lib.al_forward(desc, args, None) == _lib.AL_ERR_BAD_ARGUMENT
    desc.dtype = 0
    desc.inp_res = 254.0  # DAC without an input range
    assert lib.al_forward(desc, args, None) == _lib.AL_ERR_BAD_ARGUMENT
    assert b"input range" in lib.al_last_error()
    desc.inp_res = -1.0
    ends = (ctypes.c_int32 * 1)(7)  # last end != K
    args.tile_ends = ends
    assert lib.al_forward(desc, args, None) == _lib.AL_ERR_BAD_ARGUMENT
    with pytest.raises(AssertionError):
        _lib.check(_lib.AL_ERR_BAD_ARGUMENT)
