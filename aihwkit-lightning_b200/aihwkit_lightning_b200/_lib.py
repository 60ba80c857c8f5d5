"""ctypes binding of ``libanalog_b200.so`` (C ABI in ``include/analog_b200.h``).

There is no CPU fallback: if the library is missing the first call raises, naming the build
command.  Nothing in here touches torch; callers pass raw device pointers and a stream handle.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int32, c_int64, c_uint32, c_uint64, c_void_p

from .exceptions import ConfigError, KernelError

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libanalog_b200.so")

AL_F32, AL_BF16 = 0, 1
AL_IR_OFF, AL_IR_STATIC, AL_IR_DYNAMIC, AL_IR_FAST = 0, 1, 2, 3
AL_ENGINE_AUTO, AL_ENGINE_SIMT, AL_ENGINE_TCGEN05, AL_ENGINE_TCGEN05_PAIR, AL_ENGINE_TCGEN05_SINGLE = 0, 1, 2, 3, 4
(AL_OK, AL_ERR_BAD_ARGUMENT, AL_ERR_UNSUPPORTED, AL_ERR_CUDA, AL_ERR_DEVICE_TIMEOUT,
 AL_ERR_TOO_LARGE) = range(6)


class AlDesc(Structure):
    _fields_ = [
        ("M", c_int32), ("K", c_int32), ("N", c_int32), ("T", c_int32),
        ("dtype", c_int32), ("training", c_int32), ("ir_mode", c_int32),
        ("init_from_data", c_int32),
        ("init_std_alpha", c_double), ("decay", c_double), ("input_min_percentage", c_double),
        ("act_range_momentum", c_double),
        ("inp_res", c_double), ("out_res", c_double), ("out_bound", c_double),
        ("out_noise", c_double),
        ("out_noise_per_channel", c_int32), ("noise_type", c_int32), ("quant_type", c_int32),
        ("std_dev", c_double), ("mod_res", c_double),
        ("clip_type", c_int32), ("no_rounding", c_int32), ("ref_rounding", c_int32),
        ("engine", c_int32), ("save_for_backward", c_int32),
    ]


class AlForwardArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("bias", c_void_p),
        ("input_range", c_void_p), ("input_range_update_idx", c_void_p),
        ("x_min", c_void_p), ("x_max", c_void_p), ("learnable_weight_clip", c_void_p),
        ("tile_ends", POINTER(c_int32)),
        ("out", c_void_p), ("xq", c_void_p), ("ir_rows", c_void_p), ("w_amax", c_void_p),
        ("w_tile_max", c_void_p), ("w_mod", c_void_p), ("keep_mask", c_void_p),
        ("std_scratch", c_void_p), ("std_override", c_void_p), ("smallm_scratch", c_void_p),
        ("codes16", c_void_p), ("w_planes", c_void_p), ("w_noise", c_void_p), ("out_noise", c_void_p),
        ("codes", c_void_p), ("seed", c_uint64), ("offset", c_uint64), ("x_prequantised", c_int32),
        ("offset_base", c_void_p),
    ]


class AlBackwardArgs(Structure):
    _fields_ = [
        ("grad_out", c_void_p), ("x", c_void_p), ("xq", c_void_p), ("w_mod", c_void_p),
        ("ir_rows", c_void_p), ("keep_mask", c_void_p), ("tile_ends", POINTER(c_int32)),
        ("grad_x", c_void_p), ("grad_w", c_void_p), ("grad_bias", c_void_p),
        ("grad_input_range", c_void_p), ("reduce_scratch", c_void_p), ("reduce_scratch_floats", c_int64),
        ("codes16", c_void_p), ("w_planes", c_void_p), ("g_planes", c_void_p), ("g_planes_elems", c_int64),
        ("w", c_void_p), ("learnable_weight_clip", c_void_p), ("grad_weight_clip", c_void_p),
    ]


AL_K_COUNT = 14
AL_PEER_SIGNAL_SLOT = 192
AL_STD_STATIC_MAX_SEGMENTS = 262144


class AlProfileEntry(Structure):
    _fields_ = [("launches", c_int64), ("timed", c_int64), ("total_ms", c_double)]


# every symbol include/analog_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "al_abs_max_tiles": (c_int32, [c_int32, c_void_p, c_int32, c_int32, POINTER(c_int32), c_int32, c_void_p, c_void_p]),
    "al_std_tiles": (c_int32, [c_int32, c_void_p, c_int32, c_int32, POINTER(c_int32), c_int32, c_void_p, c_void_p, c_void_p]),
    "al_std_scratch_floats": (c_int64, [c_int32, c_int32]),
    "al_std_tiles_static": (c_int32, [c_int32, c_void_p, c_int32, c_int32, POINTER(c_int32), c_int32, c_void_p, c_void_p]),
    "al_forward": (c_int32, [POINTER(AlDesc), POINTER(AlForwardArgs), c_void_p]),
    "al_backward": (c_int32, [POINTER(AlDesc), POINTER(AlBackwardArgs), c_void_p]),
    "al_backward_scratch_floats": (c_int64, [c_int32, c_int32, c_int32, c_int32]),
    "al_smallm_scratch_floats": (c_int64, [c_int32, c_int32, c_int32]),
    "al_backward_plane_elems": (c_int64, [POINTER(AlDesc), POINTER(c_int32)]),
    "al_f32_planes": (c_int32, []),
    "al_clip_weights": (c_int32, [c_int32, c_void_p, c_int32, c_int32, c_int32, c_float, c_void_p, c_void_p]),
    "al_unfold2d": (c_int32, [c_int32, c_void_p] + [c_int32] * 12 + [c_void_p, c_void_p]),
    "al_fold2d": (c_int32, [c_int32, c_void_p] + [c_int32] * 12 + [c_void_p, c_void_p]),
    "al_conv2d_input_grad_supported": (c_int32, [c_int32] * 14),
    "al_conv2d_input_grad": (c_int32, [c_int32, c_void_p, c_void_p] + [c_int32] * 13 + [c_void_p, c_void_p]),
    "al_unfold2d_dac": (c_int32, [c_int32, c_void_p] + [c_int32] * 12 + [POINTER(c_int32), c_int32, c_double, c_void_p,
                                                                       c_void_p, c_void_p, c_void_p]),
    "al_swiglu_forward": (c_int32, [c_int32, c_void_p, c_int64, c_int32, c_void_p, c_void_p]),
    "al_swiglu_backward": (c_int32, [c_int32, c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_void_p]),
    "al_rotary_qkv": (c_int32, [c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                                c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "al_read_device_error": (c_int32, [c_void_p, POINTER(c_uint32)]),
    "al_set_device_wait_limit_ns": (c_int32, [c_uint64]),
    "al_debug_withhold_forward_signal": (c_int32, [c_int32]),
    "al_uses_tcgen05": (c_int32, [POINTER(AlDesc), POINTER(c_int32)]),
    "al_reserve_sms": (c_int32, [c_int32]),
    "al_peer_allreduce": (c_int32, [c_int32, c_int32, c_int32, POINTER(c_uint64), POINTER(c_uint64), c_uint64, c_int64,
                                    c_int64, c_uint32, c_float, c_int32, c_void_p]),
    "al_peer_read_error": (c_int32, [POINTER(c_uint32)]),
    "al_wgrad_split_plan": (c_int32, [c_int32, c_int32, c_int32, c_int32, POINTER(c_int32), POINTER(c_int32)]),
    "al_pair_work_item": (c_int32, [c_int32, c_int32, c_int32, POINTER(c_int32), POINTER(c_int32), POINTER(c_int32)]),
    "al_profile_enable": (c_int32, [c_int32]),
    "al_profile_select": (c_int32, [c_uint32]),
    "al_profile_read": (c_int32, [POINTER(AlProfileEntry), c_int32]),
    "al_kernel_class_name": (c_char_p, [c_int32]),
    "al_status_str": (c_char_p, [c_int32]),
    "al_last_error": (c_char_p, []),
    "al_version": (c_int32, []),
}

_lib = None


def load():
    """Return the loaded library; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python aihwkit-lightning_b200/build.py` "
                "(there is no CPU or PyTorch fallback for the analog layers)"
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(status: int) -> None:
    """Translate a non-zero status into the exception type the reference would raise."""
    if status == AL_OK:
        return
    lib = load()
    detail = lib.al_last_error().decode() or lib.al_status_str(status).decode()
    if status == AL_ERR_BAD_ARGUMENT:
        raise AssertionError(detail)
    if status in (AL_ERR_UNSUPPORTED, AL_ERR_TOO_LARGE):
        raise ConfigError(detail)
    raise KernelError(status, detail)


_TILE_ENDS: dict = {}


def tile_ends_array(in_sizes):
    """``int32[T]`` of the tiles' upper ends; the (read-only) arrays are kept per tiling."""
    key = tuple(in_sizes)
    arr = _TILE_ENDS.get(key)
    if arr is None:
        ends, acc = [], 0
        for size in key:
            acc += int(size)
            ends.append(acc)
        if len(_TILE_ENDS) > 4096:
            _TILE_ENDS.clear()
        arr = _TILE_ENDS[key] = (c_int32 * len(ends))(*ends)
    return arr


def profile_read(reset: bool = True) -> dict:
    """{kernel class name: (launches, timed scopes, total ms)} since the last reset."""
    lib = load()
    arr = (AlProfileEntry * AL_K_COUNT)()
    check(lib.al_profile_read(arr, int(reset)))
    return {
        lib.al_kernel_class_name(i).decode(): (arr[i].launches, arr[i].timed, arr[i].total_ms)
        for i in range(AL_K_COUNT)
    }
