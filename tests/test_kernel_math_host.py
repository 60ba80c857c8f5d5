"""Rounding chains of the CUDA kernels, compiled for the host, against the oracle.

``oracle/kernel_math_host.cpp`` compiles the host/device arithmetic header of the CUDA library
(``csrc/analog_math.cuh``) with g++ and wraps it in loops.  Codes, de-quantised inputs, abs-max,
modified weights and every tile's output stage must equal the golden intermediates bit for bit
(fp32 and bf16) -- the same functions run inside the kernels.
"""
import ctypes
import os
import subprocess

import pytest
import torch

import cases as C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
NOISE = {"None": 0, "AddNormal": 1, "AddNormalPerChannel": 2}
QUANT = {"None": 0, "Discretize": 1, "DiscretizePerChannel": 2}


@pytest.fixture(scope="module")
def km():
    src = os.path.join(ROOT, "oracle", "kernel_math_host.cpp")
    out_dir = os.path.join(ROOT, "oracle", "_build")
    os.makedirs(out_dir, exist_ok=True)
    lib = os.path.join(out_dir, "libkernel_math_host.so")
    hdr = os.path.join(ROOT, "aihwkit-lightning_b200", "csrc", "analog_math.cuh")
    if not os.path.exists(lib) or os.path.getmtime(lib) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        subprocess.check_call(
            ["g++", "-O2", "-mfma", "-ffp-contract=off", "-shared", "-fPIC", "-x", "c++", src, "-o", lib]
        )
    return ctypes.CDLL(lib)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def bits(t):
    return t.view(torch.int16) if t.dtype == torch.bfloat16 else t.view(torch.int32)


def same(a, b):
    return a.shape == b.shape and bool((a == b).all())


@pytest.mark.parametrize("name", [c["name"] for c in C.CASES])
def test_host_build_of_kernel_math_matches_golden(km, name):
    case = C.CASES_BY_NAME[name]
    want = torch.load(os.path.join(GOLDEN, name + ".pt"), weights_only=False)
    data = C.make_inputs(case)
    dt = 0 if case["dtype"] == "fp32" else 1
    m, k, n, T = data["m"], data["k"], data["n"], len(want["in_sizes"])
    ends = torch.tensor(want["in_sizes"]).cumsum(0).to(torch.int32)
    x = data["xs"][-1].reshape(m, k).contiguous()
    tiles = want["tiles"]
    ir_mode = 0 if not case["ir_enable"] else (2 if case["ir_dynamic"] else 1)

    # ---- DAC -------------------------------------------------------------------------
    if ir_mode:
        ir_static = torch.stack([t["ir"].reshape(()) for t in tiles]) if ir_mode == 1 else None
        xq = torch.empty_like(x)
        codes = torch.empty_like(x)
        ir_rows = torch.empty(T, m, dtype=x.dtype)
        km.km_dac(dt, ptr(x), m, k, ptr(ends), T, ir_mode, ptr(ir_static),
                  ctypes.c_float(case["inp_res"]), 0, ptr(xq), ptr(ir_rows), ptr(codes))
        lo = 0
        for t, size in enumerate(want["in_sizes"]):
            assert same(xq[:, lo:lo + size], tiles[t]["q"]), f"q tile {t}"
            if tiles[t]["codes"] is not None:
                assert same(codes[:, lo:lo + size], tiles[t]["codes"]), f"codes tile {t}"
            if ir_mode == 2:
                assert same(ir_rows[t], tiles[t]["ir"].reshape(-1)), f"ir tile {t}"
            lo += size

    # ---- weight modifier ---------------------------------------------------------------
    w = data["w"].contiguous()
    training = case["training"]
    noise_type = NOISE[case["noise_type"]] if training else 0
    quant_type = QUANT[case["quant_type"]]
    n_states = max(case["mod_res"], 1 / case["mod_res"]) if quant_type else 0.0
    w_mod = torch.empty_like(w)
    amax = torch.empty(T, n, dtype=w.dtype)
    clip = None
    if case["clip_type"] == "LearnablePerChannel":
        clip = want["learnable_weight_clip"].contiguous()
    km.km_weight_modify(dt, ptr(w), n, k, ptr(ends), T, quant_type, ctypes.c_float(n_states),
                        ctypes.c_float(n_states / 2), noise_type, ctypes.c_float(case["std_dev"]),
                        ptr(data["w_noise"][-1].contiguous()), 0, ptr(w_mod), ptr(amax), ptr(clip))
    lo = 0
    for t, size in enumerate(want["in_sizes"]):
        assert same(w_mod[:, lo:lo + size], tiles[t]["w_mod"]), f"w_mod tile {t}"
        if tiles[t]["amax_rows"] is not None:
            assert same(amax[t], tiles[t]["amax_rows"].reshape(-1)), f"amax tile {t}"
        lo += size

    # ---- per-tile output stage ---------------------------------------------------------
    has_noise = int(training and case["out_noise"] > 0)
    has_bound, has_adc = int(case["out_bound"] > 0), int(case["out_res"] > 0)
    noise_coef = case["out_noise"] / (T ** 0.5)
    bound_pc = case["clip_type"] in ("LayerGaussianPerChannel", "LearnablePerChannel")
    for t, tr in enumerate(tiles):
        acc = (tr["q"] @ tr["w_mod"].T).float().contiguous()
        ir = tr["ir"]
        ir_arg = None if ir is None else ir.reshape(-1).contiguous()
        amax_t = None if tr["amax_rows"] is None else tr["amax_rows"].reshape(-1).contiguous()
        tmax = None if amax_t is None else amax_t.max().reshape(1).contiguous()
        s_noise = amax_t if case["out_noise_per_channel"] else tmax
        s_bound = amax_t if bound_pc else tmax
        out = torch.empty(m, n, dtype=x.dtype)
        keep = torch.empty(m, n, dtype=torch.uint8)
        km.km_tile_stage(dt, ptr(acc), m, n, ptr(ir_arg), int(ir_mode == 2), ptr(s_noise),
                         int(case["out_noise_per_channel"]), ptr(s_bound), int(bound_pc),
                         ptr(data["out_noise"][-1][t].contiguous()), has_noise, has_bound, has_adc, 0,
                         ctypes.c_float(noise_coef), ctypes.c_float(case["out_bound"]),
                         ctypes.c_float(case["out_res"]), ptr(out), ptr(keep))
        assert same(out, tr["out_t"].reshape(m, n)), f"tile output {t}"


def test_fast_division_rint_and_rounding_are_exact(km):
    """The streaming kernels divide through a correctly rounded reciprocal (Markstein), round to
    integers with two additions and round to bf16 with integer adds; all three must agree with
    the plain operations bit for bit."""
    km.km_check_fast_ops.restype = ctypes.c_longlong
    assert km.km_check_fast_ops(ctypes.c_longlong(20_000_000), ctypes.c_ulonglong(12345)) == 0


def test_packed_bf16_adc_is_exact(km):
    """The tensor-core forward divides, rounds to an integer and multiplies back in packed bf16
    arithmetic; over every step significand and every bf16 input the codes up to +-127 equal the
    reference chain (a zero code may come out as +0 where the reference has -0), and larger ones stay beyond +-127 (where the clamp takes over)."""
    km.km_check_adc_bf16.restype = ctypes.c_longlong
    assert km.km_check_adc_bf16() == 0


def test_generator_moments(km):
    n = 1 << 18
    out = torch.empty(n)
    km.km_normals(ctypes.c_ulonglong(1234), ctypes.c_ulonglong(7), 1, ctypes.c_longlong(n), ptr(out))
    assert abs(out.mean().item()) < 0.01
    assert abs(out.std().item() - 1.0) < 0.01
    assert abs((out ** 4).mean().item() - 3.0) < 0.1
    other = torch.empty(n)
    km.km_normals(ctypes.c_ulonglong(1234), ctypes.c_ulonglong(8), 1, ctypes.c_longlong(n), ptr(other))
    assert abs(torch.corrcoef(torch.stack([out, other]))[0, 1].item()) < 0.01
