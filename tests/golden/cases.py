"""Case table shared by the golden-vector generator and the parity tests.

Each case is a flat dict; ``build_rpu_config`` turns it into a ``TorchInferenceRPUConfig`` of
whichever implementation is passed in (the reference's classes when generating, the product's
when testing), and ``make_inputs`` draws the seeded synthetic tensors on the CPU.
"""
from math import prod

import torch

DEFAULTS = dict(
    dtype="fp32",
    in_shape=(12, 40),  # leading dims + in_features
    out_features=24,
    bias=True,
    training=True,
    max_input_size=16,
    ir_enable=True,
    ir_dynamic=False,
    ir_learn=True,
    ir_init_value=1.0,
    ir_init_from_data=0,
    ir_init_std_alpha=3.0,
    ir_decay=0.001,
    ir_min_pct=0.95,
    ir_fast_mode=False,
    ir_momentum=0.95,
    inp_res=254.0,
    out_noise=0.0,
    out_noise_per_channel=False,
    out_bound=0.0,
    out_res=-1.0,
    noise_type="None",
    quant_type="None",
    std_dev=0.0,
    mod_res=0.0,
    clip_type="None",
    clip_sigma=-1.0,
    lwc_scale=1.0,  # LearnablePerChannel: the learned ranges are the per-tile abs-max times this
    weight_scale=0.3,
    seed=0,
    steps=1,  # number of forward calls (exercises init-from-data)
)


def _c(name, **kw):
    case = dict(DEFAULTS)
    case.update(kw)
    case["name"] = name
    return case


CASES = [
    _c("static_plain_eval", training=False),
    _c("static_train_noise", out_noise=0.04, noise_type="AddNormal", std_dev=0.02),
    _c("static_train_noise_pc", out_noise=0.04, out_noise_per_channel=True,
       noise_type="AddNormalPerChannel", std_dev=0.02),
    _c("static_adc", out_bound=3.0, out_res=254.0, ir_init_value=0.8),
    _c("static_adc_noise", out_bound=3.0, out_res=254.0, out_noise=0.04,
       noise_type="AddNormalPerChannel", std_dev=0.02),
    _c("static_adc_res_inverse", out_bound=2.0, out_res=1 / 254.0, inp_res=1 / 254.0),
    _c("static_init_from_data", ir_init_from_data=2, steps=3, ir_init_value=3.0),
    _c("static_no_decay", ir_decay=0.0, ir_init_value=0.5),
    _c("static_not_learned", ir_learn=False, ir_init_value=0.7),
    _c("dynamic_plain_eval", ir_dynamic=True, training=False),
    _c("dynamic_adc_noise", ir_dynamic=True, out_bound=3.0, out_res=254.0, out_noise=0.04,
       noise_type="AddNormalPerChannel", std_dev=0.02),
    _c("dynamic_adc_gauss_pc_clip", ir_dynamic=True, out_bound=4.0, out_res=254.0,
       clip_type="LayerGaussianPerChannel", clip_sigma=2.5),
    _c("dynamic_bound_only", ir_dynamic=True, out_bound=2.0),
    _c("dynamic_3d_input", ir_dynamic=True, in_shape=(3, 5, 40), out_bound=3.0, out_res=254.0),
    _c("dynamic_1d_input", ir_dynamic=True, in_shape=(40,), out_noise=0.04),
    _c("dynamic_zero_row", ir_dynamic=True, zero_row=1, out_bound=3.0, out_res=254.0),
    _c("no_ir_no_dac", ir_enable=False, inp_res=-1.0, noise_type="AddNormal", std_dev=0.05),
    _c("discretize", quant_type="Discretize", mod_res=30.0),
    _c("discretize_pc_inverse_res", quant_type="DiscretizePerChannel", mod_res=1 / 30.0),
    _c("discretize_noise", quant_type="DiscretizePerChannel", mod_res=30.0,
       noise_type="AddNormal", std_dev=0.03, ir_dynamic=True),
    _c("ragged_tiles", in_shape=(7, 43), max_input_size=10, out_features=9, ir_dynamic=True,
       out_bound=3.0, out_res=254.0, out_noise=0.02),
    _c("single_tile", max_input_size=-1, out_noise=0.04, noise_type="AddNormal", std_dev=0.02),
    _c("no_bias", bias=False, ir_dynamic=True),
    # bf16: every op of the reference rounds to bf16
    _c("bf16_dynamic_adc_noise", dtype="bf16", ir_dynamic=True, out_bound=3.0, out_res=254.0,
       out_noise=0.04, noise_type="AddNormalPerChannel", std_dev=0.02),
    _c("bf16_static_noise", dtype="bf16", out_noise=0.04, noise_type="AddNormal", std_dev=0.02),
    _c("bf16_static_adc", dtype="bf16", out_bound=3.0, out_res=254.0, ir_init_value=0.8),
    _c("bf16_dynamic_eval", dtype="bf16", ir_dynamic=True, training=False, out_bound=10.0,
       out_res=254.0, in_shape=(16, 64), out_features=32, max_input_size=32),
    _c("bf16_discretize", dtype="bf16", quant_type="DiscretizePerChannel", mod_res=254.0,
       ir_dynamic=True),
    _c("bf16_init_from_data", dtype="bf16", ir_init_from_data=2, steps=3, ir_init_value=3.0),
    # fast mode: min/max tracking of the first calls, plain clamp afterwards
    _c("fast_mode_momentum", ir_fast_mode=True, ir_init_from_data=2, steps=4, out_noise=0.04),
    _c("fast_mode_minmax", ir_fast_mode=True, ir_momentum=-1, ir_init_from_data=3, steps=3,
       out_bound=3.0, out_res=254.0),
    _c("fast_mode_fixed", ir_fast_mode=True, ir_init_from_data=0, ir_init_value=0.9),
    _c("bf16_fast_mode", dtype="bf16", ir_fast_mode=True, ir_init_from_data=2, steps=3),
    # learnable per-channel weight ranges: clamp only, and as the scale of the discretiser
    _c("learnable_clip", clip_type="LearnablePerChannel", lwc_scale=0.6, out_bound=3.0, out_res=254.0,
       out_noise=0.04, noise_type="AddNormalPerChannel", std_dev=0.02),
    _c("learnable_clip_eval", clip_type="LearnablePerChannel", lwc_scale=0.8, training=False,
       ir_dynamic=True, out_bound=2.0),
    _c("learnable_clip_discretize", clip_type="LearnablePerChannel", lwc_scale=0.8,
       quant_type="DiscretizePerChannel", mod_res=30.0, ir_dynamic=True, noise_type="AddNormal", std_dev=0.02),
    _c("learnable_clip_wide", clip_type="LearnablePerChannel", lwc_scale=1.0, weight_scale=6.0,
       in_shape=(6, 32), out_features=8, ir_dynamic=True),
    _c("bf16_learnable_clip", dtype="bf16", clip_type="LearnablePerChannel", lwc_scale=0.7,
       ir_dynamic=True, out_bound=3.0, out_res=254.0, noise_type="AddNormalPerChannel", std_dev=0.02),
    _c("bf16_learnable_clip_discretize", dtype="bf16", clip_type="LearnablePerChannel", lwc_scale=0.9,
       quant_type="DiscretizePerChannel", mod_res=254.0, ir_dynamic=True),
]

CASES_BY_NAME = {c["name"]: c for c in CASES}

TORCH_DTYPE = {"fp32": torch.float32, "bf16": torch.bfloat16}


def build_rpu_config(ns, case):
    """``ns`` must offer TorchInferenceRPUConfig and the three enums."""
    rpu = ns.TorchInferenceRPUConfig()
    rpu.forward.inp_res = case["inp_res"]
    rpu.forward.out_noise = case["out_noise"]
    rpu.forward.out_noise_per_channel = case["out_noise_per_channel"]
    rpu.forward.out_bound = case["out_bound"]
    rpu.forward.out_res = case["out_res"]
    rpu.mapping.max_input_size = case["max_input_size"]
    ir = rpu.pre_post.input_range
    ir.enable = case["ir_enable"]
    ir.dynamic = case["ir_dynamic"]
    ir.learn_input_range = case["ir_learn"]
    ir.init_value = case["ir_init_value"]
    ir.init_from_data = case["ir_init_from_data"]
    ir.init_std_alpha = case["ir_init_std_alpha"]
    ir.decay = case["ir_decay"]
    ir.input_min_percentage = case["ir_min_pct"]
    ir.fast_mode = case["ir_fast_mode"]
    ir.act_range_momentum = case["ir_momentum"]
    rpu.modifier.noise_type = ns.WeightNoiseInjectionType(case["noise_type"])
    rpu.modifier.quantization_type = ns.WeightQuantizationType(case["quant_type"])
    rpu.modifier.std_dev = case["std_dev"]
    rpu.modifier.res = case["mod_res"]
    rpu.clip.type = ns.WeightClipType(case["clip_type"])
    rpu.clip.sigma = case["clip_sigma"]
    return rpu


def make_inputs(case):
    """Seeded CPU tensors of one case: inputs per step, weight, bias, upstream gradient and
    the standard-normal draws that are replayed as weight / output noise."""
    from sys import path as _p  # noqa: F401  (keeps this module import-light)

    dtype = TORCH_DTYPE[case["dtype"]]
    gen = torch.Generator().manual_seed(1234 + case["seed"])
    in_shape = tuple(case["in_shape"])
    k = in_shape[-1]
    n = case["out_features"]
    m = prod(in_shape[:-1]) if len(in_shape) > 1 else 1
    n_tiles = 1 if case["max_input_size"] <= 0 else -(-k // case["max_input_size"])
    xs = []
    for _ in range(case["steps"]):
        x = torch.randn(in_shape, generator=gen)
        if case.get("zero_row") is not None:
            x.reshape(m, k)[case["zero_row"]] = 0.0
        xs.append(x.to(dtype))
    w = ((torch.rand(n, k, generator=gen) * 2 - 1) * case["weight_scale"]).to(dtype)
    b = (torch.randn(n, generator=gen) * 0.1).to(dtype) if case["bias"] else None
    g = torch.randn(in_shape[:-1] + (n,), generator=gen).to(dtype)
    w_noise = [torch.randn(n, k, generator=gen).to(dtype) for _ in range(case["steps"])]
    out_noise = [torch.randn(n_tiles, m, n, generator=gen).to(dtype) for _ in range(case["steps"])]
    return dict(xs=xs, w=w, b=b, g=g, w_noise=w_noise, out_noise=out_noise, m=m, k=k, n=n,
                n_tiles=n_tiles, dtype=dtype)
