"""Generate the golden vectors under ``tests/golden/`` from the unmodified reference.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference/src

For every case of ``cases.CASES`` the script
1. builds the reference ``AnalogLinear``, replaces the ``randn_like`` the reference's torch
   backend draws its noise from by a replay of pre-drawn standard normals, runs forward
   (``steps`` times) and one backward through autograd;
2. runs the oracle (``oracle/analog_oracle.py``) on the same tensors and noise and asserts
   bit-identical outputs, gradients and updated input ranges -- this is what pins the oracle;
3. writes inputs-free results (everything is re-derivable from the seeds in ``cases.py``)
   to ``tests/golden/<name>.pt``.
"""
import os
import sys
from types import SimpleNamespace

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import cases as C  # noqa: E402
import analog_oracle as O  # noqa: E402


def same(a, b):
    if a is None or b is None:
        return a is None and b is None
    return a.shape == b.shape and a.dtype == b.dtype and bool(((a == b) | (a.isnan() & b.isnan())).all())


def run_reference(ref, case, data):
    import aihwkit_lightning.nn.modules.torch_utils.torch_linear as TL

    rpu = C.build_rpu_config(ref, case)
    layer = ref.AnalogLinear(data["k"], data["n"], bias=case["bias"], rpu_config=rpu)
    layer = layer.to(dtype=data["dtype"])
    layer.set_weights_and_biases(data["w"], data["b"])
    layer.train(case["training"])
    if layer.learnable_weight_clip is not None:
        layer.learnable_weight_clip.data.mul_(case["lwc_scale"])

    queue = []
    original = TL.randn_like

    def replay(like):
        return queue.pop(0).to(like.dtype).reshape(like.shape)

    TL.randn_like = replay
    try:
        for step in range(case["steps"]):
            queue.clear()
            lo = 0
            for t, size in enumerate(layer.in_sizes):
                if case["training"] and case["noise_type"] != "None":
                    queue.append(data["w_noise"][step][:, lo : lo + size])
                if case["training"] and case["out_noise"] > 0:
                    queue.append(data["out_noise"][step][t])
                lo += size
            x = data["xs"][step].clone().requires_grad_(True)
            layer.zero_grad()
            out = layer(x)
            assert not queue, "noise replay out of sync with the reference"
        out.backward(data["g"])
    finally:
        TL.randn_like = original
    return dict(
        out=out.detach(),
        grad_x=x.grad,
        grad_w=layer.weight.grad,
        grad_bias=None if layer.bias is None else layer.bias.grad,
        grad_ir=None if layer.input_range is None else layer.input_range.grad,
        grad_clip=None if layer.learnable_weight_clip is None else layer.learnable_weight_clip.grad,
        learnable_weight_clip=None if layer.learnable_weight_clip is None
        else layer.learnable_weight_clip.detach().clone(),
        input_range=None if layer.input_range is None else layer.input_range.detach().clone(),
        input_range_update_idx=None
        if layer.input_range_update_idx is None
        else layer.input_range_update_idx.clone(),
        x_min=None if getattr(layer, "x_min", None) is None else layer.x_min.clone(),
        x_max=None if getattr(layer, "x_max", None) is None else layer.x_max.clone(),
        in_sizes=list(layer.in_sizes),
    )


def run_oracle(ns, case, data):
    rpu = C.build_rpu_config(ns, case)
    in_sizes = O.split_sizes(data["k"], case["max_input_size"])
    static = case["ir_enable"] and not case["ir_dynamic"]
    ir = idx = x_min = x_max = None
    if static:
        ir = torch.full((len(in_sizes),), case["ir_init_value"], dtype=data["dtype"])
        idx = torch.zeros(len(in_sizes), dtype=data["dtype"])
        x_min = torch.zeros(len(in_sizes), dtype=data["dtype"]) - 1e-5
        x_max = torch.zeros(len(in_sizes), dtype=data["dtype"]) + 1e-5
    lwc = None
    if case["clip_type"] == "LearnablePerChannel":
        lwc = O.sliced_abs_max(in_sizes, data["w"]) * case["lwc_scale"]
    for step in range(case["steps"]):
        rec = O.forward(
            data["xs"][step], data["w"], data["b"], ir, idx, x_min, x_max, in_sizes,
            case["training"], rpu,
            O.NoiseReplay(data["w_noise"][step], data["out_noise"][step]),
            learnable_weight_clip=lwc,
        )
    grads = O.backward(rec, data["g"], data["w"], case["bias"], ir, rpu)
    if static and not case["ir_learn"]:
        grads["grad_ir"] = None
    return rec, grads, ir, idx, x_min, x_max


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to the reference's src directory>")
    ref_src = sys.argv[1]
    sys.path.insert(0, ref_src)
    import aihwkit_lightning.nn as ref_nn
    import aihwkit_lightning.simulator.configs as ref_cfg

    ref = SimpleNamespace(
        AnalogLinear=ref_nn.AnalogLinear,
        TorchInferenceRPUConfig=ref_cfg.TorchInferenceRPUConfig,
        WeightNoiseInjectionType=ref_cfg.WeightNoiseInjectionType,
        WeightQuantizationType=ref_cfg.WeightQuantizationType,
        WeightClipType=ref_cfg.WeightClipType,
    )
    torch.set_num_threads(1)
    for case in C.CASES:
        data = C.make_inputs(case)
        want = run_reference(ref, case, data)
        rec, grads, ir, idx, x_min, x_max = run_oracle(ref, case, data)
        checks = dict(
            out=same(want["out"], rec.out),
            grad_x=same(want["grad_x"], grads["grad_x"]),
            grad_w=same(want["grad_w"], grads["grad_w"]),
            grad_bias=same(want["grad_bias"], grads["grad_bias"]),
            grad_ir=same(want["grad_ir"], grads["grad_ir"]),
            grad_clip=same(want["grad_clip"], grads["grad_clip"]),
            input_range=same(want["input_range"], ir),
            update_idx=same(want["input_range_update_idx"], idx),
            x_min=same(want["x_min"], x_min),
            x_max=same(want["x_max"], x_max),
        )
        bad = [k for k, ok in checks.items() if not ok]
        assert not bad, f"oracle differs from the reference in case {case['name']}: {bad}"
        assert want["in_sizes"] == O.split_sizes(data["k"], case["max_input_size"])
        want["tiles"] = [
            dict(
                ir=tr.ir, codes=tr.codes, q=tr.q, amax_rows=tr.amax_rows, w_mod=tr.w_mod,
                bound=tr.bound, out_t=tr.out_t,
            )
            for tr in rec.tiles
        ]
        want["case"] = case
        torch.save(want, os.path.join(HERE, case["name"] + ".pt"))
        print(f"ok  {case['name']}")
    print(f"{len(C.CASES)} cases: the oracle reproduces the reference bit for bit")


if __name__ == "__main__":
    main()
