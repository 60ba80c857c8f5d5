"""Runs the reference's `calibrate_input_ranges` on two small CPU models and stores the
calibrated ranges next to the seeds that reproduce models and batches.

Usage (needs the reference tree, which the test machines do not have):
    python tests/golden/make_calibration_golden.py <path to the reference's src directory>
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import calibration_cases as CC  # noqa: E402


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_calibration_golden.py <path to the reference's src directory>")
    ref_src = sys.argv[1]
    sys.path.insert(0, ref_src)
    from aihwkit_lightning.inference import InputRangeCalibrationType, calibrate_input_ranges
    from aihwkit_lightning.nn.conversion import convert_to_analog
    from aihwkit_lightning.simulator.configs import TorchInferenceRPUConfig

    out = {}
    for model_name in CC.MODELS:
        for kind, kwargs in CC.KINDS:
            rpu = CC.make_rpu_config(TorchInferenceRPUConfig)
            model = convert_to_analog(CC.build_model(model_name), rpu).eval()
            batches = CC.make_batches(model_name)
            calibrate_input_ranges(model, InputRangeCalibrationType(kind), iter([((b,), {}) for b in batches]),
                                   verbose=False, **kwargs)
            ranges = {name: layer.input_range.detach().clone() for name, layer in model.named_analog_layers()}
            for name, layer in model.named_analog_layers():
                assert layer.rpu_config.pre_post.input_range.enable
            out[(model_name, kind, tuple(sorted(kwargs.items())))] = ranges
            print("ok", model_name, kind, {k: [round(v, 4) for v in r.tolist()] for k, r in ranges.items()})
    torch.save(out, os.path.join(HERE, "calibration.pt"))


if __name__ == "__main__":
    main()
