"""`calibrate_input_ranges` against the ranges the reference produced for the same models and
batches (fixture `tests/golden/calibration.pt`, written by `tests/golden/make_calibration_golden.py`)."""
import os

import pytest
import torch

import calibration_cases as CC
from util import GOLDEN

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("model_name", CC.MODELS)
@pytest.mark.parametrize("kind,kwargs", CC.KINDS, ids=[f"{k}-{'-'.join(map(str, kw.values()))}" for k, kw in CC.KINDS])
def test_calibrated_ranges_match_reference(model_name, kind, kwargs):
    from aihwkit_lightning_b200.inference import InputRangeCalibrationType, calibrate_input_ranges
    from aihwkit_lightning_b200.nn import AnalogLayerBase, convert_to_analog
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    want = torch.load(os.path.join(GOLDEN, "calibration.pt"), weights_only=False)[
        (model_name, kind, tuple(sorted(kwargs.items())))]
    rpu = CC.make_rpu_config(TorchInferenceRPUConfig)
    model = convert_to_analog(CC.build_model(model_name), rpu).cuda().eval()
    batches = [b.cuda() for b in CC.make_batches(model_name)]
    calibrate_input_ranges(model, InputRangeCalibrationType(kind), iter([((b,), {}) for b in batches]), **kwargs)
    assert isinstance(model, AnalogLayerBase)
    layers = dict(model.named_analog_layers())
    assert set(layers) == set(want)
    for name, layer in layers.items():
        cfg = layer.rpu_config
        assert cfg.pre_post.input_range.enable and not cfg.pre_post.input_range.dynamic
        assert cfg.forward.out_noise == 0.03          # the noise settings come back untouched
        assert torch.isinf(layer.input_range_update_idx).all()
        got = layer.input_range.detach().float().cpu()
        assert torch.allclose(got, want[name].float(), rtol=2e-4, atol=1e-5), (name, got, want[name])
    # the calibrated model runs with its static ranges
    out = model(batches[0])
    assert torch.isfinite(out).all()


def test_calibration_refuses_wrong_state():
    from aihwkit_lightning_b200.exceptions import ConfigError
    from aihwkit_lightning_b200.inference import InputRangeCalibrationType, calibrate_input_ranges
    from aihwkit_lightning_b200.nn import convert_to_analog
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    rpu = CC.make_rpu_config(TorchInferenceRPUConfig)
    model = convert_to_analog(CC.build_model("mlp"), rpu).cuda()
    with pytest.raises(ConfigError):   # training mode
        calibrate_input_ranges(model.train(), InputRangeCalibrationType.MAX, iter([]))
    rpu2 = CC.make_rpu_config(TorchInferenceRPUConfig)
    rpu2.pre_post.input_range.enable = True
    model2 = convert_to_analog(CC.build_model("mlp"), rpu2).cuda().eval()
    with pytest.raises(ConfigError):   # already has input ranges
        calibrate_input_ranges(model2, InputRangeCalibrationType.MAX, iter([]))
    rpu3 = CC.make_rpu_config(TorchInferenceRPUConfig)
    rpu3.forward.inp_res = 254
    model3 = convert_to_analog(CC.build_model("mlp"), rpu3).cuda().eval()
    with pytest.raises(ConfigError):   # finite input resolution
        calibrate_input_ranges(model3, InputRangeCalibrationType.MAX, iter([]))
