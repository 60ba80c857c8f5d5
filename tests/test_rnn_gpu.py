"""`AnalogRNN` on the GPU against what the reference's `AnalogRNN` produced on the CPU for the
same seeded modules and inputs (fixture `tests/golden/rnn.pt`, written by
`tests/golden/make_rnn_golden.py`): outputs, final states and, for the training cases, the
gradients of the input and of every parameter."""
import os

import pytest
import torch

import rnn_cases as RC
from util import GOLDEN, rel_fro

pytestmark = pytest.mark.gpu

# fp32 layers agree to 1e-5 per call; the recurrence feeds each step's difference into the next,
# and one flipped ADC level (a tie decided differently by the two accumulation orders) is a full
# quantisation step, hence the wider bound for the case with an ADC
TOL = {"gru_eval_adc": 2e-3}


def _build(case):
    from aihwkit_lightning_b200.nn import AnalogRNN, convert_to_analog
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    rpu = RC.make_rpu_config(TorchInferenceRPUConfig, case)
    model = convert_to_analog(RC.build_digital(case), rpu, ensure_analog_root=False).cuda()
    assert isinstance(model, AnalogRNN)
    return model.train(case["train"])


@pytest.mark.parametrize("name", list(RC.CASES))
def test_rnn_matches_reference(name):
    case = RC.CASES[name]
    want = torch.load(os.path.join(GOLDEN, "rnn.pt"), weights_only=False)[name]
    tol = TOL.get(name, 2e-5)
    model = _build(case)
    x, g = RC.make_input(case)
    x = x.cuda().requires_grad_(case["train"])
    y, states = model(x)
    assert rel_fro(y.detach().cpu(), want["out"]) <= tol
    flat = [s for pair in states for s in pair] if case["module"].get("bidirectional") else states
    for got, ref in zip([s[0] for s in flat], want["h"]):
        assert rel_fro(got.detach().cpu(), ref) <= tol
    for got, ref in zip([s[1] for s in flat if s[1] is not None], want["c"]):
        assert rel_fro(got.detach().cpu(), ref) <= tol
    if not case["train"]:
        return
    (y * g.cuda()).sum().backward()
    assert rel_fro(x.grad.cpu(), want["grad_x"]) <= 1e-4
    grads = {k: p.grad for k, p in model.named_parameters() if p.grad is not None}
    assert set(grads) == set(want["grads"])
    for key, ref in want["grads"].items():
        assert rel_fro(grads[key].cpu(), ref) <= 1e-4, key


@pytest.mark.parametrize("name", ["lstm_bidir_eval", "gru_eval_adc", "rnn_nobias_eval"])
def test_sequence_projection_equals_per_step(name):
    """Evaluation mode projects the whole sequence in one analog call; the values are those of
    one call per step."""
    from aihwkit_lightning_b200.nn import AnalogRNNLayer

    case = RC.CASES[name]
    model = _build(case)
    x = RC.make_input(case)[0].cuda()
    with torch.no_grad():
        fused, _ = model(x)
        for mod in model.modules():
            if isinstance(mod, AnalogRNNLayer):
                mod.batch_input_projection = False
        stepped, _ = model(x)
    assert rel_fro(fused.cpu(), stepped.cpu()) <= TOL.get(name, 2e-5)


def test_bf16_decoding_shape_runs_on_few_rows_path():
    """A bf16 LSTM layer stepping a batch of 8 through 6 time steps: the hidden projection has
    8 rows per call, the input projection 48."""
    from aihwkit_lightning_b200.nn import AnalogLSTMCell, AnalogRNN
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    rpu = RC.make_rpu_config(TorchInferenceRPUConfig, dict(adc=True, train=False))
    rpu.mapping.max_input_size = 256
    torch.manual_seed(0)
    model = AnalogRNN(AnalogLSTMCell, 512, 512, rpu_config=rpu).to(device="cuda", dtype=torch.bfloat16).eval()
    x = torch.randn(6, 8, 512, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        out, states = model(x)
        ideal = AnalogRNN.to_digital(model)(x)[0]
    assert out.shape == (6, 8, 512) and torch.isfinite(out).all()
    assert rel_fro(out.float().cpu(), ideal.float().cpu()) <= 0.1    # quantisation error only
    assert states[0][1].shape == (8, 512)
