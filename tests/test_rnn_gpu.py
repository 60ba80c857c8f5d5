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


class _Mixed(torch.nn.Module):
    """Convolutions, linears and all three recurrent families in one model."""

    def __init__(self):
        super().__init__()
        nn = torch.nn
        self.c1 = nn.Conv1d(2, 4, 3, padding=1)
        self.c2 = nn.Conv2d(4, 6, 3)
        self.fc = nn.Linear(6, 12)
        self.gru = nn.GRU(12, 8, 1)
        self.lstm = nn.LSTM(8, 10, 2, bidirectional=True)
        self.lstm_nb = nn.LSTM(20, 6, 1, bias=False, bidirectional=True)
        self.rnn = nn.RNN(12, 5, 2)

    def forward(self, x):                      # x [B, 2, 36]
        x = self.c1(x).reshape(x.shape[0], 4, 6, 6)
        x = self.c2(x).reshape(x.shape[0], 6, 16).permute(2, 0, 1)   # [16, B, 6]
        x = self.fc(x)
        x, _ = self.gru(x)
        x, _ = self.lstm(x)
        x, _ = self.lstm_nb(x)
        x, _ = self.rnn(x)
        return x


def test_mixed_model_trains_like_its_digital_twin_and_checkpoints_interchange():
    """With the default configuration (no quantisation, no noise) the converted model is the
    digital one: same loss, same first AdamW moment after one step through `AnalogOptimizer`;
    digital and analog checkpoints load into each other (reference:
    `tests/test_conversion.py:200-270`)."""
    import io

    from aihwkit_lightning_b200.nn import AnalogRNN, AnalogWrapper, convert_to_analog, convert_to_digital
    from aihwkit_lightning_b200.optim import AnalogOptimizer
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    torch.manual_seed(0)
    cudnn_tf32, matmul_tf32 = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
    torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = False
    try:
        model = _Mixed().cuda()
        digital_state = {k: v.clone() for k, v in model.state_dict().items()}
        x = torch.randn(3, 2, 36, device="cuda")
        analog = convert_to_analog(model, TorchInferenceRPUConfig())
        assert isinstance(analog, AnalogWrapper) and isinstance(analog.lstm, AnalogRNN)
        analog.load_state_dict(digital_state)                       # digital -> analog
        back = convert_to_digital(analog)

        opt_d = torch.optim.AdamW(model.parameters(), lr=0.01)
        loss_d = model(x).sum()
        loss_d.backward()
        opt_d.step()
        opt_a = AnalogOptimizer(torch.optim.AdamW, analog.analog_layers, analog.parameters(), lr=0.01)
        loss_a = analog(x).sum()
        loss_a.backward()
        opt_a.step()
        assert abs(loss_a.item() - loss_d.item()) <= 1e-4 * max(1.0, abs(loss_d.item()))
        assert torch.allclose(back(x).sum(), loss_d.detach(), rtol=1e-4, atol=1e-4)
        # parameters come in the same order in both models (c1.weight first)
        m_a = opt_a.state_dict()["state"][0]["exp_avg"]
        m_d = opt_d.state_dict()["state"][0]["exp_avg"]
        assert m_a.squeeze().shape == m_d.shape
        assert rel_fro(m_a.squeeze(), m_d) <= 1e-3

        buf = io.BytesIO()
        torch.save(analog.state_dict(), buf)                        # analog -> file -> analog -> digital
        buf.seek(0)
        state = torch.load(buf, weights_only=False)
        analog.load_state_dict(state)
        _Mixed().cuda().load_state_dict(state)
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = cudnn_tf32, matmul_tf32
