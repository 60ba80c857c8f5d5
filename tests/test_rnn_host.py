"""Host logic of the containers, the recurrent modules and the conversion functions (no GPU).

The analog matrix product itself needs the CUDA library, so the tests that run a forward pass
replace ``AnalogLinear.forward`` by the plain affine map: what is checked here is the wiring
around it (gate order, time loop, reverse direction, stacking, the single projection of a whole
sequence in evaluation mode) against torch's own LSTM / GRU / RNN.
"""
import copy
import pickle

import pytest
import torch
from torch import nn

from aihwkit_lightning_b200.exceptions import ArgumentError
from aihwkit_lightning_b200.nn import (
    AnalogLayerBase, AnalogLinear, AnalogLSTMCell, AnalogLSTMCellCombinedWeight, AnalogRNN, AnalogSequential,
    AnalogWrapper, convert_to_analog, convert_to_digital)
from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig


@pytest.fixture
def digital_linear(monkeypatch):
    calls = []

    def forward(self, inp):
        calls.append(tuple(inp.shape))
        return torch.nn.functional.linear(inp, self.weight, self.bias)

    monkeypatch.setattr(AnalogLinear, "forward", forward)
    return calls


@pytest.mark.parametrize("kind", ["LSTM", "GRU", "RNN"])
@pytest.mark.parametrize("bidir", [False, True])
@pytest.mark.parametrize("train", [False, True])
def test_wiring_matches_torch(kind, bidir, train, digital_linear):
    torch.manual_seed(0)
    digital = getattr(nn, kind)(6, 10, num_layers=2, bidirectional=bidir)
    analog = convert_to_analog(digital, TorchInferenceRPUConfig(), ensure_analog_root=False)
    assert isinstance(analog, AnalogRNN)
    analog.train(train)
    x = torch.randn(7, 3, 6)
    want, want_state = digital(x)
    got, states = analog(x)
    assert torch.allclose(got, want, atol=1e-6)
    flat = [s for pair in states for s in pair] if bidir else states
    h_n = want_state[0] if kind == "LSTM" else want_state
    for i, state in enumerate(flat):          # torch orders (layer, direction) the same way
        assert torch.allclose(state[0], h_n[i], atol=1e-6)
        if kind == "LSTM":
            assert torch.allclose(state[1], want_state[1][i], atol=1e-6)
    # evaluation: one input projection of [steps, batch, .] per cell; training: one per step
    per_cell = [c for c in digital_linear if len(c) == 3]
    n_cells = 2 * (2 if bidir else 1)
    assert len(per_cell) == (0 if train else n_cells)
    assert len(digital_linear) == (n_cells * 7 * 2 if train else n_cells * (7 + 1))


def test_unbatched_input_and_given_states(digital_linear):
    torch.manual_seed(1)
    analog = AnalogRNN(AnalogLSTMCell, 4, 5, rpu_config=TorchInferenceRPUConfig()).eval()
    digital = AnalogRNN.to_digital(analog)
    x = torch.randn(6, 4)
    got, _ = analog(x)
    want, _ = digital(x)
    assert got.shape == (6, 1, 5) and torch.allclose(got[:, 0], want, atol=1e-6)
    states = analog.get_zero_state(2)
    got2, _ = analog(torch.randn(3, 2, 4), states)
    assert got2.shape == (3, 2, 5)


def test_combined_weight_cell(digital_linear):
    torch.manual_seed(2)
    analog = AnalogRNN(AnalogLSTMCellCombinedWeight, 4, 5, rpu_config=TorchInferenceRPUConfig()).eval()
    out, states = analog(torch.randn(3, 2, 4))
    assert out.shape == (3, 2, 5) and states[0][1].shape == (2, 5)
    assert digital_linear == [(2, 9)] * 3


def test_errors():
    rpu = TorchInferenceRPUConfig()
    with pytest.raises(RuntimeError, match="batch_first"):
        AnalogRNN(AnalogLSTMCell, 4, 4, batch_first=True, rpu_config=rpu)
    with pytest.raises(RuntimeError, match="proj_size"):
        AnalogRNN(AnalogLSTMCell, 4, 4, proj_size=2, rpu_config=rpu)
    with pytest.raises(ValueError, match="rpu_config"):
        AnalogRNN(AnalogLSTMCell, 4, 4)
    net = AnalogRNN(AnalogLSTMCell, 4, 4, num_layers=2, rpu_config=rpu)
    with pytest.raises(RuntimeError, match="2D or 3D"):
        net(torch.zeros(4))
    with pytest.raises(RuntimeError, match="Expecting 2 states"):
        net(torch.zeros(3, 2, 4), net.get_zero_state(2)[:1])
    with pytest.raises(RuntimeError, match="input.size"):
        net(torch.zeros(3, 2, 5))
    with pytest.raises(RuntimeError, match="Expected hidden size"):
        net(torch.zeros(3, 2, 4), net.get_zero_state(3))
    with pytest.raises(RuntimeError, match="should be 1-D"):
        net(torch.zeros(3, 4), net.get_zero_state(1))
    with pytest.raises(ArgumentError):
        convert_to_analog(nn.Linear(2, 2), rpu, conversion_map=[nn.Linear])
    with pytest.raises(ArgumentError):
        convert_to_digital(nn.Linear(2, 2), conversion_set=[AnalogLinear])


def test_state_dict_uses_torch_names_both_ways():
    torch.manual_seed(3)
    rpu = TorchInferenceRPUConfig()
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = False
    digital = nn.GRU(4, 6, num_layers=2, bidirectional=True)
    analog = AnalogRNN.from_digital(digital, rpu)
    state = analog.state_dict()
    assert set(digital.state_dict()) <= set(state)
    assert "input_range_hh_l1_reverse" in state and "input_range_update_idx_ih_l0" in state
    for key, value in digital.state_dict().items():
        assert torch.equal(state[key], value)
    # a torch checkpoint loads into the analog module (the analog-only state stays as it is) ...
    other = AnalogRNN.from_digital(nn.GRU(4, 6, num_layers=2, bidirectional=True), rpu)
    result = other.load_state_dict(digital.state_dict(), strict=False)
    assert not result.unexpected_keys
    assert torch.equal(other.rnn.layers[1].directions[1].cell.weight_ih.weight, digital.weight_ih_l1_reverse)
    # ... the analog checkpoint loads strictly into another analog module, nested or not ...
    other.load_state_dict(state)
    holder = nn.ModuleDict({"enc": AnalogRNN.from_digital(nn.GRU(4, 6, num_layers=2, bidirectional=True), rpu)})
    holder.load_state_dict({f"enc.{k}": v for k, v in state.items()})
    assert set(holder.state_dict()) == {f"enc.{k}" for k in state}
    # ... and its weights load into torch's module
    back = nn.GRU(4, 6, num_layers=2, bidirectional=True)
    back.load_state_dict({k: v for k, v in state.items() if k in back.state_dict()})
    assert torch.equal(back.bias_hh_l0_reverse, digital.bias_hh_l0_reverse)


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(1, 2, 3), nn.ReLU(), nn.Sequential(nn.Linear(3, 3)))
        self.rnn = nn.LSTM(3, 4)
        self.head = nn.Linear(4, 2)
        self.skip = nn.Linear(4, 2)


def test_conversion_tree_and_round_trip():
    torch.manual_seed(4)

    seen = []

    def per_layer(name, module, rpu):
        seen.append(name)
        if name == "head":
            rpu.forward.inp_res = 14
        return rpu

    rpu = TorchInferenceRPUConfig()
    net = Net()
    analog = convert_to_analog(net, rpu, specific_rpu_config_fun=per_layer, exclude_modules=["skip"])
    assert isinstance(analog, AnalogWrapper) and isinstance(analog, Net) and isinstance(analog, AnalogLayerBase)
    assert type(analog).__name__ == "AnalogWrapperNet"
    assert isinstance(analog.stem, AnalogSequential) and isinstance(analog.stem[2], AnalogSequential)
    assert isinstance(analog.rnn, AnalogRNN) and isinstance(analog.skip, nn.Linear)
    assert not isinstance(analog.skip, AnalogLinear)
    assert seen == ["stem", "stem.0", "stem.2", "stem.2.0", "rnn", "head"]
    assert analog.head.rpu_config.forward.inp_res == 14 and analog.stem[0].rpu_config.forward.inp_res != 14
    assert analog.head.rpu_config is not analog.stem[0].rpu_config
    names = [n for n, _ in analog.named_analog_layers()]
    assert names == ["stem.0", "stem.2.0", "rnn.rnn.layers.0.cell.weight_ih", "rnn.rnn.layers.0.cell.weight_hh", "head"]
    assert net.head.weight is not analog.head.weight          # not in place: the original is untouched
    assert set(analog.state_dict()) == set(net.state_dict())  # checkpoint names survive the conversion
    clone = copy.deepcopy(analog)
    assert type(clone) is type(analog) and clone.head.weight is not analog.head.weight
    assert type(pickle.loads(pickle.dumps(analog))).__name__ == "AnalogWrapperNet"
    digital = convert_to_digital(analog)
    assert type(digital) is Net and type(digital.stem) is nn.Sequential and type(digital.rnn) is nn.LSTM
    for key, value in net.state_dict().items():
        assert torch.equal(digital.state_dict()[key], value), key
    # no wrapper when not asked for, or when the root is analog already
    assert type(convert_to_analog(Net(), rpu, ensure_analog_root=False)) is Net
    assert type(convert_to_analog(nn.Linear(2, 2), rpu)) is AnalogLinear
