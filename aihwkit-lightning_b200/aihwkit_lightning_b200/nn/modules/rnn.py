"""Recurrent networks whose matrix products run on analog tiles.

Same module tree, constructor arguments, state-dict keys and errors as the reference's
``nn/modules/rnn/{cells,layers,rnn}.py`` -- every weight matrix is an :class:`AnalogLinear`, so
all the arithmetic of a step goes through the library's forward / backward entry points.

One thing is organised differently.  The input projection ``weight_ih(x_t)`` of a cell does not
depend on the recurrence, and every per-call quantity of the analog forward pass is either local
to an input row (dynamic range, DAC codes, ADC bound) or a function of the weights alone, unless
the layer is in training mode (fresh weight noise per call, range statistics per call).  In
evaluation mode a layer therefore projects the whole ``[steps, batch, features]`` sequence in ONE
analog call -- a GEMM with ``steps * batch`` rows instead of ``steps`` launches with ``batch``
rows -- and only the hidden projection stays inside the time loop.  The values are those of the
per-step evaluation; in training mode the per-step order of calls is kept.
"""
import math
import re
import warnings
from collections import namedtuple
from typing import Any, Callable, List, Optional, Tuple, Type, Union

import torch
from torch import Tensor, cat, sigmoid, stack, tanh, zeros
from torch.nn import GRU, LSTM, RNN, Dropout, Linear, Module, ModuleList, init

from .container import AnalogContainerBase
from .linear import AnalogLinear

LSTMState = namedtuple("LSTMState", ["hx", "cx"])


def _require_config(rpu_config) -> None:
    if rpu_config is None:
        raise ValueError("rpu_config must be provided. Try TorchInferenceRPUConfig()")


class _AnalogCell(Module):
    """Shared plumbing of the cells: a zero state and the split of a step into the part that
    can be taken out of the time loop (``project_input``) and the rest (``step``)."""

    HAS_CELL_STATE = False
    SPLIT_INPUT = True  # False: the input takes part in the recurrent product itself

    input_size: int
    hidden_size: int

    def get_zero_state(self, batch_size: int) -> LSTMState:
        param = next(self.parameters())
        h_x = zeros(batch_size, self.hidden_size, device=param.device, dtype=param.dtype)
        c_x = zeros(batch_size, self.hidden_size, device=param.device, dtype=param.dtype) if self.HAS_CELL_STATE else None
        return LSTMState(h_x, c_x)

    def project_input(self, input_: Tensor) -> Tensor:
        return self.weight_ih(input_)

    def step(self, projected: Tensor, state):
        raise NotImplementedError

    def forward(self, input_: Tensor, state):  # pylint: disable=arguments-differ
        return self.step(self.project_input(input_) if self.SPLIT_INPUT else input_, state)


class AnalogVanillaRNNCell(_AnalogCell):
    """``h' = tanh(W_ih x + W_hh h)`` (`rnn/cells.py:40-104`)."""

    def __init__(self, input_size: int, hidden_size: int, bias: bool, device=None, dtype=None, rpu_config=None):
        super().__init__()
        _require_config(rpu_config)
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.weight_ih = AnalogLinear(input_size, hidden_size, bias, device, dtype, rpu_config)
        self.weight_hh = AnalogLinear(hidden_size, hidden_size, bias, device, dtype, rpu_config)

    def step(self, projected: Tensor, state):
        h_x, _ = state
        out = tanh(projected + self.weight_hh(h_x))
        return out, (out, None)


def _lstm_gates(gates: Tensor, c_x: Tensor) -> Tuple[Tensor, Tuple[Tensor, Tensor]]:
    in_gate, forget_gate, cell_gate, out_gate = gates.chunk(4, 1)
    in_gate = sigmoid(in_gate)
    forget_gate = sigmoid(forget_gate)
    cell_gate = tanh(cell_gate)
    out_gate = sigmoid(out_gate)
    c_y = (forget_gate * c_x) + (in_gate * cell_gate)
    h_y = out_gate * tanh(c_y)
    return h_y, (h_y, c_y)


class AnalogLSTMCell(_AnalogCell):
    """LSTM cell with separate input and hidden matrices, gate order i, f, g, o
    (`rnn/cells.py:107-176`)."""

    HAS_CELL_STATE = True

    def __init__(self, input_size: int, hidden_size: int, bias: bool, device=None, dtype=None, rpu_config=None):
        super().__init__()
        _require_config(rpu_config)
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.weight_ih = AnalogLinear(input_size, 4 * hidden_size, bias, device, dtype, rpu_config)
        self.weight_hh = AnalogLinear(hidden_size, 4 * hidden_size, bias, device, dtype, rpu_config)

    def step(self, projected: Tensor, state):
        h_x, c_x = state
        return _lstm_gates(projected + self.weight_hh(h_x), c_x)


class AnalogLSTMCellCombinedWeight(_AnalogCell):
    """LSTM cell with one ``[4 hidden, input + hidden]`` matrix applied to ``cat(x, h)``
    (`rnn/cells.py:179-251`); nothing of it can leave the time loop."""

    HAS_CELL_STATE = True
    SPLIT_INPUT = False

    def __init__(self, input_size: int, hidden_size: int, bias: bool, device=None, dtype=None, rpu_config=None):
        super().__init__()
        _require_config(rpu_config)
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.weight = AnalogLinear(input_size + hidden_size, 4 * hidden_size, bias, device, dtype, rpu_config)

    def step(self, projected: Tensor, state):
        h_x, c_x = state
        return _lstm_gates(self.weight(cat((projected, h_x), 1)), c_x)


class AnalogGRUCell(_AnalogCell):
    """GRU cell, gate order r, z, n (`rnn/cells.py:254-333`)."""

    def __init__(self, input_size: int, hidden_size: int, bias: bool, device=None, dtype=None, rpu_config=None):
        super().__init__()
        _require_config(rpu_config)
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.weight_ih = AnalogLinear(input_size, 3 * hidden_size, bias, device, dtype, rpu_config)
        self.weight_hh = AnalogLinear(hidden_size, 3 * hidden_size, bias, device, dtype, rpu_config)

    def step(self, projected: Tensor, state):
        h_x, _ = state
        i_r, i_i, i_n = projected.chunk(3, 1)
        h_r, h_i, h_n = self.weight_hh(h_x).chunk(3, 1)
        reset_gate = sigmoid(i_r + h_r)
        input_gate = sigmoid(i_i + h_i)
        new_gate = tanh(i_n + reset_gate * h_n)
        hidden_y = new_gate + input_gate * (h_x - new_gate)
        return hidden_y, (hidden_y, None)


class AnalogRNNLayer(Module):
    """Runs one cell over the leading (time) axis of ``[steps, batch, features]``
    (`rnn/layers.py:20-62`)."""

    REVERSE = False

    def __init__(self, cell: Type, *cell_args: Any):
        super().__init__()
        self.cell = cell(*cell_args)
        self.batch_input_projection = True  # see the module docstring; only acts in eval mode

    def get_zero_state(self, batch_size: int) -> LSTMState:
        return self.cell.get_zero_state(batch_size)

    def forward(self, input_: Tensor, state):  # pylint: disable=arguments-differ
        cell = self.cell
        steps = input_.shape[0]
        order = range(steps - 1, -1, -1) if self.REVERSE else range(steps)
        outputs: List[Optional[Tensor]] = [None] * steps
        if not isinstance(cell, _AnalogCell):  # a user-supplied cell: only its forward is known
            for i in order:
                outputs[i], state = cell(input_[i], state)
            return stack(outputs), state
        hoist = cell.SPLIT_INPUT and self.batch_input_projection and not cell.training and steps > 1
        # one analog call for all steps, or the per-step calls in time order
        seq = cell.project_input(input_) if hoist else input_
        for i in order:
            item = seq[i]
            if not hoist and cell.SPLIT_INPUT:
                item = cell.project_input(item)
            outputs[i], state = cell.step(item, state)
        return stack(outputs), state


class AnalogReverseRNNLayer(AnalogRNNLayer):
    """The same, walking the sequence from its end; outputs stay in input order
    (`rnn/layers.py:65-111`)."""

    REVERSE = True

    @staticmethod
    def reverse(lst: List[Tensor]) -> List[Tensor]:
        return lst[::-1]


class AnalogBidirRNNLayer(Module):
    """A forward and a reverse layer on the same input, outputs concatenated on the feature
    axis (`rnn/layers.py:114-166`)."""

    def __init__(self, cell: Type, *cell_args: Any):
        super().__init__()
        self.directions = ModuleList([AnalogRNNLayer(cell, *cell_args), AnalogReverseRNNLayer(cell, *cell_args)])

    def get_zero_state(self, batch_size: int) -> Tuple[LSTMState, LSTMState]:
        return (self.directions[0].get_zero_state(batch_size), self.directions[1].get_zero_state(batch_size))

    def forward(self, input_: Tensor, states):  # pylint: disable=arguments-differ
        outputs, out_states = [], []
        for direction, state in zip(self.directions, states):
            out, out_state = direction(input_, state)
            outputs.append(out)
            out_states.append(out_state)
        return cat(outputs, -1), out_states


class ModularRNN(Module):
    """A stack of layers with dropout between them (`rnn/rnn.py:40-136`)."""

    def __init__(self, num_layers: int, layer: Type, dropout: float, first_layer_args: Any, other_layer_args: Any):
        super().__init__()
        self.layers = self.init_stacked_analog_lstm(num_layers, layer, first_layer_args, other_layer_args)
        self.num_layers = num_layers
        if num_layers == 1 and dropout > 0:
            warnings.warn(
                "dropout lstm adds dropout layers after all but last recurrent layer, it expects "
                "num_layers greater than 1, but got num_layers = 1"
            )
        self.dropout_layer = Dropout(dropout) if dropout > 0.0 else None

    @staticmethod
    def init_stacked_analog_lstm(num_layers: int, layer: Type, first_layer_args: Any, other_layer_args: Any) -> ModuleList:
        return ModuleList([layer(*first_layer_args)] + [layer(*other_layer_args) for _ in range(num_layers - 1)])

    def get_zero_state(self, batch_size: int) -> List:
        return [lay.get_zero_state(batch_size) for lay in self.layers]

    def forward(self, inp: Tensor, states: List) -> Tuple[Tensor, List]:  # pylint: disable=arguments-differ
        out_states = []
        output = inp
        for i, rnn_layer in enumerate(self.layers):
            output, out_state = rnn_layer(output, states[i])
            if i < self.num_layers - 1 and self.dropout_layer is not None:
                output = self.dropout_layer(output)
            out_states.append(out_state)
        return output, out_states


_ANALOG_KEY = re.compile(r"^rnn\.layers\.(\d+)\.(?:directions\.(\d+)\.)?cell\.weight_(ih|hh)\.(\w+)$")
_TORCH_KEY = re.compile(
    r"^(weight|bias|x_min|x_max|input_range_update_idx|input_range|learnable_weight_clip)_(ih|hh)_l(\d+)(_reverse)?$"
)
_CELL_OF = {RNN: AnalogVanillaRNNCell, GRU: AnalogGRUCell, LSTM: AnalogLSTMCell}


class AnalogRNN(AnalogContainerBase, Module):
    """Multi-layer, optionally bidirectional RNN / LSTM / GRU on analog tiles
    (`rnn/rnn.py:139-578`).

    ``cell`` is the cell class; input is ``[steps, batch, input_size]`` (or ``[steps,
    input_size]`` unbatched), ``batch_first`` and ``proj_size != 0`` raise ``RuntimeError`` as in
    the reference.  ``state_dict()`` uses torch's ``nn.LSTM`` key names (``weight_ih_l0``,
    ``bias_hh_l1_reverse``, and likewise ``input_range_ih_l0`` for the analog state), and
    ``load_state_dict`` accepts those names as well as the module-tree names.
    """

    def __init__(self, cell: Type, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True,
                 batch_first: bool = False, bidir: bool = False, dropout: float = 0.0, proj_size: int = 0,
                 xavier: bool = False, device=None, dtype=None, rpu_config=None):
        # pylint: disable=too-many-arguments
        super().__init__()
        layer = AnalogBidirRNNLayer if bidir else AnalogRNNLayer
        num_dirs = 2 if bidir else 1
        if batch_first:
            raise RuntimeError("batch_first is not supported for AnalogRNN")
        if proj_size != 0:
            raise RuntimeError("proj_size != 0 not supported for AnalogRNN")
        self.proj_size = 0
        self.rnn = ModularRNN(
            num_layers, layer, dropout,
            first_layer_args=[cell, input_size, hidden_size, bias, device, dtype, rpu_config],
            other_layer_args=[cell, num_dirs * hidden_size, hidden_size, bias, device, dtype, rpu_config],
        )
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.num_layers = num_layers
        self.batch_first = batch_first
        self.dropout = dropout
        self.bidirectional = bidir
        self.reset_parameters(xavier)
        self._register_load_state_dict_pre_hook(self.update_state_dict)
        self._register_state_dict_hook(self.return_pytorch_state_dict)

    # -- initialisation -------------------------------------------------------------------------
    @torch.no_grad()
    def init_layers(self, weight_init_fn: Callable, bias_init_fn: Optional[Callable] = None) -> None:
        """Apply in-place initialisers to every weight matrix (and bias; the weight initialiser
        is used for the bias when none is given)."""
        for module in self.modules():
            if isinstance(module, (AnalogLinear, Linear)):
                weight_init_fn(module.weight.data)
                if module.bias is not None:
                    (bias_init_fn or weight_init_fn)(module.bias.data)

    def reset_parameters(self, xavier: bool = False) -> None:
        """torch's RNN default ``U(-1/sqrt(hidden), 1/sqrt(hidden))``, or Xavier-uniform weights
        with zero biases."""
        if xavier:
            self.init_layers(init.xavier_uniform_, init.zeros_)
        else:
            stdv = 1.0 / math.sqrt(self.hidden_size)
            self.init_layers(lambda x: x.uniform_(-stdv, stdv))

    def get_zero_state(self, batch_size: int) -> List:
        return self.rnn.get_zero_state(batch_size)

    # -- forward ----------------------------------------------------------------------------------
    def _flat_states(self, states: List) -> List:
        return [s for pair in states for s in pair] if self.bidirectional else list(states)

    def forward(self, inp: Tensor, states: Optional[List] = None) -> Tuple[Tensor, List]:
        # pylint: disable=arguments-differ
        if inp.dim() not in (2, 3):
            raise RuntimeError(f"RNN: Expected input to be 2D or 3D, got {inp.dim()}D tensor instead")
        if states is not None and len(states) != self.num_layers:
            raise RuntimeError(f"Expecting {self.num_layers} states, but received {len(states)}")
        batched = inp.dim() == 3
        if states is not None:
            want = 2 if batched else 1
            what = "batched 3-D" if batched else "unbatched 2-D"
            for state in self._flat_states(states):
                for t_name in ("hx", "cx"):
                    d = getattr(state, t_name).dim()
                    if d != want:
                        raise RuntimeError(
                            f"For {what} input, {t_name} should be {want}-D but got {d}-D tensor"
                        )
        if not batched:
            inp = inp.unsqueeze(1)
        batch = inp.size(1)
        if states is None:
            states = self.get_zero_state(batch)
        for state in self._flat_states(states):
            self.check_forward_args(inp, state, batch)
        return self.rnn(inp, states)

    def check_input(self, inp: Tensor) -> None:
        if self.input_size != inp.size(-1):
            raise RuntimeError(
                f"input.size(-1) must be equal to input_size. Expected {self.input_size}, got {inp.size(-1)}"
            )

    def check_hidden_size(self, h_x: Tensor, expected_hidden_size: Tuple[int, int],
                          msg: str = "Expected hidden size {}, got {}") -> None:
        if h_x.size() != expected_hidden_size:
            raise RuntimeError(msg.format(expected_hidden_size, list(h_x.size())))

    def check_forward_args(self, inp: Tensor, hidden: LSTMState, batch_size: int) -> None:
        self.check_input(inp)
        self.check_hidden_size(hidden.hx, (batch_size, self.hidden_size))
        if hidden.cx is not None:
            self.check_hidden_size(hidden.cx, (batch_size, self.hidden_size))

    # -- state-dict key translation -------------------------------------------------------------------
    def update_state_dict(self, state_dict, prefix="", *_args, **_kwargs) -> None:
        """Load pre-hook: rename torch-style keys below ``prefix`` (``weight_ih_l0_reverse`` ...)
        to this module's tree (``rnn.layers.0.directions.1.cell.weight_ih.weight``)."""
        bidir = self.bidirectional
        for key in list(state_dict.keys()):
            if not key.startswith(prefix):
                continue
            found = _TORCH_KEY.match(key[len(prefix):])
            if found is None:
                continue
            tensor_name, i_h, layer, reverse = found.groups()
            direction = f".directions.{1 if reverse else 0}" if bidir else ""
            state_dict[f"{prefix}rnn.layers.{layer}{direction}.cell.weight_{i_h}.{tensor_name}"] = state_dict.pop(key)

    @staticmethod
    def return_pytorch_state_dict(module, state_dict, prefix, local_metadata) -> None:
        """State-dict hook: the inverse renaming, so that a checkpoint of this module loads into
        ``nn.LSTM`` / ``nn.GRU`` / ``nn.RNN`` (its weights and biases) and vice versa."""
        # pylint: disable=unused-argument
        for key in list(state_dict.keys()):
            if not key.startswith(prefix):
                continue
            found = _ANALOG_KEY.match(key[len(prefix):])
            if found is None:
                continue
            layer, direction, i_h, tensor_name = found.groups()
            reverse = "_reverse" if direction == "1" else ""
            state_dict[f"{prefix}{tensor_name}_{i_h}_l{layer}{reverse}"] = state_dict.pop(key)

    # -- conversion ---------------------------------------------------------------------------------
    def _cells(self, layer: int) -> List[Module]:
        """Cells of stacked layer ``layer``: [forward] or [forward, reverse]."""
        lay = self.rnn.layers[layer]
        return [d.cell for d in lay.directions] if self.bidirectional else [lay.cell]

    @staticmethod
    def update_digital_attrs(digital_layer: Union[RNN, LSTM, GRU], analog_cell: Module, layer: int,
                             reverse: bool) -> None:
        """Copy one cell's matrices (and biases) into torch's flat parameters."""
        suffix = f"_l{layer}" + ("_reverse" if reverse else "")
        for i_h in ("ih", "hh"):
            lin = getattr(analog_cell, f"weight_{i_h}")
            getattr(digital_layer, f"weight_{i_h}{suffix}").copy_(lin.weight.detach())
            if lin.bias is not None:
                getattr(digital_layer, f"bias_{i_h}{suffix}").copy_(lin.bias.detach())

    @classmethod
    def to_digital(cls, module: "AnalogRNN", *_: Any, **__: Any) -> Union[RNN, LSTM, GRU]:
        """The ``nn.RNN`` / ``nn.LSTM`` / ``nn.GRU`` with this module's shape and weights."""
        first = module._cells(0)[0]  # pylint: disable=protected-access
        weight = first.weight_ih.weight
        has_bias = first.weight_hh.bias is not None
        common = dict(bias=has_bias, batch_first=module.batch_first, dropout=module.dropout,
                      bidirectional=module.bidirectional, device=weight.device, dtype=weight.dtype)
        if isinstance(first, AnalogVanillaRNNCell):
            digital: Union[RNN, LSTM, GRU] = RNN(module.input_size, module.hidden_size, module.num_layers,
                                                 nonlinearity="tanh", **common)
        elif isinstance(first, AnalogLSTMCell):
            digital = LSTM(module.input_size, module.hidden_size, module.num_layers, proj_size=module.proj_size,
                           **common)
        elif isinstance(first, AnalogGRUCell):
            digital = GRU(module.input_size, module.hidden_size, module.num_layers, **common)
        else:
            raise TypeError(f"no torch counterpart for cell type {type(first).__name__}")
        with torch.no_grad():
            for layer in range(module.num_layers):
                for direction, cell in enumerate(module._cells(layer)):  # pylint: disable=protected-access
                    cls.update_digital_attrs(digital, cell, layer, direction == 1)
        return digital

    @classmethod
    def from_digital(cls, module: Union[RNN, LSTM, GRU], rpu_config=None,
                     realistic_read_write: bool = False) -> "AnalogRNN":
        """An ``AnalogRNN`` with the cell type, shape and weights of a torch recurrent module.
        The third argument is handed on as ``xavier`` (as the reference does); the weights are
        overwritten by the digital ones either way."""
        analog = cls(_CELL_OF[type(module)], module.input_size, module.hidden_size, module.num_layers,
                     module.bias is not False, module.batch_first, module.bidirectional, module.dropout,
                     module.proj_size, realistic_read_write, module.weight_hh_l0.device, module.weight_hh_l0.dtype,
                     rpu_config)
        for layer in range(analog.num_layers):
            for direction, cell in enumerate(analog._cells(layer)):  # pylint: disable=protected-access
                suffix = f"_l{layer}" + ("_reverse" if direction == 1 else "")
                for i_h in ("ih", "hh"):
                    bias = getattr(module, f"bias_{i_h}{suffix}") if module.bias is not False else None
                    getattr(cell, f"weight_{i_h}").set_weights_and_biases(getattr(module, f"weight_{i_h}{suffix}"), bias)
        return analog


__all__ = ["LSTMState", "AnalogVanillaRNNCell", "AnalogLSTMCell", "AnalogLSTMCellCombinedWeight", "AnalogGRUCell",
           "AnalogRNNLayer", "AnalogReverseRNNLayer", "AnalogBidirRNNLayer", "ModularRNN", "AnalogRNN"]
