"""Recurrent models, inputs and settings shared by the RNN fixture generator and its tests."""
import torch

# name -> (torch class, kwargs of the torch module, mode, forward settings)
CASES = {
    "lstm_bidir_eval": dict(kind="LSTM", module=dict(num_layers=2, bidirectional=True), train=False, adc=False),
    "gru_eval_adc": dict(kind="GRU", module=dict(num_layers=1), train=False, adc=True),
    "rnn_nobias_eval": dict(kind="RNN", module=dict(num_layers=2, bias=False), train=False, adc=False),
    "lstm_train_static": dict(kind="LSTM", module=dict(num_layers=1), train=True, adc=False),
    "gru_bidir_train": dict(kind="GRU", module=dict(num_layers=2, bidirectional=True), train=True, adc=False),
}
STEPS, BATCH, INPUT, HIDDEN = 5, 3, 12, 16


def make_rpu_config(cls, case):
    """Quantised inputs on two tiles per matrix, no noise (the fixture is deterministic);
    evaluation cases use the dynamic input range, training cases a fixed learned one."""
    rpu = cls()
    rpu.mapping.max_input_size = 8
    rpu.forward.inp_res = 254
    rpu.forward.out_noise = 0.0
    if case["adc"]:
        rpu.forward.out_res = 254
        rpu.forward.out_bound = 10.0
    ir = rpu.pre_post.input_range
    ir.enable = True
    if case["train"]:
        ir.dynamic = False
        ir.learn_input_range = True
        ir.init_value = 1.5
        ir.init_from_data = 0
        ir.decay = 0.01
        ir.input_min_percentage = 0.95
    else:
        ir.dynamic = True
    return rpu


def build_digital(case):
    torch.manual_seed(5)
    cls = getattr(torch.nn, case["kind"])
    return cls(INPUT, HIDDEN, **case["module"])


def make_input(case):
    gen = torch.Generator().manual_seed(13)
    x = torch.randn(STEPS, BATCH, INPUT, generator=gen)
    n_dir = 2 if case["module"].get("bidirectional") else 1
    g = torch.randn(STEPS, BATCH, HIDDEN * n_dir, generator=gen)
    return x, g
