"""Runs the reference's `AnalogRNN` (converted from seeded torch LSTM / GRU / RNN modules) on
the CPU and stores outputs, final states and -- for the training cases -- gradients.

Usage (needs the reference tree, which the test machines do not have):
    python tests/golden/make_rnn_golden.py <path to the reference's src directory>
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import rnn_cases as RC  # noqa: E402


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_rnn_golden.py <path to the reference's src directory>")
    sys.path.insert(0, sys.argv[1])
    from aihwkit_lightning.nn.conversion import convert_to_analog
    from aihwkit_lightning.simulator.configs import TorchInferenceRPUConfig

    out = {}
    for name, case in RC.CASES.items():
        rpu = RC.make_rpu_config(TorchInferenceRPUConfig, case)
        model = convert_to_analog(RC.build_digital(case), rpu, ensure_analog_root=False)
        model.train(case["train"])
        x, g = RC.make_input(case)
        x.requires_grad_(case["train"])
        y, states = model(x)
        rec = dict(out=y.detach().clone())
        flat = [s for pair in states for s in pair] if case["module"].get("bidirectional") else states
        rec["h"] = [s[0].detach().clone() for s in flat]
        rec["c"] = [s[1].detach().clone() for s in flat if s[1] is not None]
        if case["train"]:
            (y * g).sum().backward()
            rec["grad_x"] = x.grad.clone()
            rec["grads"] = {k: p.grad.clone() for k, p in model.named_parameters() if p.grad is not None}
        out[name] = rec
        print("ok", name, tuple(y.shape), float(y.abs().mean()), sorted(rec.get("grads", {}))[:3])
    torch.save(out, os.path.join(HERE, "rnn.pt"))


if __name__ == "__main__":
    main()
