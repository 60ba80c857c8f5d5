"""Small instances of the two model families the benchmark configurations name, written against
plain ``nn.Linear`` / ``nn.Conv2d`` so that they can be converted to analog layers by the
product (GPU) or by the oracle wrappers below (CPU): a Phi-3-shaped decoder (fused qkv and
gate_up projections, RMSNorm, rotary embedding, causal attention, analog lm_head) and a
CIFAR-shaped ResNet of basic blocks."""
import math

import torch
from torch import nn
from torch.nn import functional as TF

import analog_oracle as O


# ---------------------------------------------------------------------------------------------
class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return (v * self.weight.float()).to(x.dtype)


def rotary(q, k):
    b, h, s, d = q.shape
    pos = torch.arange(s, device=q.device, dtype=torch.float32)
    inv = 1.0 / (10000 ** (torch.arange(0, d, 2, device=q.device, dtype=torch.float32) / d))
    ang = pos[:, None] * inv[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)

    def rot(x):
        x1, x2 = x[..., : d // 2], x[..., d // 2:]
        return torch.cat([-x2, x1], -1)

    qf, kf = q.float(), k.float()
    return (qf * cos + rot(qf) * sin).to(q.dtype), (kf * cos + rot(kf) * sin).to(k.dtype)


class DecoderLayer(nn.Module):
    def __init__(self, d, heads, mlp):
        super().__init__()
        self.heads = heads
        self.norm1, self.norm2 = RMSNorm(d), RMSNorm(d)
        self.qkv_proj = nn.Linear(d, 3 * d, bias=False)
        self.o_proj = nn.Linear(d, d, bias=False)
        self.gate_up_proj = nn.Linear(d, 2 * mlp, bias=False)
        self.down_proj = nn.Linear(mlp, d, bias=False)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv_proj(self.norm1(x)).chunk(3, dim=-1)
        shape = lambda t: t.view(b, s, self.heads, d // self.heads).transpose(1, 2)  # noqa: E731
        q, k = rotary(shape(q), shape(k))
        att = TF.scaled_dot_product_attention(q.float(), k.float(), shape(v).float(), is_causal=True).to(x.dtype)
        x = x + self.o_proj(att.transpose(1, 2).reshape(b, s, d))
        gate, up = self.gate_up_proj(self.norm2(x)).chunk(2, dim=-1)
        return x + self.down_proj(TF.silu(gate) * up)


class TinyPhi3(nn.Module):
    """Phi-3-mini layout at reduced width: every Linear (including lm_head) becomes analog."""

    def __init__(self, vocab=512, d=256, heads=4, mlp=512, layers=2):
        super().__init__()
        self.embed = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList([DecoderLayer(d, heads, mlp) for _ in range(layers)])
        self.norm = RMSNorm(d)
        self.lm_head = nn.Linear(d, vocab, bias=False)

    def forward(self, ids):
        x = self.embed(ids)
        for layer in self.layers:
            x = layer(x)
        return self.lm_head(self.norm(x))


# ---------------------------------------------------------------------------------------------
class BasicBlock(nn.Module):
    def __init__(self, cin, cout, stride):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, cout, 3, stride=stride, padding=1, bias=False)
        self.bn1 = nn.BatchNorm2d(cout)
        self.conv2 = nn.Conv2d(cout, cout, 3, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(cout)
        self.short = None
        if stride != 1 or cin != cout:
            self.short = nn.Conv2d(cin, cout, 1, stride=stride, bias=False)

    def forward(self, x):
        y = TF.relu(self.bn1(self.conv1(x)))
        y = self.bn2(self.conv2(y))
        return TF.relu(y + (x if self.short is None else self.short(x)))


class TinyResNet(nn.Module):
    """ResNet-32 layout (3 stages of basic blocks, 16/32/64 channels, 3x3 convs, FC 64->10) with
    ``blocks`` blocks per stage (5 gives ResNet-32)."""

    def __init__(self, blocks=1, classes=10):
        super().__init__()
        self.conv = nn.Conv2d(3, 16, 3, padding=1, bias=False)
        self.bn = nn.BatchNorm2d(16)
        layers, cin = [], 16
        for cout, stride in ((16, 1), (32, 2), (64, 2)):
            for i in range(blocks):
                layers.append(BasicBlock(cin, cout, stride if i == 0 else 1))
                cin = cout
        self.blocks = nn.Sequential(*layers)
        self.fc = nn.Linear(64, classes)

    def forward(self, x):
        x = TF.relu(self.bn(self.conv(x)))
        x = self.blocks(x)
        return self.fc(x.mean((2, 3)))


# ---------------------------------------------------------------------------------------------
# CPU stand-ins that evaluate a layer through the oracle (autograd flavour)
class OracleLinear(nn.Module):
    def __init__(self, module: nn.Linear, rpu_config):
        super().__init__()
        self.weight, self.bias, self.rpu_config = module.weight, module.bias, rpu_config
        self.in_sizes = O.split_sizes(module.in_features, rpu_config.mapping.max_input_size)
        irp = rpu_config.pre_post.input_range
        self.input_range = None
        if irp.enable and not irp.dynamic:
            self.input_range = nn.Parameter(torch.full((len(self.in_sizes),), float(irp.init_value),
                                                       dtype=module.weight.dtype))
            self.register_buffer("idx", torch.zeros(len(self.in_sizes), dtype=module.weight.dtype))

    def forward(self, x):
        return O.linear_autograd(x, self.weight, self.bias, self.input_range,
                                 getattr(self, "idx", None), self.in_sizes, self.training, self.rpu_config)


class OracleConv2d(nn.Module):
    def __init__(self, module: nn.Conv2d, rpu_config):
        super().__init__()
        self.conv, self.rpu_config = module, rpu_config
        k = module.in_channels * module.kernel_size[0] * module.kernel_size[1]
        self.in_sizes = O.split_sizes(k, rpu_config.mapping.max_input_size)

    def forward(self, x):
        c = self.conv
        patches = TF.unfold(x, c.kernel_size, dilation=c.dilation, padding=c.padding, stride=c.stride).transpose(-1, -2)
        out = O.linear_autograd(patches, c.weight.view(c.out_channels, -1), c.bias, None, None, self.in_sizes,
                                self.training, self.rpu_config)
        ho = (x.shape[-2] + 2 * c.padding[0] - c.dilation[0] * (c.kernel_size[0] - 1) - 1) // c.stride[0] + 1
        return out.transpose(-1, -2).reshape(x.shape[0], c.out_channels, ho, -1)


def to_oracle(model: nn.Module, rpu_config) -> nn.Module:
    for name, child in list(model.named_children()):
        if isinstance(child, nn.Linear):
            setattr(model, name, OracleLinear(child, rpu_config))
        elif isinstance(child, nn.Conv2d):
            setattr(model, name, OracleConv2d(child, rpu_config))
        else:
            to_oracle(child, rpu_config)
    return model
