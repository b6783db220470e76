"""RWKV-6 ("Finch") blocks: data-dependent token-shift mixing through a low-rank adapter, per-channel
data-dependent decay, the wkv6 linear-attention recurrence (``ops/wkv6.py``), group-norm + gate, and the
squared-ReLU channel mix.  Parameter names and initialisation schedules follow the reference
(``megatron/model/rwkv/v6/rwkv.py:100-366``) so checkpoints interchange.  Tensor parallelism is not
supported for this mixer (enforced by the config system); activations are ``[b, t, c]`` inside the block."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.wkv6 import wkv6

TIME_MIX_EXTRA_DIM = 32
TIME_DECAY_EXTRA_DIM = 64


def _dev():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None


def _shift(x):
    """x[t-1] with zeros at t = 0 (token shift along dim 1)."""
    return F.pad(x, (0, 0, 1, -1))


class RWKV_TimeMix(nn.Module):
    def __init__(self, neox_args, layer_number):
        super().__init__()
        a = neox_args
        self.neox_args, self.layer_number = a, layer_number
        h, da, L = a.hidden_size, a.dim_att, a.num_layers
        dev, dt = _dev(), a.params_dtype
        with torch.no_grad():
            r01 = layer_number / max(L - 1, 1)
            r10 = 1.0 - layer_number / L
            ddd = (torch.arange(h, dtype=torch.float32) / h).view(1, 1, h)
            mk = lambda t: nn.Parameter(t.to(device=dev, dtype=dt))
            self.time_maa_x = mk(1.0 - torch.pow(ddd, r10))
            self.time_maa_w = mk(1.0 - torch.pow(ddd, r10))
            self.time_maa_k = mk(1.0 - torch.pow(ddd, r10))
            self.time_maa_v = mk(1.0 - (torch.pow(ddd, r10) + 0.3 * r01))
            self.time_maa_r = mk(1.0 - torch.pow(ddd, 0.5 * r10))
            self.time_maa_g = mk(1.0 - torch.pow(ddd, 0.5 * r10))
            self.time_maa_w1 = mk(torch.zeros(h, TIME_MIX_EXTRA_DIM * 5).uniform_(-1e-4, 1e-4))
            self.time_maa_w2 = mk(torch.zeros(5, TIME_MIX_EXTRA_DIM, h).uniform_(-1e-4, 1e-4))
            n = torch.arange(da, dtype=torch.float32)
            decay_speed = -6 + 5 * (n / max(da - 1, 1)) ** (0.7 + 1.3 * r01)
            self.time_decay = mk(decay_speed.reshape(1, 1, da))
            self.time_decay_w1 = mk(torch.zeros(h, TIME_DECAY_EXTRA_DIM).uniform_(-1e-4, 1e-4))
            self.time_decay_w2 = mk(torch.zeros(TIME_DECAY_EXTRA_DIM, da).uniform_(-1e-4, 1e-4))
            zigzag = ((n + 1) % 3 - 1) * 0.1
            faaaa = r01 * (1 - n / max(da - 1, 1)) + zigzag
            self.time_faaaa = mk(faaaa.reshape(a.num_attention_heads, a.head_size))
        lin = lambda i, o: nn.Linear(i, o, bias=False, device=dev, dtype=dt)
        self.receptance, self.key, self.value = lin(h, da), lin(h, da), lin(h, da)
        self.output, self.gate = lin(da, h), lin(h, da)
        self.ln_x = nn.GroupNorm(a.num_attention_heads, da, eps=(1e-5) * (8 ** 2), device=dev, dtype=dt)

    def forward(self, x):
        B, T, C = x.size()
        H = self.neox_args.num_attention_heads
        xx = _shift(x) - x
        xxx = x + xx * self.time_maa_x
        xxx = torch.tanh(xxx @ self.time_maa_w1).view(B * T, 5, -1).transpose(0, 1)
        mw, mk, mv, mr, mg = torch.bmm(xxx, self.time_maa_w2).view(5, B, T, -1).unbind(dim=0)
        xw = x + xx * (self.time_maa_w + mw)
        xk = x + xx * (self.time_maa_k + mk)
        xv = x + xx * (self.time_maa_v + mv)
        xr = x + xx * (self.time_maa_r + mr)
        xg = x + xx * (self.time_maa_g + mg)
        r, k, v = self.receptance(xr), self.key(xk), self.value(xv)
        g = F.silu(self.gate(xg))
        w = self.time_decay + torch.tanh(xw @ self.time_decay_w1) @ self.time_decay_w2
        y = wkv6(r, k, v, w, self.time_faaaa)
        y = self.ln_x(y.view(B * T, -1)).view(B, T, -1)
        return self.output(y * g)


class RWKV_ChannelMix(nn.Module):
    def __init__(self, neox_args, layer_number):
        super().__init__()
        a = neox_args
        dev, dt = _dev(), a.params_dtype
        with torch.no_grad():
            r10 = 1.0 - layer_number / a.num_layers
            ddd = (torch.arange(a.hidden_size, dtype=torch.float32) / a.hidden_size).view(1, 1, -1)
            self.time_maa_k = nn.Parameter((1.0 - torch.pow(ddd, r10)).to(device=dev, dtype=dt))
            self.time_maa_r = nn.Parameter((1.0 - torch.pow(ddd, r10)).to(device=dev, dtype=dt))
        self.key = nn.Linear(a.hidden_size, a.ffn_dim, bias=False, device=dev, dtype=dt)
        self.receptance = nn.Linear(a.hidden_size, a.hidden_size, bias=False, device=dev, dtype=dt)
        self.value = nn.Linear(a.ffn_dim, a.hidden_size, bias=False, device=dev, dtype=dt)

    def forward(self, x):
        xx = _shift(x) - x
        k = torch.relu(self.key(x + xx * self.time_maa_k)) ** 2
        return torch.sigmoid(self.receptance(x + xx * self.time_maa_r)) * self.value(k)


class RWKVResidualLayer(nn.Module):
    def __init__(self, neox_args, layer_number):
        super().__init__()
        a = neox_args
        self.neox_args, self.layer_number = a, layer_number
        assert a.intermediate_size is None or a.expansion_factor is None, \
            "Must pass either the absolute intermediate size or the relative expansion factor"
        if a.dim_att is None:
            a.dim_att = a.hidden_size
        ffn = a.intermediate_size if a.intermediate_size else int((a.expansion_factor or 3.5) * a.hidden_size)
        a.ffn_dim = int(ffn // 32 * 32)
        assert a.hidden_size % 32 == 0 and a.dim_att % 32 == 0 and a.ffn_dim % 32 == 0
        assert a.dim_att % a.num_attention_heads == 0
        a.head_size = a.dim_att // a.num_attention_heads
        dev, dt = _dev(), a.params_dtype
        self.ln1 = nn.LayerNorm(a.hidden_size, device=dev, dtype=dt)
        self.ln2 = nn.LayerNorm(a.hidden_size, device=dev, dtype=dt)
        self.att = RWKV_TimeMix(a, layer_number)
        self.ffn = RWKV_ChannelMix(a, layer_number)
        self.drop0 = nn.Dropout(p=a.attention_dropout) if a.attention_dropout > 0 else nn.Identity()
        self.drop1 = nn.Dropout(p=a.hidden_dropout) if a.hidden_dropout > 0 else nn.Identity()

    def forward(self, x):
        # the stack hands over [s, b, h]; the recurrence wants time on dim 1
        x = x.transpose(0, 1)
        if self.layer_number == 0:
            x = self.ln1(x)
        x = self.drop0(x + self.att(self.ln1(x)))
        x = self.drop1(x + self.ffn(self.ln2(x)))
        return x.transpose(0, 1).contiguous()


class RWKVResidualLayerPipe(RWKVResidualLayer):
    def forward(self, args):
        assert len(args) == 2
        hidden_states, mask = args
        return super().forward(hidden_states), mask
