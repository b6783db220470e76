"""gMLP / aMLP blocks (Liu et al. 2021, "Pay Attention to MLPs"; reference ``megatron/model/gmlp.py:28-141``):
channel projection -> GeLU -> spatial gating unit (a causal, lower-triangular sequence x sequence projection
applied to half of the channels, optionally helped by a tiny single-head attention for ``amlp``) ->
channel projection, with a pre-norm residual."""
from __future__ import annotations


import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from ..ops.linear import linear
from ..parallel import mpu
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
from .norms import get_norm


class TinyAttention(nn.Module):
    def __init__(self, neox_args, d_attn, d_ff, mask_fn):
        super().__init__()
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None
        self.proj_qkv = nn.Linear(d_ff * 2, 3 * d_attn, device=dev, dtype=neox_args.params_dtype)
        self.scale = d_attn ** -0.5
        self.proj_ffn = nn.Linear(d_attn, d_ff, device=dev, dtype=neox_args.params_dtype)

    def forward(self, x, attention_mask):
        q, k, v = torch.chunk(self.proj_qkv(x), 3, dim=-1)          # x: [s, b, 2*d_ff]
        w = torch.einsum("snd,tnd->nst", q, k).unsqueeze(1)           # [b, 1, s, s]
        s = w.shape[-1]
        if attention_mask is None:
            attention_mask = torch.ones(s, s, dtype=torch.bool, device=x.device).triu(1)[None, None]
        a = OF.scaled_masked_softmax(w, attention_mask.expand(w.shape[0] if attention_mask.shape[0] > 1 else 1, 1, s, s),
                                     self.scale).squeeze(1)
        return self.proj_ffn(torch.einsum("nst,tnd->snd", a.to(v.dtype), v))


class SpatialGatingUnit(nn.Module):
    def __init__(self, neox_args, d_ff, d_attn=None, causal=True, mask_fn=None):
        super().__init__()
        self.causal = causal
        self.use_attn = d_attn is not None
        norm, eps = get_norm(neox_args)
        self.norm = norm(d_ff, eps=eps)
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None
        self.proj = nn.Linear(neox_args.seq_length, neox_args.seq_length, device=dev, dtype=neox_args.params_dtype)
        if self.use_attn:
            self.attn = TinyAttention(neox_args, d_attn, d_ff, mask_fn)
        nn.init.zeros_(self.proj.weight)
        nn.init.constant_(self.proj.bias, 1.0)

    def forward(self, x, attention_mask):
        n = x.shape[0]
        x = x.transpose(0, 1)                                        # [b, s, d]
        res, gate = x.chunk(2, dim=-1)
        gate = self.norm(gate)
        weight, bias = self.proj.weight, self.proj.bias
        if self.causal:
            weight = weight[:n, :n].tril()
            bias = bias[:n]
        gate = linear(gate.transpose(2, 1).contiguous(), weight.contiguous(), bias).transpose(2, 1)
        if self.use_attn:
            gate = gate + self.attn(x.transpose(0, 1), attention_mask).transpose(0, 1)
        return (gate * res).transpose(0, 1)


class GMLPBlock(nn.Module):
    def __init__(self, neox_args, init_method, output_layer_init_method, layer_number, ff_mult=4, mask_fn=None):
        super().__init__()
        self.layer_number = layer_number
        ff_dim = neox_args.hidden_size * ff_mult
        norm, eps = get_norm(neox_args)
        self.norm = norm(neox_args.hidden_size, eps=eps)
        self.input_linear = ColumnParallelLinear(neox_args, neox_args.hidden_size, ff_dim * 2, gather_output=False,
                                                 init_method=init_method, skip_bias_add=True)
        self.activation_func = lambda t: F.gelu(t, approximate="tanh")
        ff_dim_parallel = mpu.divide(ff_dim, mpu.get_model_parallel_world_size())
        d_attn = neox_args.gmlp_attn_dim if neox_args.attention_config[layer_number] == "amlp" else None
        self.sgu = SpatialGatingUnit(neox_args, ff_dim_parallel, d_attn, causal=True, mask_fn=mask_fn)
        self.output_linear = RowParallelLinear(neox_args, ff_dim, neox_args.hidden_size, input_is_parallel=True,
                                               init_method=output_layer_init_method, skip_bias_add=True)

    def forward(self, args):
        assert len(args) == 2, "GMLPBlock expects 2 arguments"
        x, attention_mask = args
        h = self.norm(x)
        h, _ = self.input_linear(h)
        h = self.activation_func(h)
        h = self.sgu(h, attention_mask)
        h, _ = self.output_linear(h)
        return h + x, attention_mask
