"""Mamba (selective state space) mixer with the inner dimension sharded over tensor-parallel ranks
(reference ``megatron/model/mamba/mamba.py:26-413``): ``in_proj`` column-parallel, depth-wise causal conv1d and
the scan act per channel so they need no communication, ``x_proj`` row-parallel with an explicit all-reduce
(every rank needs the full ``dt``, ``B``, ``C``), ``dt_proj`` local, ``A_log`` / ``D`` kept in fp32 and excluded
from weight decay, ``out_proj`` row-parallel.  Everything stays channel-last (``[b, l, d]``)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.selective_scan import causal_conv1d, selective_scan
from ..parallel import mappings as M
from ..parallel import mpu
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
from .norms import get_norm


class ParallelMambaBlock(nn.Module):
    def __init__(self, neox_args, init_method, output_layer_init_method):
        super().__init__()
        a = neox_args
        self.neox_args = a
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None
        dt = a.params_dtype
        assert not (a.mamba_use_bias_in_linears and a.mamba_inner_func_fusion), \
            "Mamba fused inner fn and bias in x_proj not compatible!"
        assert a.intermediate_size is None or a.expansion_factor is None, \
            "Must pass either the absolute intermediate size or the relative expansion factor for the mamba projections"
        self.d_model, self.d_state, self.d_conv = a.hidden_size, 16, 4
        self.d_inner = a.intermediate_size if a.intermediate_size else int((a.expansion_factor or 2) * self.d_model)
        self.dt_rank = math.ceil(self.d_model / 16)
        tp = mpu.get_model_parallel_world_size()
        self.d_inner_per_rank = mpu.divide(self.d_inner, tp)
        use_bias = a.mamba_use_bias_in_linears
        self.in_proj = ColumnParallelLinear(a, self.d_model, self.d_inner * 2, gather_output=False,
                                            init_method=init_method, skip_bias_add=not use_bias, bias=use_bias)
        self.conv1d = nn.Conv1d(self.d_inner_per_rank, self.d_inner_per_rank, bias=a.mamba_use_bias_in_conv,
                                kernel_size=self.d_conv, groups=self.d_inner_per_rank, padding=self.d_conv - 1,
                                device=dev, dtype=dt)
        self.x_proj = RowParallelLinear(a, self.d_inner, self.dt_rank + self.d_state * 2, input_is_parallel=True,
                                        init_method=init_method, skip_bias_add=not use_bias, parallel_output=True,
                                        bias=use_bias)
        self.dt_proj = nn.Linear(self.dt_rank, self.d_inner_per_rank, bias=True, device=dev, dtype=dt)
        std = self.dt_rank ** -0.5
        nn.init.uniform_(self.dt_proj.weight, -std, std)
        dt_min, dt_max, floor = 0.001, 0.1, 1e-4
        dtv = torch.exp(torch.rand(self.d_inner_per_rank) * (math.log(dt_max) - math.log(dt_min))
                        + math.log(dt_min)).clamp(min=floor)
        with torch.no_grad():
            self.dt_proj.bias.copy_((dtv + torch.log(-torch.expm1(-dtv))).to(dt))
        A = torch.arange(1, self.d_state + 1, dtype=torch.float32).repeat(self.d_inner_per_rank, 1)
        p_dtype = torch.float32 if a.mamba_selective_fp32_params else dt
        self.A_log = nn.Parameter(torch.log(A).to(device=dev, dtype=p_dtype))
        self.D = nn.Parameter(torch.ones(self.d_inner_per_rank, device=dev, dtype=p_dtype))
        self.A_log._no_weight_decay = True
        self.D._no_weight_decay = True
        for p in (self.A_log, self.D, self.conv1d.weight, self.dt_proj.weight, self.dt_proj.bias):
            p.model_parallel = tp > 1
        if self.conv1d.bias is not None:
            self.conv1d.bias.model_parallel = tp > 1
        self.out_proj = RowParallelLinear(a, self.d_inner, self.d_model, input_is_parallel=True,
                                          init_method=output_layer_init_method, skip_bias_add=not use_bias,
                                          bias=use_bias, parallel_output=False)

    def forward(self, hidden_states):
        seqlen, batch, _ = hidden_states.shape
        xz, _ = self.in_proj(hidden_states)                       # [l, b, 2*d/tp]
        xz = xz.transpose(0, 1)                                   # [b, l, 2*d/tp]
        x, z = xz.chunk(2, dim=-1)
        x = causal_conv1d(x, self.conv1d.weight.squeeze(1), self.conv1d.bias, activation="silu")
        x_dbl, _ = self.x_proj(x.reshape(batch * seqlen, -1))
        x_dbl = M.reduce_from_model_parallel_region(x_dbl)        # dt, B, C are needed in full on every rank
        dt, B, C = torch.split(x_dbl, [self.dt_rank, self.d_state, self.d_state], dim=-1)
        dt = F.linear(dt, self.dt_proj.weight).view(batch, seqlen, -1)
        B = B.reshape(batch, seqlen, self.d_state)
        C = C.reshape(batch, seqlen, self.d_state)
        A = -torch.exp(self.A_log.float())
        y = selective_scan(x.contiguous(), dt, A, B, C, self.D.float(), z.contiguous(), self.dt_proj.bias.float())
        out, _ = self.out_proj(y)
        return out.transpose(0, 1).contiguous()


class ParallelMambaResidualLayer(nn.Module):
    """Pre-norm residual wrapper around the Mamba mixer."""

    def __init__(self, neox_args, init_method, output_layer_init_method, layer_number):
        super().__init__()
        self.layer_number = layer_number
        norm, eps = get_norm(neox_args)
        self.norm = norm(neox_args.hidden_size, eps=eps)
        self.mixer = ParallelMambaBlock(neox_args, init_method, output_layer_init_method)

    def forward(self, x, attention_mask=None, layer_past=None):
        return self.mixer(self.norm(x)) + x


class ParallelMambaResidualLayerPipe(ParallelMambaResidualLayer):
    def forward(self, args):
        assert len(args) == 2, "MambaResidualLayerPipe expects 2 arguments - hidden_states and attention_mask"
        hidden_states, attention_mask = args
        return super().forward(hidden_states, attention_mask), attention_mask
