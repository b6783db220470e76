"""Normalisation layers (reference ``megatron/model/norms.py:19-107``, ``fused_layer_norm.py:34-262``).

``get_norm(args)`` -> ``(constructor, eps)``.  LayerNorm parameters are ``weight``/``bias``, RMSNorm's
gain is called ``scale`` (checkpoint-visible names).  RMSNorm keeps the reference's non-standard
form ``x / (rms(x) + eps)`` (eps outside the root).  All of them dispatch to the fused sm_100a kernels
on GPU whatever the ``*_fusion`` flags say: the unfused path only exists on CPU.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as OF


class LayerNorm(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5, elementwise_affine=True, bias=True, device=None, dtype=None):
        super().__init__()
        self.dim = normalized_shape if isinstance(normalized_shape, int) else normalized_shape[-1]
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(self.dim, device=device, dtype=dtype))
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.dim, device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        return OF.layer_norm(x, self.weight, self.bias, self.eps)


class RMSNorm(nn.Module):
    def __init__(self, dim, p=-1.0, eps=1e-8, bias=False, device=None, dtype=None):
        super().__init__()
        self.eps, self.d, self.p = eps, dim, p
        self.scale = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        if bias:
            self.offset = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype))
        else:
            self.register_parameter("offset", None)

    def forward(self, x):
        if 0.0 <= self.p <= 1.0:
            # partial RMSNorm: statistics from the first p*d features only
            k = int(self.d * self.p)
            xf = x.float()
            rms = xf[..., :k].norm(2, dim=-1, keepdim=True) * (k ** -0.5)
            y = (xf / (rms + self.eps) * self.scale.float())
            if self.offset is not None:
                y = y + self.offset.float()
            return y.to(x.dtype)
        return OF.rms_norm(x, self.scale, self.offset, self.eps)


class ScaleNorm(nn.Module):
    def __init__(self, dim, eps=1e-5, device=None, dtype=None):
        super().__init__()
        self.g = nn.Parameter(torch.ones(1, device=device, dtype=dtype))
        self.eps = eps

    def forward(self, x):
        n = torch.norm(x.float(), dim=-1, keepdim=True).clamp(min=self.eps)
        return (x.float() / n * self.g.float()).to(x.dtype)


def get_norm(args):
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None
    dt = args.params_dtype
    use_bias = getattr(args, "use_bias_in_norms", True)
    if args.norm in ("rmsnorm", "te_rmsnorm"):
        eps = args.rms_norm_epsilon
        return (lambda dim, eps=eps: RMSNorm(dim, eps=eps, device=dev, dtype=dt)), eps
    if args.norm in ("layernorm", "te_layernorm"):
        eps = args.layernorm_epsilon
        return (lambda dim, eps=eps: LayerNorm(dim, eps=eps, bias=use_bias, device=dev, dtype=dt)), eps
    if args.norm == "scalenorm":
        eps = args.scalenorm_epsilon
        return (lambda dim, eps=eps: ScaleNorm(dim, eps=eps, device=dev, dtype=dt)), eps
    raise ValueError(f"norm {args.norm} not recognized")
