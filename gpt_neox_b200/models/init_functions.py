"""Weight initialisers selectable by config name (reference ``megatron/model/init_functions.py:25-227``).

``get_init_methods(args)`` returns ``(init_method, output_layer_init_method)``.  Formulas:
normal N(0, s); scaled_normal N(0, s/sqrt(2L)); orthogonal (gain 1) and scaled_orthogonal (gain
1/sqrt(2L)); xavier_uniform / xavier_normal; small_init N(0, sqrt(2/(5d))) (Nguyen & Salazar 2019);
wang_init N(0, 2/(L sqrt(d))); single_residual_scaled_normal N(0, s/sqrt(L)).  With muP enabled the
std of matrix-like parameters is divided by sqrt(width_mult) at (re)initialisation.
"""
from __future__ import annotations

import math

import torch


def _mup_scale(tensor, use_mup, mup_init_scale):
    if use_mup:
        mult = getattr(tensor, "mup_width_mult", None)
        if mult is None and hasattr(tensor, "infshape"):
            mult = tensor.infshape.width_mult()
        with torch.no_grad():
            tensor.mul_(mup_init_scale)
            if mult:
                tensor.div_(math.sqrt(mult))
    return tensor


def _normal(std, use_mup_outer=False, mup_init_scale=1.0):
    def init_(tensor, use_mup=use_mup_outer):
        torch.nn.init.normal_(tensor, mean=0.0, std=std)
        return _mup_scale(tensor, use_mup, mup_init_scale)
    return init_


def init_method_normal(sigma, use_mup_outer=False, mup_init_scale=1.0):
    return _normal(sigma, use_mup_outer, mup_init_scale)


def scaled_init_method_normal(sigma, num_layers, use_mup_outer=False, mup_init_scale=1.0, num_residuals_per_layer=2):
    return _normal(sigma / math.sqrt(num_residuals_per_layer * num_layers), use_mup_outer, mup_init_scale)


def _orthogonal(tensor, gain=1.0):
    """QR-based orthogonal init done in fp32 (QR has no half-precision kernel)."""
    if tensor.ndimension() < 2:
        raise ValueError("Only tensors with 2 or more dimensions are supported")
    rows, cols = tensor.size(0), tensor.numel() // tensor.size(0)
    flat = torch.empty(rows, cols, dtype=torch.float32).normal_(0, 1)
    if rows < cols:
        flat.t_()
    q, r = torch.linalg.qr(flat)
    q *= torch.diag(r, 0).sign()
    if rows < cols:
        q.t_()
    with torch.no_grad():
        tensor.view_as(q).copy_(q.to(tensor.dtype))
        tensor.mul_(gain)
    return tensor


def orthogonal_init_method(n_layers=1, use_mup=False, mup_init_scale=1.0):
    if use_mup:
        raise ValueError("Orthogonal init needs to be patched to support mup. Disable mup or use a different init")
    return lambda t: _orthogonal(t, math.sqrt(2 / n_layers))


def xavier_uniform_init_method(use_mup_outer=False, mup_init_scale=1.0):
    def init_(tensor, use_mup=use_mup_outer):
        torch.nn.init.xavier_uniform_(tensor)
        return _mup_scale(tensor, use_mup, mup_init_scale)
    return init_


def xavier_normal_init_method(use_mup_outer=False, mup_init_scale=1.0):
    def init_(tensor, use_mup=use_mup_outer):
        torch.nn.init.xavier_normal_(tensor)
        return _mup_scale(tensor, use_mup, mup_init_scale)
    return init_


def small_init_init_method(dim, use_mup_outer=False, mup_init_scale=1.0):
    return _normal(math.sqrt(2 / (5 * dim)), use_mup_outer, mup_init_scale)


def wang_init_method(n_layers, dim, use_mup_outer=False, mup_init_scale=1.0):
    return _normal(2 / n_layers / math.sqrt(dim), use_mup_outer, mup_init_scale)


def get_init_methods(args):
    if getattr(args, "use_mup", False):
        use_mup, scale = True, args.mup_init_scale
    else:
        use_mup, scale = False, 1.0

    def pick(name):
        if name == "normal":
            return init_method_normal(args.init_method_std, use_mup, scale)
        if name == "scaled_normal":
            return scaled_init_method_normal(args.init_method_std, args.num_layers, use_mup, scale)
        if name == "orthogonal":
            return orthogonal_init_method(use_mup=use_mup, mup_init_scale=scale)
        if name == "scaled_orthogonal":
            return orthogonal_init_method(args.num_layers, use_mup, scale)
        if name == "xavier_uniform":
            return xavier_uniform_init_method(use_mup, scale)
        if name == "xavier_normal":
            return xavier_normal_init_method(use_mup, scale)
        if name == "wang_init":
            return wang_init_method(args.num_layers, args.hidden_size, use_mup, scale)
        if name == "small_init":
            return small_init_init_method(args.hidden_size, use_mup, scale)
        if name == "single_residual_scaled_normal":
            return scaled_init_method_normal(args.init_method_std, args.num_layers, use_mup, scale,
                                             num_residuals_per_layer=1)
        raise NotImplementedError(f"Unknown init method {name}")

    return pick(args.init_method), pick(args.output_layer_init_method)
