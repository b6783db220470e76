"""Fused element-wise, normalisation, softmax, rotary and loss operators.

Every operator has two bodies that compute the same math:

* ``*_ref``  -- plain PyTorch (fp32 internally).  It is the CPU path and the oracle of the GPU tests.
* the CUDA kernel in ``csrc/`` reached through ctypes, used whenever the input lives on a GPU and
  has a supported dtype.  There is no silent fallback on a GPU for supported dtypes: if the library
  cannot be loaded the call raises.

Reference call sites these replace: apex/TorchScript fused ops in ``megatron/model/fused_layer_norm.py``,
``norms.py``, ``activations.py:78-112``, ``fused_bias_dropout.py:28-55``, ``fused_softmax.py:24-205``,
``fused_rope.py`` and ``megatron/mpu/cross_entropy.py:27-117``.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.nn.functional as F

from . import native

_DT = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}


def _k(*ts) -> bool:
    """Kernel path usable for these tensors?"""
    t0 = ts[0]
    return t0.is_cuda and native.available() and t0.dtype in _DT


def _s():
    return ctypes.c_void_p(native.stream_ptr())


_workspaces = {}


def workspace(nbytes: int, device, tag="ws") -> torch.Tensor:
    """A cached per-device scratch buffer of at least ``nbytes`` (grown geometrically, never shrunk)."""
    key = (device, tag)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _param_grad(param, g32):
    """Hand an fp32 parameter gradient to the optimizer: added to ``param.main_grad`` (the flat fp32 gradient buffer)
    when it exists -- no round trip through the 16-bit ``.grad`` and its accumulate hook -- else returned in the
    parameter's type."""
    if param is None:
        return None
    from .linear import main_grad_of
    mg = main_grad_of(param)
    if mg is not None and mg.dtype == torch.float32 and mg.shape == g32.shape:
        mg.add_(g32)
        param.grad_in_main = True
        ready = getattr(param, "_grad_ready", None)
        if ready is not None:
            ready()
        return None
    return g32.to(param.dtype)


# ------------------------------------------------------------------------------------ LayerNorm
def layer_norm_ref(x, weight, bias, eps):
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = xf.var(-1, unbiased=False, keepdim=True)
    y = (xf - mean) * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        cols = x.shape[-1]
        x2 = x.reshape(-1, cols)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = native.lib().neox_layernorm_fwd(native.ptr(x2), native.ptr(weight), native.ptr(bias), native.ptr(y),
                                             native.ptr(mean), native.ptr(rstd), rows, cols, ctypes.c_float(eps),
                                             _DT[x.dtype], _s())
        native.check(rc, "neox_layernorm_fwd")
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.has_bias = bias is not None
        ctx.bias_ref = bias
        ctx.shape = x.shape
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, g):
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, cols = x2.shape
        g2 = g.reshape(rows, cols)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        dx = torch.empty_like(x2)
        nblk = int(native.lib().neox_norm_bwd_blocks(rows))
        ws = workspace(2 * nblk * cols * 4, x2.device, "ln_bwd")
        dgamma = torch.empty(cols, dtype=torch.float32, device=x2.device)
        dbeta = torch.empty(cols, dtype=torch.float32, device=x2.device)
        rc = native.lib().neox_layernorm_bwd(native.ptr(g2), native.ptr(x2), native.ptr(weight), native.ptr(mean),
                                             native.ptr(rstd), native.ptr(dx), native.ptr(dgamma), native.ptr(dbeta),
                                             native.ptr(ws), rows, cols, _DT[x2.dtype], _s())
        native.check(rc, "neox_layernorm_bwd")
        return (dx.reshape(ctx.shape), _param_grad(weight, dgamma) if ctx.needs_input_grad[1] else None,
                _param_grad(ctx.bias_ref, dbeta) if ctx.has_bias and ctx.needs_input_grad[2] else None, None)


def layer_norm(x, weight, bias, eps=1e-5):
    if _k(x) and weight is not None and weight.dtype == x.dtype and x.shape[-1] % 8 == 0:
        return _LayerNormFn.apply(x, weight, bias, eps)
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


# ------------------------------------------------------------------------------------ RMSNorm
def rms_norm_ref(x, scale, bias, eps):
    """``x / (||x||_2 * d^-1/2 + eps) * scale (+ bias)``: eps is added to the RMS, not under the root
    (reference ``megatron/model/norms.py:81-96``)."""
    xf = x.float()
    rms = xf.norm(2, dim=-1, keepdim=True) * (x.shape[-1] ** -0.5)
    y = xf / (rms + eps) * scale.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, bias, eps):
        cols = x.shape[-1]
        x2 = x.reshape(-1, cols)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rinv = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = native.lib().neox_rmsnorm_fwd(native.ptr(x2), native.ptr(scale), native.ptr(bias), native.ptr(y),
                                           native.ptr(rinv), rows, cols, ctypes.c_float(eps), _DT[x.dtype], _s())
        native.check(rc, "neox_rmsnorm_fwd")
        ctx.save_for_backward(x2, scale, rinv)
        ctx.has_bias = bias is not None
        ctx.bias_ref = bias
        ctx.eps = eps
        ctx.shape = x.shape
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, g):
        x2, scale, rinv = ctx.saved_tensors
        rows, cols = x2.shape
        g2 = g.reshape(rows, cols)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        dx = torch.empty_like(x2)
        nblk = int(native.lib().neox_norm_bwd_blocks(rows))
        ws = workspace(2 * nblk * cols * 4, x2.device, "ln_bwd")
        dscale = torch.empty(cols, dtype=torch.float32, device=x2.device)
        dbias = torch.empty(cols, dtype=torch.float32, device=x2.device)
        rc = native.lib().neox_rmsnorm_bwd(native.ptr(g2), native.ptr(x2), native.ptr(scale), native.ptr(rinv),
                                           native.ptr(dx), native.ptr(dscale), native.ptr(dbias), native.ptr(ws),
                                           rows, cols, ctypes.c_float(ctx.eps), _DT[x2.dtype], _s())
        native.check(rc, "neox_rmsnorm_bwd")
        return (dx.reshape(ctx.shape), _param_grad(scale, dscale) if ctx.needs_input_grad[1] else None,
                _param_grad(ctx.bias_ref, dbias) if ctx.has_bias and ctx.needs_input_grad[2] else None, None)


def rms_norm(x, scale, bias=None, eps=1e-8):
    if _k(x) and scale.dtype == x.dtype and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, scale, bias, eps)
    return rms_norm_ref(x, scale, bias, eps)


# ------------------------------------------------------------------------------------ activations
def gelu_ref(x):
    return F.gelu(x.float(), approximate="tanh").to(x.dtype)


def _dgelu(xf):
    k0, k1 = 0.7978845608028654, 0.044715
    t = torch.tanh(k0 * xf * (1 + k1 * xf * xf))
    return 0.5 * xf * ((1 - t * t) * (k0 + 3 * k0 * k1 * xf * xf)) + 0.5 * (1 + t)


def dgelu_mul(g, pre):
    """``g * gelu'(pre)`` (tanh approximation)."""
    if _k(g) and g.dtype == pre.dtype and g.is_contiguous() and pre.is_contiguous():
        out = torch.empty_like(g)
        rc = native.lib().neox_dgelu_mul(native.ptr(g), native.ptr(pre), native.ptr(out),
                                         ctypes.c_longlong(g.numel()), _DT[g.dtype], _s())
        native.check(rc, "neox_dgelu_mul")
        return out
    return (g.float() * _dgelu(pre.float())).to(g.dtype)


class _BiasGeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        x2 = x.contiguous()
        out = torch.empty_like(x2)
        cols = x.shape[-1]
        rc = native.lib().neox_bias_gelu_fwd(native.ptr(x2), native.ptr(bias), native.ptr(out),
                                             ctypes.c_longlong(x2.numel() // cols), cols, _DT[x.dtype], _s())
        native.check(rc, "neox_bias_gelu_fwd")
        ctx.save_for_backward(x2, bias)
        return out

    @staticmethod
    def backward(ctx, g):
        x2, bias = ctx.saved_tensors
        cols = x2.shape[-1]
        g2 = g.contiguous()
        dx = torch.empty_like(x2)
        rc = native.lib().neox_bias_gelu_bwd(native.ptr(g2), native.ptr(x2), native.ptr(bias), native.ptr(dx),
                                             ctypes.c_longlong(x2.numel() // cols), cols, _DT[x2.dtype], _s())
        native.check(rc, "neox_bias_gelu_bwd")
        db = dx.reshape(-1, cols).sum(0) if bias is not None else None
        return dx, db


def bias_gelu(x, bias=None):
    """``gelu(x + bias)`` with the tanh approximation (reference ``activations.py:78-112``)."""
    if _k(x) and x.shape[-1] % 8 == 0 and (bias is None or bias.dtype == x.dtype):
        return _BiasGeluFn.apply(x, bias)
    y = x if bias is None else x + bias
    return F.gelu(y, approximate="tanh")


_GATED = {"geglu": 0, "swiglu": 1, "reglu": 2, "bilinear": 3, "glu": 4}


def _gate_fn(kind, gate):
    return {"geglu": lambda t: F.gelu(t, approximate="tanh"), "swiglu": F.silu, "reglu": F.relu,
            "bilinear": lambda t: t, "glu": torch.sigmoid}[kind](gate)


def gated_act_ref(x, kind, bias=None):
    """``x, gate = chunk(2); out = act(gate) * x`` (reference ``transformer.py:190-206``)."""
    if bias is not None:
        x = x + bias
    a, gate = x.float().chunk(2, dim=-1)
    return (_gate_fn(kind, gate) * a).to(x.dtype)


class _GatedActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kind):
        x2 = x.contiguous()
        cols = x.shape[-1] // 2
        rows = x2.numel() // (2 * cols)
        out = torch.empty(*x.shape[:-1], cols, dtype=x.dtype, device=x.device)
        rc = native.lib().neox_gated_act_fwd(native.ptr(x2), native.ptr(out), ctypes.c_longlong(rows), cols,
                                             _GATED[kind], _DT[x.dtype], _s())
        native.check(rc, "neox_gated_act_fwd")
        ctx.save_for_backward(x2)
        ctx.kind = kind
        return out

    @staticmethod
    def backward(ctx, g):
        (x2,) = ctx.saved_tensors
        cols = x2.shape[-1] // 2
        rows = x2.numel() // (2 * cols)
        g2 = g.contiguous()
        dx = torch.empty_like(x2)
        rc = native.lib().neox_gated_act_bwd(native.ptr(g2), native.ptr(x2), native.ptr(dx), ctypes.c_longlong(rows),
                                             cols, _GATED[ctx.kind], _DT[x2.dtype], _s())
        native.check(rc, "neox_gated_act_bwd")
        return dx, None


def gated_act(x, kind, bias=None):
    if bias is not None:
        x = x + bias
    if _k(x) and (x.shape[-1] // 2) % 8 == 0:
        return _GatedActFn.apply(x, kind)
    return gated_act_ref(x, kind)


def get_activation(name):
    """Non-gated activations by config name (reference ``activations.py:27-66``)."""
    table = {
        "gelu": lambda x: F.gelu(x, approximate="tanh"),
        "relu": F.relu,
        "softsign": F.softsign,
        "swish": F.silu,
        "silu": F.silu,
        "mish": F.mish,
    }
    if name not in table:
        raise ValueError(f"Activation function {name} not recognized")
    return table[name]


# ------------------------------------------------------------------------------------ bias + dropout + add
def bias_dropout_add(x, bias, residual, prob, training):
    """``residual + dropout(x + bias)`` (reference ``fused_bias_dropout.py:28-55``)."""
    if prob == 0.0 or not training:
        if _k(x) and x.is_contiguous() and residual.is_contiguous() and x.dtype == residual.dtype \
                and not (torch.is_grad_enabled() and (x.requires_grad or residual.requires_grad)) \
                and x.shape[-1] % 8 == 0 and (bias is None or bias.dtype == x.dtype):
            out = torch.empty_like(x)
            cols = x.shape[-1]
            rc = native.lib().neox_bias_residual_add(native.ptr(x), native.ptr(bias), native.ptr(residual),
                                                     native.ptr(out), ctypes.c_longlong(x.numel() // cols), cols,
                                                     _DT[x.dtype], _s())
            native.check(rc, "neox_bias_residual_add")
            return out
        if bias is not None:
            x = x + bias
        return residual + x
    if _k(x) and x.is_contiguous() and residual.is_contiguous() and x.dtype == residual.dtype \
            and x.shape[-1] % 8 == 0 and (bias is None or bias.dtype == x.dtype) and 0.0 < prob < 1.0:
        return _BiasDropoutAdd.apply(x, bias, residual, float(prob))
    if bias is not None:
        x = x + bias
    return residual + F.dropout(x, p=prob, training=training)


def philox_mask_ref(n, p, seed, offset, device="cpu"):
    """The keep-mask the dropout kernels generate for ``n`` elements (n % 8 == 0): Philox-4x32-10 with key = seed,
    counter = offset + 2 * (i // 8) + (i % 8) // 4, element kept when its 32 random bits >= p * 2^32.  Pure torch
    (int64 arithmetic), used by the tests."""
    idx = torch.arange(n // 4, dtype=torch.int64, device=device)         # one counter per 4 elements
    ctr = offset + idx
    M32 = 0xFFFFFFFF
    c = [ctr & M32, (ctr >> 32) & M32, torch.zeros_like(ctr), torch.zeros_like(ctr)]
    k0, k1 = seed & M32, (seed >> 32) & M32

    def mulhilo(a, b):
        # 32 x 32 -> 64-bit product without overflowing int64: split b into 16-bit halves
        lo16, hi16 = b & 0xFFFF, b >> 16
        p0 = a * lo16                       # < 2^48
        p1 = a * hi16                       # < 2^48
        lo = (p0 + ((p1 & 0xFFFF) << 16))
        carry = lo >> 32
        hi = (p1 >> 16) + carry
        return hi & M32, lo & M32
    for _ in range(10):
        hi0, lo0 = mulhilo(torch.full_like(ctr, 0xD2511F53), c[0])
        hi1, lo1 = mulhilo(torch.full_like(ctr, 0xCD9E8D57), c[2])
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
        k0, k1 = (k0 + 0x9E3779B9) & M32, (k1 + 0xBB67AE85) & M32
    r = torch.stack(c, dim=1).reshape(-1)
    thr = min(4294967295, int(p * 4294967296.0))
    return r >= thr


class _BiasDropoutAdd(torch.autograd.Function):
    """``residual + dropout(x + bias)`` in one pass; the mask is regenerated in backward from the Philox (seed, offset)
    taken from the device's default generator -- host-side reads only, replayed by activation checkpointing and
    distinct per tensor-parallel rank inside the model-parallel RNG fork."""

    @staticmethod
    def forward(ctx, x, bias, residual, p):
        gen = torch.cuda.default_generators[x.device.index if x.device.index is not None else torch.cuda.current_device()]
        seed, offset = gen.initial_seed(), gen.get_offset()
        cols = x.shape[-1]
        n = x.numel()
        gen.set_offset(offset + ((n // 4 + 3) // 4) * 4)       # one counter value per four elements
        out = torch.empty_like(x)
        rc = native.lib().neox_bias_dropout_add_fwd(native.ptr(x), native.ptr(bias), native.ptr(residual),
                                                    native.ptr(out), ctypes.c_longlong(n // cols), cols,
                                                    ctypes.c_float(p), ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
                                                    ctypes.c_ulonglong(offset), _DT[x.dtype], _s())
        native.check(rc, "neox_bias_dropout_add_fwd")
        ctx.cfg = (p, seed & (2 ** 64 - 1), offset, bias is not None, cols)
        return out

    @staticmethod
    def backward(ctx, g):
        p, seed, offset, has_bias, cols = ctx.cfg
        g = g.contiguous()
        dx = torch.empty_like(g)
        rc = native.lib().neox_dropout_bwd(native.ptr(g), native.ptr(dx), ctypes.c_longlong(g.numel()),
                                           ctypes.c_float(p), ctypes.c_ulonglong(seed), ctypes.c_ulonglong(offset),
                                           _DT[g.dtype], _s())
        native.check(rc, "neox_dropout_bwd")
        gb = dx.reshape(-1, cols).sum(0) if has_bias and ctx.needs_input_grad[1] else None
        return dx, gb, g, None




# ------------------------------------------------------------------------------------ norms + residual fan-out
class _NormFanOutFn(torch.autograd.Function):
    """``x -> (norm_1(x), ..., norm_n(x), x)``: the head of a residual block, where the block input feeds one or two
    norms and the residual connection.  Autograd would add the n + 1 gradient contributions of ``x`` with separate
    element-wise passes (a clone and an add per contribution, each a full pass over the activations); here every norm
    backward kernel adds what has been accumulated so far while it writes ``dx`` (``neox_*norm_bwd_add``), so the
    sum costs no pass of its own.  ``specs``: tuple of ``("ln" | "rms", eps)`` per norm; parameters follow as
    ``weight_1, bias_1, ..., weight_n, bias_n``."""

    @staticmethod
    def forward(ctx, x, specs, *params):
        cols = x.shape[-1]
        x2 = x.reshape(-1, cols)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        L = native.lib()
        outs, stats = [], []
        for i, (kind, eps) in enumerate(specs):
            w, b = params[2 * i], params[2 * i + 1]
            y = torch.empty_like(x2)
            s1 = torch.empty(rows, dtype=torch.float32, device=x.device)
            if kind == "ln":
                s0 = torch.empty(rows, dtype=torch.float32, device=x.device)
                rc = L.neox_layernorm_fwd(native.ptr(x2), native.ptr(w), native.ptr(b), native.ptr(y), native.ptr(s0),
                                          native.ptr(s1), rows, cols, ctypes.c_float(eps), _DT[x.dtype], _s())
            else:
                s0 = None
                rc = L.neox_rmsnorm_fwd(native.ptr(x2), native.ptr(w), native.ptr(b), native.ptr(y), native.ptr(s1),
                                        rows, cols, ctypes.c_float(eps), _DT[x.dtype], _s())
            native.check(rc, "norm forward")
            outs.append(y.reshape(x.shape))
            stats += [s0 if s0 is not None else s1, s1]
        ctx.specs, ctx.shape, ctx.params = specs, x.shape, params
        ctx.save_for_backward(x2, *stats)
        ctx.set_materialize_grads(False)
        return (*outs, x.view_as(x))

    @staticmethod
    def backward(ctx, *grads):
        x2, *stats = ctx.saved_tensors
        rows, cols = x2.shape
        L = native.lib()
        acc = grads[-1]                                   # gradient arriving through the residual connection
        if acc is not None:
            acc = acc.reshape(rows, cols)
            if not acc.is_contiguous():
                acc = acc.contiguous()
        dx = None
        pgrads = []
        nblk = int(L.neox_norm_bwd_blocks(rows))
        for i, (kind, eps) in enumerate(ctx.specs):
            w, b = ctx.params[2 * i], ctx.params[2 * i + 1]
            g = grads[i]
            if g is None:
                pgrads += [None, None]
                continue
            g2 = g.reshape(rows, cols)
            if not g2.is_contiguous():
                g2 = g2.contiguous()
            if dx is None:
                dx = torch.empty_like(x2)
            ws = workspace(2 * nblk * cols * 4, x2.device, "ln_bwd")
            d0 = torch.empty(cols, dtype=torch.float32, device=x2.device)
            d1 = torch.empty(cols, dtype=torch.float32, device=x2.device)
            if kind == "ln":
                rc = L.neox_layernorm_bwd_add(native.ptr(g2), native.ptr(x2), native.ptr(w), native.ptr(stats[2 * i]),
                                              native.ptr(stats[2 * i + 1]), native.ptr(dx), native.ptr(d0),
                                              native.ptr(d1), native.ptr(ws), rows, cols, _DT[x2.dtype],
                                              native.ptr(acc), _s())
            else:
                rc = L.neox_rmsnorm_bwd_add(native.ptr(g2), native.ptr(x2), native.ptr(w), native.ptr(stats[2 * i + 1]),
                                            native.ptr(dx), native.ptr(d0), native.ptr(d1), native.ptr(ws), rows, cols,
                                            ctypes.c_float(eps), _DT[x2.dtype], native.ptr(acc), _s())
            native.check(rc, "norm backward")
            acc = dx
            pgrads.append(_param_grad(w, d0) if ctx.needs_input_grad[2 + 2 * i] else None)
            pgrads.append(_param_grad(b, d1) if b is not None and ctx.needs_input_grad[3 + 2 * i] else None)
        gx = acc.reshape(ctx.shape) if acc is not None else None
        return (gx, None, *pgrads)


def norm_fan_out(x, norms):
    """``(norm_1(x), ..., norm_n(x), x_for_the_residual)`` for ``norms`` = modules with ``weight``/``bias``/``eps``
    (LayerNorm) or ``scale``/``offset``/``eps`` (RMSNorm).  One fused autograd node on a GPU (see
    ``_NormFanOutFn``); plain calls otherwise."""
    specs, params = [], []
    ok = (_k(x) and x.shape[-1] % 8 == 0 and torch.is_grad_enabled() and x.requires_grad
          and os.environ.get("NEOX_NORM_FANOUT", "1") != "0")
    for m in norms:
        if hasattr(m, "scale") and not hasattr(m, "weight"):
            kind, w, b = "rms", m.scale, getattr(m, "offset", None)
            ok = ok and not (0.0 <= getattr(m, "p", -1.0) <= 1.0)
        elif hasattr(m, "weight") and hasattr(m, "eps") and hasattr(m, "dim"):
            kind, w, b = "ln", m.weight, m.bias
        else:
            ok = False
            break
        ok = ok and w.dtype == x.dtype and (b is None or b.dtype == x.dtype)
        specs.append((kind, float(m.eps)))
        params += [w, b]
    if not ok:
        return (*[m(x) for m in norms], x)
    return _NormFanOutFn.apply(x, tuple(specs), *params)

# ------------------------------------------------------------------------------------ bias gradient
def bias_grad(g2, bias=None):
    """Column sums of ``g2`` ([rows, cols]): the gradient of a bias added to every row.  On a GPU one two-pass kernel
    (fixed summation order) that accumulates straight into ``bias.main_grad`` when the optimizer provides that fp32
    buffer -- then ``None`` is returned and the parameter is reported ready, as the weight-gradient GEMMs do."""
    cols = g2.shape[-1]
    if (_k(g2) and g2.dtype in (torch.bfloat16, torch.float16) and g2.dim() == 2 and g2.stride(1) == 1
            and cols % 8 == 0 and g2.stride(0) % 8 == 0 and g2.data_ptr() % 16 == 0):
        L = native.lib()
        rows = g2.shape[0]
        nblk = L.neox_colsum_blocks(ctypes.c_longlong(rows))
        ws = workspace(nblk * cols * 4, g2.device, "colsum")
        from .linear import main_grad_of
        mg = main_grad_of(bias) if bias is not None else None
        into_main = mg is not None and mg.dtype == torch.float32 and mg.is_contiguous()
        out = mg if into_main else torch.empty(cols, dtype=g2.dtype, device=g2.device)
        rc = L.neox_colsum(native.ptr(g2), native.ptr(out), native.ptr(ws), ctypes.c_longlong(rows), cols,
                           ctypes.c_longlong(g2.stride(0)), _DT[g2.dtype], 1 if into_main else _DT[g2.dtype],
                           int(into_main), _s())
        native.check(rc, "neox_colsum")
        if into_main:
            bias.grad_in_main = True
            ready = getattr(bias, "_grad_ready", None)
            if ready is not None:
                ready()
            return None
        return out
    return g2.sum(0)

# ------------------------------------------------------------------------------------ softmax
def scaled_masked_softmax_ref(x, mask, scale, fill=-10000.0):
    """softmax(mask ? fill : x*scale) over the last dim; ``mask`` is True/1 where attention is NOT allowed."""
    xf = x.float() * scale
    if mask is not None:
        xf = xf.masked_fill(mask.bool(), fill)
    return torch.softmax(xf, dim=-1).to(x.dtype)


def scaled_causal_softmax_ref(x, scale):
    """Causal softmax over square [..., s, s] scores; entries above the diagonal are exactly 0."""
    s = x.shape[-1]
    xf = x.float() * scale
    m = torch.ones(s, s, dtype=torch.bool, device=x.device).triu(1)
    xf = xf.masked_fill(m, float("-inf"))
    return torch.softmax(xf, dim=-1).to(x.dtype)


class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, scale, causal):
        x2 = x.contiguous()
        sk = x.shape[-1]
        sq = x.shape[-2]
        rows = x2.numel() // sk
        y = torch.empty_like(x2)
        mask_rows_mod = 0
        mptr = None
        if mask is not None:
            m = mask.to(torch.uint8).contiguous()
            # mask is [b or 1, 1, sq, sk]; heads share it
            assert m.dim() == 4 and m.shape[1] == 1 and m.shape[-1] == sk and m.shape[-2] == sq
            ctx.mask_keep = m
            mptr = native.ptr(m)
            mask_rows_mod = m.shape[0]
        heads = x.shape[1] if x.dim() == 4 else 1
        rc = native.lib().neox_softmax_fwd(native.ptr(x2), mptr, native.ptr(y), ctypes.c_longlong(rows), sq, sk,
                                           heads, mask_rows_mod, ctypes.c_float(scale), int(causal), _DT[x.dtype],
                                           _s())
        native.check(rc, "neox_softmax_fwd")
        ctx.save_for_backward(y)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        g2 = g.contiguous()
        sk = y.shape[-1]
        dx = torch.empty_like(y)
        rc = native.lib().neox_softmax_bwd(native.ptr(g2), native.ptr(y), native.ptr(dx),
                                           ctypes.c_longlong(y.numel() // sk), sk, ctypes.c_float(ctx.scale),
                                           _DT[y.dtype], _s())
        native.check(rc, "neox_softmax_bwd")
        return dx, None, None, None


def scaled_masked_softmax(x, mask, scale):
    """x: [b, np, sq, sk]; mask: [b|1, 1, sq, sk] (nonzero = masked).  Any sk (reference kernel: sk <= 2048)."""
    if _k(x):
        return _SoftmaxFn.apply(x, mask, scale, False)
    return scaled_masked_softmax_ref(x, mask, scale)


def scaled_upper_triang_masked_softmax(x, scale):
    """x: [attn_batches, s, s] causal softmax."""
    if _k(x):
        return _SoftmaxFn.apply(x, None, scale, True)
    return scaled_causal_softmax_ref(x, scale)


# ------------------------------------------------------------------------------------ rotary
def rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope_ref(x, cos, sin):
    """x: [s, b, h, d]; cos/sin: [s, 1, 1, rot]; rotates the first ``rot`` dims of every head."""
    rot = cos.shape[-1]
    xr, xp = x[..., :rot], x[..., rot:]
    xr = (xr.float() * cos.float() + rotate_half(xr.float()) * sin.float()).to(x.dtype)
    return torch.cat((xr, xp), dim=-1) if xp.shape[-1] else xr


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, inverse):
        s, b, h, d = x.shape
        rot = cos.shape[-1]
        xs = x if x.stride(-1) == 1 else x.contiguous()
        out = torch.empty((s, b, h, d), dtype=x.dtype, device=x.device)
        c = cos.reshape(-1, rot)[:s].float().contiguous()
        sn = sin.reshape(-1, rot)[:s].float().contiguous()
        rc = native.lib().neox_rope(native.ptr(xs), native.ptr(out), native.ptr(c), native.ptr(sn), s, b, h, d, rot,
                                    ctypes.c_longlong(xs.stride(0)), ctypes.c_longlong(xs.stride(1)),
                                    ctypes.c_longlong(xs.stride(2)), int(inverse), _DT[x.dtype], _s())
        native.check(rc, "neox_rope")
        ctx.save_for_backward(c, sn)
        ctx.inverse = inverse
        ctx.rot = rot
        return out

    @staticmethod
    def backward(ctx, g):
        c, sn = ctx.saved_tensors
        return _RopeFn.apply(g, c.reshape(-1, 1, 1, ctx.rot), sn.reshape(-1, 1, 1, ctx.rot), not ctx.inverse), None, None, None


def rope(x, cos, sin):
    """Apply (partial) rotary position embedding to [s, b, h, d]; strided inputs are read in place."""
    if _k(x):
        return _RopeFn.apply(x, cos, sin, False)
    return rope_ref(x, cos, sin)


# ------------------------------------------------------------------------------------ cross entropy
def cross_entropy_ref(logits, target):
    """Per-token CE on fp32-cast logits: [..., V], [...] -> [...]."""
    return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), target.reshape(-1),
                           reduction="none").reshape(target.shape)
