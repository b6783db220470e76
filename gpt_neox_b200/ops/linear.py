"""Linear layer autograd function on top of the tcgen05 GEMM.

forward   ``y = act(x W^T + b) (+ residual)``           -> one GEMM, bias / GeLU / residual in the epilogue
backward  ``dx = dy W``  and  ``dW = dy^T x``           -> two GEMMs reading the *same* row-major tensors
                                                          (MN-major operand descriptors, no transposes)

When the weight carries a ``main_grad`` attribute (an fp32 view into the engine's contiguous gradient
buffer) the weight-gradient GEMM accumulates straight into it from its epilogue and autograd sees no
``.grad`` for that parameter; this replaces both the separate accumulation kernel and the
bf16 -> fp32 copy of a DeepSpeed-style bf16 optimizer.

On CPU, or for dtypes the kernel does not take, the same math runs through ``torch`` ops.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import gemm as G
from . import flop_count, native


def main_grad_of(param):
    """The fp32 gradient accumulator of ``param`` inside the optimizer's flat buffer, or ``None`` when there is no
    such optimizer.  Under ZeRO stage 2 the buffer is transient: the first request of a micro-batch allocates it."""
    mg = getattr(param, "main_grad", None)
    if mg is None:
        bucket = getattr(param, "_bucket", None)
        if bucket is not None and bucket.partition_grads:
            bucket.ensure_grad_buffer()
            mg = param.main_grad
    return mg


def notify_grad_ready(weight):
    """Tell the optimizer (if it listens) that ``weight.main_grad`` now holds this backward pass' contribution."""
    cb = getattr(weight, "_grad_ready", None)
    if cb is not None:
        cb()


_DEAD = [False]


class dead_outputs:
    """Inside this context the OUTPUT VALUES of linear layers are not needed (only their saved inputs are, for the
    backward pass of a recomputed block): the GEMM -- and the tensor-parallel reduction that follows it -- is skipped
    and an uninitialised tensor of the right shape is returned."""

    def __init__(self, flag=True):
        self.flag = bool(flag)

    def __enter__(self):
        self.old, _DEAD[0] = _DEAD[0], self.flag

    def __exit__(self, *exc):
        _DEAD[0] = self.old
        return False


def output_is_dead() -> bool:
    return _DEAD[0]


_warned = set()


def warn_fallback(what, why):
    """A CUDA tensor that misses the native kernel is a performance bug worth one line in the log (never silent)."""
    key = (what, why)
    if key not in _warned:
        _warned.add(key)
        import warnings
        warnings.warn(f"{what}: CUDA input falls back to the library / eager path ({why})", RuntimeWarning, stacklevel=3)


def kernel_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    if not (x.is_cuda and native.available()):
        return False
    ok = (x.dtype in (torch.bfloat16, torch.float16) and w.dtype == x.dtype
          and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0 and w.is_contiguous())
    if not ok:
        warn_fallback("linear", f"dtypes {x.dtype}/{w.dtype}, shapes {tuple(x.shape)} x {tuple(w.shape)}")
    return ok


class _LinearFn(torch.autograd.Function):
    """``split_pre``: also return the pre-activation (non-differentiable) and expect the incoming gradient to be
    w.r.t. the PRE-activation already.  ``dgelu_aux``: the pre-activation of the layer that produced ``x``; the data
    gradient is multiplied by GeLU'(aux) in the dgrad GEMM's epilogue.  Together they move the GeLU backward of an
    MLP out of a separate element-wise pass and into the second linear's dgrad GEMM."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, act, dgelu_aux=None, split_pre=False):
        ctx.act = act
        ctx.split_pre = split_pre
        ctx.x_shape = x.shape
        # the pre-activation output is not differentiable: without this autograd would hand backward a zero tensor
        # of its size (a full pass over [tokens, 4h]) for it
        ctx.set_materialize_grads(False)
        N, K = weight.shape
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        res2 = residual.reshape(-1, N) if residual is not None else None
        need_pre = act == "gelu" and any(ctx.needs_input_grad[:3])
        use_k = kernel_ok(x2, weight) and (bias is None or bias.dtype == x2.dtype)
        ctx.use_k = use_k
        pre = None
        if _DEAD[0] and act is None and not split_pre:
            out = torch.empty(x2.shape[0], N, dtype=x2.dtype, device=x2.device)
        elif use_k:
            r = G.gemm(x2, weight, bias=bias, add=res2, act=G.ACT_GELU if act == "gelu" else G.ACT_NONE,
                       want_preact=need_pre)
            out, pre = r if need_pre else (r, None)
        else:
            flop_count.gemm(x2.shape[0], N, x2.shape[1])
            out = F.linear(x2, weight, bias)
            if act == "gelu":
                pre = out if need_pre else None
                out = F.gelu(out, approximate="tanh")
            if res2 is not None:
                out = out + res2
        ctx.has_bias = bias is not None
        ctx.bias_ref = bias
        ctx.has_res = residual is not None
        ctx.has_aux = dgelu_aux is not None
        aux2 = dgelu_aux.reshape(-1, K) if dgelu_aux is not None else None
        ctx.save_for_backward(x2, weight, None if split_pre else pre, aux2)
        out = out.reshape(*x.shape[:-1], N)
        if split_pre:
            if pre is not None:
                pre = pre.reshape(*x.shape[:-1], N)
                ctx.mark_non_differentiable(pre)
            return out, pre
        return out

    @staticmethod
    def backward(ctx, g, g_pre=None):
        x2, weight, pre, aux2 = ctx.saved_tensors
        N, K = weight.shape
        if g is None:
            return None, None, None, None, None, None, None
        g_in = g
        g2 = g.reshape(-1, N)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        g_res = g_in if ctx.has_res else None
        if ctx.act == "gelu" and not ctx.split_pre:
            from .functional import dgelu_mul
            g2 = dgelu_mul(g2, pre)
        gx = gw = gb = None
        if ctx.use_k and g2.dtype == x2.dtype:
            if ctx.needs_input_grad[0]:
                if aux2 is not None:
                    gx = G.gemm(g2, weight, a_mn=False, b_mn=True, act=G.ACT_DGELU, aux=aux2).reshape(ctx.x_shape)
                else:
                    gx = G.gemm(g2, weight, a_mn=False, b_mn=True).reshape(ctx.x_shape)
            if ctx.needs_input_grad[1]:
                mg = main_grad_of(weight)
                if mg is not None:
                    G.gemm(g2, x2, a_mn=True, b_mn=True, out=mg, add=mg)
                    weight.grad_in_main = True
                    notify_grad_ready(weight)
                else:
                    gw = G.gemm(g2, x2, a_mn=True, b_mn=True)
        else:
            if ctx.needs_input_grad[0]:
                gx = g2 @ weight
                if aux2 is not None:
                    gx = (gx.float() * G.dgelu_tanh_ref(aux2.float())).to(gx.dtype)
                gx = gx.reshape(ctx.x_shape)
            if ctx.needs_input_grad[1]:
                gw = g2.t() @ x2
                mg = main_grad_of(weight)
                if mg is not None:
                    mg.add_(gw)
                    weight.grad_in_main = True
                    gw = None
                    notify_grad_ready(weight)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from .functional import bias_grad
            gb = bias_grad(g2, ctx.bias_ref)
        return gx, gw, gb, g_res, None, None, None


def linear(x, weight, bias=None, residual=None, act=None, dgelu_aux=None, split_pre=False):
    """``act(x @ weight.T + bias) + residual`` with the epilogue fused into the GEMM (see ``_LinearFn`` for the
    two GeLU-backward options)."""
    return _LinearFn.apply(x, weight, bias, residual, act, dgelu_aux, split_pre)
