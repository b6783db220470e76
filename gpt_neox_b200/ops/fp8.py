"""Per-tensor-scaled FP8 training on the fp8 tensor cores (``csrc/gemm_fp8_sm100.cu``).

``cast`` turns a bf16 tensor into an ``Fp8Tensor`` (E4M3 or E5M2 bytes + a device-resident inverse scale);
``gemm_fp8`` multiplies two of them with ``tcgen05.mma.kind::f8f6f4`` (fp32 accumulation) and the same fused epilogue
as the bf16 GEMM.  ``fp8_linear`` is the linear layer built from them:

=========  ==================  =============================  ==============================
pass       math                A                              B
=========  ==================  =============================  ==============================
forward    Y  = X W^T          X  e4m3, K-major               W  e4m3, K-major
dgrad      dX = dY W           dY e5m2 (hybrid) / e4m3        W  e4m3, MN-major (same bytes)
wgrad      dW = dY^T X         dY, MN-major (same bytes)      X  e4m3, MN-major (saved fp8)
=========  ==================  =============================  ==============================

Scaling is per tensor, so one quantised copy of each tensor serves every GEMM that reads it (the kernel takes either
storage order) and the activation saved for backward is the fp8 copy, half the bf16 bytes.  Two recipes:

* ``current``: amax pass, then cast with ``scale = fp8_max / (amax * 2^margin)``;
* ``delayed``: cast with a scale derived from a history of earlier amaxes while recording the new one -- the recipe
  Transformer Engine applies in the reference (``megatron/model/transformer_engine.py``; keys
  ``te_fp8_amax_history_len``, ``te_fp8_amax_compute_algo``, ``te_fp8_margin``).

Quantised weights are cached until ``invalidate_weight_cache()`` (the engine calls it after every optimizer step and
checkpoint load) or until the parameter's storage / version changes.

On CPU the same functions evaluate the identical math with torch's float8 dtypes (oracle and CPU test path).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from . import gemm as G
from . import flop_count, native
from .linear import main_grad_of

E4M3_MAX, E5M2_MAX = 448.0, 57344.0


@dataclass
class Fp8Tensor:
    q: torch.Tensor            # uint8, the shape of the source tensor
    inv: torch.Tensor          # float32 [1] on the same device: 1 / scale
    e5m2: bool = False

    def dequant(self):
        dt = torch.float8_e5m2 if self.e5m2 else torch.float8_e4m3fn
        return self.q.view(dt).float() * self.inv


class DelayedMeta:
    """Amax history and scale of one tensor role (layout documented at ``fp8_delayed_update_kernel``)."""

    def __init__(self, device, length=1024, e5m2=False, margin=0, most_recent=False):
        self.len, self.e5m2, self.margin, self.most_recent = int(length), bool(e5m2), int(margin), bool(most_recent)
        self.buf = torch.zeros(4 + self.len, dtype=torch.float32, device=device)

    def update(self):
        if self.buf.is_cuda:
            rc = native.lib().neox_fp8_delayed_update(native.ptr(self.buf), self.len, int(self.e5m2), self.margin,
                                                      int(self.most_recent), ctypes.c_void_p(native.stream_ptr()))
            native.check(rc, "neox_fp8_delayed_update")
            return
        b = self.buf
        pos = int(b[3])
        cur = float(b[2])
        b[4 + pos] = cur
        b[2] = 0.0
        b[3] = (pos + 1) % self.len
        amax = cur if self.most_recent else max(cur, float(b[4:].max()))
        if 0 < amax < 3e38:
            s = (E5M2_MAX if self.e5m2 else E4M3_MAX) / (amax * 2.0 ** self.margin)
            b[0], b[1] = s, 1.0 / s
        elif float(b[0]) == 0.0:
            b[0], b[1] = 1.0, 1.0


def _cast_ref(x, e5m2, margin, meta):
    lim = E5M2_MAX if e5m2 else E4M3_MAX
    xf = x.float()
    amax = xf.abs().max()
    if meta is not None:
        scale = meta.buf[0].clone()
        meta.buf[2] = torch.maximum(meta.buf[2], amax)
    else:
        scale = torch.where((amax > 0) & torch.isfinite(amax), lim / (amax * 2.0 ** margin), torch.ones_like(amax))
    dt = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    q = (xf * scale).clamp(-lim, lim).to(dt).view(torch.uint8)
    return Fp8Tensor(q, (1.0 / scale).reshape(1).float(), e5m2)


def cast(x, e5m2=False, margin=0, meta: DelayedMeta | None = None) -> Fp8Tensor:
    """Quantise a bf16 tensor with one scale for the whole tensor.  With ``meta`` the scale comes from its history
    (call ``meta.update()`` once before) and the tensor's amax is recorded for later steps."""
    if not (x.is_cuda and native.available() and x.dtype == torch.bfloat16):
        return _cast_ref(x, e5m2, margin, meta)
    x = x.contiguous()
    n = x.numel()
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    L = native.lib()
    st = ctypes.c_void_p(native.stream_ptr())
    if meta is not None:
        b = meta.buf
        base = b.data_ptr()
        rc = L.neox_fp8_cast(native.ptr(x), native.ptr(q), ctypes.c_longlong(n), ctypes.c_void_p(base), 0, int(e5m2),
                             0, ctypes.c_void_p(base + 4), ctypes.c_void_p(base + 8), st)
        native.check(rc, "neox_fp8_cast")
        return Fp8Tensor(q, b[1:2].clone(), e5m2)       # the history buffer moves on before backward reads this
    s = torch.zeros(2, dtype=torch.float32, device=x.device)        # [amax, 1/scale]
    native.check(L.neox_fp8_amax(native.ptr(x), ctypes.c_longlong(n), native.ptr(s), st), "neox_fp8_amax")
    rc = L.neox_fp8_cast(native.ptr(x), native.ptr(q), ctypes.c_longlong(n), native.ptr(s), 1, int(e5m2), int(margin),
                         ctypes.c_void_p(s.data_ptr() + 4), None, st)
    native.check(rc, "neox_fp8_cast")
    return Fp8Tensor(q, s[1:2], e5m2)


def gemm_fp8_ref(a: Fp8Tensor, b: Fp8Tensor, a_mn=False, b_mn=False, **kw):
    return G.gemm_ref(a.dequant(), b.dequant(), a_mn, b_mn, **kw)


def gemm_fp8(a: Fp8Tensor, b: Fp8Tensor, a_mn=False, b_mn=False, out=None, out_dtype=torch.bfloat16, bias=None,
             add=None, act=G.ACT_NONE, aux=None, alpha=1.0, want_preact=False):
    """``epilogue(alpha * op(a) @ op(b))`` on fp8 operands; arguments as ``ops.gemm.gemm``."""
    aq, bq = a.q, b.q
    if flop_count.ACTIVE[0] is not None:
        flop_count.gemm(aq.shape[1] if a_mn else aq.shape[0], bq.shape[1] if b_mn else bq.shape[0],
                        aq.shape[0] if a_mn else aq.shape[1])
    if not aq.is_cuda:
        r = gemm_fp8_ref(a, b, a_mn, b_mn, out_dtype=out_dtype if out is None else out.dtype, bias=bias, add=add,
                         act=act, aux=aux, alpha=alpha, want_preact=want_preact)
        if out is not None:
            if want_preact:
                out.copy_(r[0]); return out, r[1]
            out.copy_(r); return out
        return r
    assert aq.dim() == 2 and bq.dim() == 2 and aq.stride(1) == 1 and bq.stride(1) == 1
    K, M = aq.shape if a_mn else aq.shape[::-1]
    Kb, N = bq.shape if b_mn else bq.shape[::-1]
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, device=aq.device, dtype=out_dtype)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    pre = torch.empty(M, N, device=aq.device, dtype=torch.bfloat16) if want_preact else None
    if add is not None:
        assert add.shape == (M, N) and add.stride(1) == 1 and add.dtype in (torch.bfloat16, torch.float32)
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N and bias.is_contiguous()
    if act == G.ACT_DGELU:
        assert aux is not None and aux.shape == (M, N) and aux.dtype == torch.bfloat16 and aux.stride(1) == 1
    L = native.lib()
    rc = (L.neox_gemm_fp8_2cta if G.use_pair_kernel(M, N, K) else L.neox_gemm_fp8)(
        native.ptr(aq), native.ptr(bq), native.ptr(out), M, N, K,
        ctypes.c_longlong(aq.stride(0)), ctypes.c_longlong(bq.stride(0)), ctypes.c_longlong(out.stride(0)),
        int(a_mn), int(b_mn), int(a.e5m2), int(b.e5m2), native.ptr(a.inv), native.ptr(b.inv),
        int(out.dtype == torch.float32),
        native.ptr(bias), native.ptr(add), ctypes.c_longlong(add.stride(0) if add is not None else 0),
        int(add is not None and add.dtype == torch.float32),
        native.ptr(pre), ctypes.c_longlong(pre.stride(0) if pre is not None else 0),
        native.ptr(aux), ctypes.c_longlong(aux.stride(0) if aux is not None else 0),
        int(act), ctypes.c_float(alpha), ctypes.c_void_p(native.stream_ptr()))
    native.check(rc, "neox_gemm_fp8")
    return (out, pre) if want_preact else out


def shapes_ok(tokens, n_out, n_in):
    """TMA wants every row pitch of the byte matrices to be a multiple of 16."""
    return n_out % 16 == 0 and n_in % 16 == 0


# ------------------------------------------------------------------ the linear layer
@dataclass
class Fp8Recipe:
    recipe: str = "current"            # "current" | "delayed"
    hybrid: bool = True                # gradients in E5M2
    fp8_wgrad: bool = True
    margin: int = 0
    history_len: int = 1024
    most_recent: bool = False
    metas: dict = field(default_factory=dict)

    def meta(self, role, device, e5m2):
        if self.recipe != "delayed":
            return None
        m = self.metas.get(role)
        if m is None or m.buf.device != device:
            m = self.metas[role] = DelayedMeta(device, self.history_len, e5m2, self.margin, self.most_recent)
        m.update()
        return m


_weight_epoch = 0
_weight_cache: dict = {}


def invalidate_weight_cache():
    """Call whenever parameters change outside autograd's sight (optimizer step, checkpoint load)."""
    global _weight_epoch
    _weight_epoch += 1
    if len(_weight_cache) > 4096:
        _weight_cache.clear()


def _cast_weight(weight, recipe: Fp8Recipe):
    key = id(weight)
    tag = (_weight_epoch, weight.data_ptr(), weight._version, tuple(weight.shape))
    hit = _weight_cache.get(key)
    if hit is not None and hit[0] == tag:
        return hit[1]
    w = cast(weight.detach(), False, recipe.margin, recipe.meta("w", weight.device, False))
    _weight_cache[key] = (tag, w)
    return w


class _Fp8LinearFn(torch.autograd.Function):
    """``residual``, ``act``, ``dgelu_aux`` and ``split_pre`` mean what they mean in ``ops.linear._LinearFn``: bias,
    GeLU and residual ride in the forward GEMM's epilogue, and the GeLU backward of an MLP rides in the second
    linear's dgrad epilogue."""

    @staticmethod
    def forward(ctx, x, weight, bias, recipe, residual=None, act=None, dgelu_aux=None, split_pre=False):
        N, K = weight.shape
        x2 = x.reshape(-1, K)
        res2 = residual.reshape(-1, N) if residual is not None else None
        xq = cast(x2, False, recipe.margin, recipe.meta("x", x.device, False))
        wq = _cast_weight(weight, recipe)
        need_pre = act == "gelu" and any(ctx.needs_input_grad[:3])
        r = gemm_fp8(xq, wq, bias=bias, add=res2, act=G.ACT_GELU if act == "gelu" else G.ACT_NONE,
                     want_preact=need_pre)
        out, pre = r if need_pre else (r, None)
        aux2 = dgelu_aux.reshape(-1, K) if dgelu_aux is not None else None
        ctx.save_for_backward(xq.q, xq.inv, wq.q, wq.inv, x2 if not recipe.fp8_wgrad else None,
                              None if split_pre else pre, aux2)
        ctx.weight = weight
        ctx.cfg = (x.shape, recipe, bias is not None, residual is not None, act, split_pre)
        out = out.reshape(*x.shape[:-1], N)
        if split_pre:
            if pre is not None:
                pre = pre.reshape(*x.shape[:-1], N)
                ctx.mark_non_differentiable(pre)
            return out, pre
        return out

    @staticmethod
    def backward(ctx, g, g_pre=None):
        xq_q, xq_inv, wq_q, wq_inv, x2, pre, aux2 = ctx.saved_tensors
        x_shape, recipe, has_bias, has_res, act, split_pre = ctx.cfg
        weight = ctx.weight
        N, K = weight.shape
        g_res = g if has_res else None
        g2 = g.reshape(-1, N).contiguous()
        if act == "gelu" and not split_pre:
            from .functional import dgelu_mul
            g2 = dgelu_mul(g2, pre)
        e5 = recipe.hybrid
        gq = cast(g2, e5, recipe.margin, recipe.meta("g", g.device, e5))
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            wq = Fp8Tensor(wq_q, wq_inv, False)
            if aux2 is not None:
                gx = gemm_fp8(gq, wq, a_mn=False, b_mn=True, act=G.ACT_DGELU, aux=aux2).reshape(x_shape)
            else:
                gx = gemm_fp8(gq, wq, a_mn=False, b_mn=True).reshape(x_shape)
        if ctx.needs_input_grad[1]:
            mg = main_grad_of(weight)
            if recipe.fp8_wgrad:
                xa = Fp8Tensor(xq_q, xq_inv, False)
                run = lambda **kw: gemm_fp8(gq, xa, a_mn=True, b_mn=True, **kw)
            else:
                run = lambda **kw: G.gemm(g2, x2, a_mn=True, b_mn=True, **kw)
            if mg is not None:
                run(out=mg, add=mg)
                weight.grad_in_main = True
                from .linear import notify_grad_ready
                notify_grad_ready(weight)
            else:
                gw = run()
        if has_bias and ctx.needs_input_grad[2]:
            gb = g2.sum(0)
        return gx, gw, gb, None, g_res, None, None, None


def fp8_linear(x, weight, bias=None, recipe: Fp8Recipe | None = None, residual=None, act=None, dgelu_aux=None,
               split_pre=False):
    """``act(x @ weight.T + bias) + residual`` with the three GEMMs of the layer on the fp8 tensor cores."""
    return _Fp8LinearFn.apply(x, weight, bias, recipe or Fp8Recipe(), residual, act, dgelu_aux, split_pre)
