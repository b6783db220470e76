"""Adam with block-wise 8-bit optimizer states (what ``use_bnb_optimizer`` selects; the reference delegates to
bitsandbytes' ``Adam8bit``, ``megatron/training.py:1148-1152``).

Both moments are stored as one signed / unsigned byte per element plus one fp32 scale per block of 256 elements:

* ``exp_avg``    : ``q = round(127 * m / absmax_block)``                     (linear, signed)
* ``exp_avg_sq`` : ``q = round(255 * sqrt(v / max_block))``                  (square-root domain, unsigned: the second
  moment spans many orders of magnitude inside a block and its square root is what the update divides by)

Every step de-quantises a block, applies the usual Adam(W) recurrences in fp32 and re-quantises (on a GPU in one
kernel, ``adam8bit_kernel`` in ``ops/csrc/misc_kernels.cu``: one CTA per block of 256), so the state costs
2 bytes + 1/32 byte per parameter instead of 8.  The update itself is element-wise, so it works on the flat fp32 master
shard of the mixed-precision optimizer like any other inner optimizer (and writes the bf16 model copy when the shard
carries ``model_out``).  Large tensors are processed in chunks to bound the fp32 temporaries.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import native
from ..ops.functional import _DT

BLOCK = 256
CHUNK = 1 << 24      # elements per pass (multiple of BLOCK)


def _quant_signed(x):
    xb = x.view(-1, BLOCK)
    amax = xb.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    q = torch.round(xb / amax * 127.0).to(torch.int8)
    return q.view(-1), amax.view(-1)


def _dequant_signed(q, amax):
    return (q.view(-1, BLOCK).float() * (amax.view(-1, 1) / 127.0)).view(-1)


def _quant_sqrt(v):
    vb = v.view(-1, BLOCK)
    vmax = vb.amax(dim=1, keepdim=True).clamp_min(1e-38)
    q = torch.round(torch.sqrt(vb / vmax) * 255.0).to(torch.uint8)
    return q.view(-1), vmax.view(-1)


def _dequant_sqrt(q, vmax):
    r = q.view(-1, BLOCK).float() / 255.0
    return (r * r * vmax.view(-1, 1)).view(-1)


class Adam8bit(torch.optim.Optimizer):
    supports_grad_scale = True      # the flat optimizer passes 1 / (loss scale * clip) as group["grad_scale"]

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adam_w_mode=True,
                 bias_correction=True, min_8bit_size=4096):
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, bias_correction=bias_correction)
        super().__init__(params, defaults)
        self.adam_w_mode = adam_w_mode
        self.min_8bit_size = min_8bit_size

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            group["step"] = group.get("step", 0) + 1
            t = group["step"]
            bc1, bc2 = (1.0 - b1 ** t, 1.0 - b2 ** t) if group["bias_correction"] else (1.0, 1.0)
            gs = float(group.get("grad_scale", 1.0))
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                n = p.numel()
                st = self.state[p]
                flat_p, flat_g = p.data.view(-1), p.grad.view(-1)
                out = getattr(p, "model_out", None)
                small = n < self.min_8bit_size
                if not st:
                    if small:
                        st["m"] = torch.zeros(n, dtype=torch.float32, device=p.device)
                        st["v"] = torch.zeros(n, dtype=torch.float32, device=p.device)
                    else:
                        pad = (-n) % BLOCK
                        st["pad"] = pad
                        st["qm"] = torch.zeros(n + pad, dtype=torch.int8, device=p.device)
                        st["qv"] = torch.zeros(n + pad, dtype=torch.uint8, device=p.device)
                        st["sm"] = torch.zeros((n + pad) // BLOCK, dtype=torch.float32, device=p.device)
                        st["sv"] = torch.zeros((n + pad) // BLOCK, dtype=torch.float32, device=p.device)
                if (not small and p.is_cuda and native.available() and p.dtype == torch.float32
                        and flat_g.dtype == torch.float32 and flat_p.is_contiguous() and flat_g.is_contiguous()):
                    # one kernel: de-quantise, update, re-quantise, write the parameter (and its 16-bit copy)
                    rc = native.lib().neox_adam8bit_step(
                        native.ptr(flat_p), native.ptr(st["qm"]), native.ptr(st["qv"]), native.ptr(st["sm"]),
                        native.ptr(st["sv"]), native.ptr(flat_g), native.ptr(out),
                        _DT[out.dtype] if out is not None else 1, ctypes.c_longlong(n), ctypes.c_float(lr),
                        ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(eps), ctypes.c_float(wd),
                        ctypes.c_float(bc1), ctypes.c_float(bc2), ctypes.c_float(gs), int(self.adam_w_mode),
                        ctypes.c_void_p(native.stream_ptr()))
                    native.check(rc, "neox_adam8bit_step")
                    continue
                for lo in range(0, n, CHUNK):
                    hi = min(lo + CHUNK, n)
                    g = flat_g[lo:hi].float() * gs
                    w = flat_p[lo:hi]
                    if not self.adam_w_mode and wd != 0:
                        g = g + wd * w
                    if small:
                        m, v = st["m"][lo:hi], st["v"][lo:hi]
                        m.mul_(b1).add_(g, alpha=1 - b1)
                        v.mul_(b2).addcmul_(g, g, value=1 - b2)
                    else:
                        hi_b = min((hi + BLOCK - 1) // BLOCK * BLOCK, n + st["pad"])       # whole blocks
                        bl, bh = lo // BLOCK, hi_b // BLOCK
                        m = _dequant_signed(st["qm"][lo:hi_b], st["sm"][bl:bh])
                        v = _dequant_sqrt(st["qv"][lo:hi_b], st["sv"][bl:bh])
                        gp = g if hi_b - lo == hi - lo else torch.nn.functional.pad(g, (0, hi_b - hi))
                        m.mul_(b1).add_(gp, alpha=1 - b1)
                        v.mul_(b2).addcmul_(gp, gp, value=1 - b2)
                        st["qm"][lo:hi_b], st["sm"][bl:bh] = _quant_signed(m)
                        st["qv"][lo:hi_b], st["sv"][bl:bh] = _quant_sqrt(v)
                        m, v = m[: hi - lo], v[: hi - lo]
                    upd = (m / bc1) / ((v / bc2).sqrt_().add_(eps))
                    if self.adam_w_mode and wd != 0:
                        upd = upd + wd * w
                    w.add_(upd, alpha=-lr)
                    if out is not None:
                        out.view(-1)[lo:hi].copy_(w)
        return loss


class StableEmbeddingNorm(torch.nn.LayerNorm):
    """LayerNorm applied to the token embeddings (the normalisation half of bitsandbytes' ``StableEmbedding``, which
    the reference swaps in together with the 8-bit optimizer, ``megatron/model/word_embeddings.py:71-80``): it keeps
    the embedding gradients well scaled, which is what lets 8-bit states work for that highly non-uniform tensor."""
