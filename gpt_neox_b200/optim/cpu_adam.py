"""Adam on host memory through the OpenMP/AVX2 C++ kernel ``neox_cpu_adam_step``
(``ops/csrc/host/cpu_adam.cpp``): the optimizer of the state-offload path (``optimizer.type: cpu_adam``,
``zero_optimization.cpu_offload`` / ``offload_optimizer``), the role DeepSpeed's ``DeepSpeedCPUAdam`` has for the
reference."""
from __future__ import annotations

import ctypes

import torch

from ..ops import native


class CPUAdam(torch.optim.Optimizer):
    """Parameters that already live in host memory (fp32, contiguous: the offloaded master shards of the flat
    optimizer) are updated in place, and a host bf16 tensor hung on the parameter as ``model_out`` receives the
    rounded copy in the same pass.  A parameter on a device is staged through a host copy kept in the state."""
    supports_grad_scale = True
    writes_host_out = True

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adamw_mode=True,
                 bias_correction=True, **_ignored):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                                      bias_correction=bias_correction, grad_scale=1.0))
        self.adamw_mode = adamw_mode

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        lib = native.host_lib()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            group["step"] = group.get("step", 0) + 1
            t = group["step"]
            bc1, bc2 = (1 - b1 ** t, 1 - b2 ** t) if group["bias_correction"] else (1.0, 1.0)
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                in_place = p.device.type == "cpu" and p.dtype == torch.float32 and p.is_contiguous()
                if not st:
                    st["exp_avg"] = torch.zeros(p.numel(), dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros(p.numel(), dtype=torch.float32)
                    if not in_place:
                        st["host_param"] = p.detach().float().cpu().reshape(-1).clone()
                host_p = p.data.view(-1) if in_place else st["host_param"]
                g = p.grad.detach()
                if g.device.type != "cpu" or g.dtype != torch.float32 or not g.is_contiguous():
                    g = g.float().cpu().contiguous()
                g = g.view(-1)
                out = getattr(p, "model_out", None)
                out_ptr = None
                if in_place and out is not None and out.device.type == "cpu" and out.dtype == torch.bfloat16:
                    out_ptr = ctypes.c_void_p(out.data_ptr())
                lib.neox_cpu_adam_step(ctypes.c_void_p(host_p.data_ptr()), ctypes.c_void_p(st["exp_avg"].data_ptr()),
                                       ctypes.c_void_p(st["exp_avg_sq"].data_ptr()), ctypes.c_void_p(g.data_ptr()),
                                       out_ptr, ctypes.c_longlong(host_p.numel()), ctypes.c_float(group["lr"]),
                                       ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(group["eps"]),
                                       ctypes.c_float(group["weight_decay"]), ctypes.c_float(bc1), ctypes.c_float(bc2),
                                       ctypes.c_float(float(group.get("grad_scale", 1.0))), int(self.adamw_mode))
                if not in_place:
                    p.copy_(host_p.view_as(p).to(p.device, non_blocking=True))
        return loss
