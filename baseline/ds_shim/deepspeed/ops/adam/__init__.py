"""FusedAdam stand-in: torch's fused (multi-tensor CUDA) Adam/AdamW with DeepSpeed's constructor."""
import torch


class FusedAdam(torch.optim.AdamW):
    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, adam_w_mode=True,
                 weight_decay=0.0, amsgrad=False, set_grad_none=True):
        assert not amsgrad
        params = list(params)
        first = params[0]["params"][0] if isinstance(params[0], dict) else params[0]
        super().__init__(params, lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                         fused=bool(first.is_cuda))
        self.adam_w_mode = adam_w_mode


class DeepSpeedCPUAdam(torch.optim.AdamW):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, **_):
        super().__init__(params, lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
