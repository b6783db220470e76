"""fp16 loss scaling: static, or dynamic with hysteresis (config block ``fp16``: ``loss_scale``,
``initial_scale_power``, ``loss_scale_window``, ``hysteresis``, ``min_loss_scale``)."""
from __future__ import annotations


class StaticLossScaler:
    dynamic = False

    def __init__(self, scale=1.0):
        self.cur_scale = float(scale)

    def update_scale(self, overflow):
        pass

    def state_dict(self):
        return {"cur_scale": self.cur_scale}

    def load_state_dict(self, sd):
        self.cur_scale = float(sd.get("cur_scale", self.cur_scale))


class DynamicLossScaler:
    """Halve the scale on overflow (after ``hysteresis`` consecutive overflows have been absorbed),
    double it after ``scale_window`` clean steps."""
    dynamic = True

    def __init__(self, init_scale=2 ** 16, scale_factor=2.0, scale_window=1000, min_scale=1.0, hysteresis=2,
                 consecutive_hysteresis=False):
        self.cur_scale = float(init_scale)
        self.scale_factor, self.scale_window, self.min_scale = scale_factor, scale_window, min_scale
        self.delayed_shift = hysteresis
        self.cur_hysteresis = hysteresis
        self.consecutive_hysteresis = consecutive_hysteresis
        self.cur_iter, self.last_overflow_iter = 0, -1

    def update_scale(self, overflow):
        if overflow:
            if self.delayed_shift == 1 or self.cur_hysteresis == 1:
                self.cur_scale = max(self.cur_scale / self.scale_factor, self.min_scale)
            else:
                self.cur_hysteresis -= 1
            self.last_overflow_iter = self.cur_iter
        else:
            if self.consecutive_hysteresis:
                self.cur_hysteresis = self.delayed_shift
            if (self.cur_iter - self.last_overflow_iter) % self.scale_window == 0:
                if not self.consecutive_hysteresis:
                    self.cur_hysteresis = self.delayed_shift
                self.cur_scale *= self.scale_factor
        self.cur_iter += 1

    def state_dict(self):
        return {k: getattr(self, k) for k in ("cur_scale", "cur_iter", "last_overflow_iter", "cur_hysteresis")}

    def load_state_dict(self, sd):
        for k, v in sd.items():
            setattr(self, k, v)
