"""TEST INFRASTRUCTURE — Python restatement of the reference's loss scalers and
of the engine's config mapping.  Checker only; the product keeps this state on
the GPU.

Follows patrickstar/fp16/loss_scaler.py:46-76 (LossScaler), :107-182
(DynamicLossScaler) and patrickstar/runtime/engine.py:79-99 (config -> scaler).
Pinned against the reference's own class by tests/golden/scaler_*.json.
"""


class StaticScalerOracle:
    """loss_scaler.py:46-76 — never overflows, never changes."""

    def __init__(self, scale=1):
        self.cur_scale = scale

    def update_scale(self, overflow):
        pass

    @property
    def loss_scale(self):
        return self.cur_scale

    dynamic = False


class DynamicScalerOracle:
    """loss_scaler.py:107-182."""

    dynamic = True

    def __init__(self, init_scale=2 ** 32, scale_factor=2.0, scale_window=1000, min_scale=1,
                 delayed_shift=1, consecutive_hysteresis=False):
        self.cur_scale = init_scale
        self.cur_iter = 0
        self.last_overflow_iter = -1
        self.scale_factor = scale_factor
        self.scale_window = scale_window
        self.min_scale = min_scale
        self.delayed_shift = delayed_shift
        self.cur_hysteresis = delayed_shift
        self.consecutive_hysteresis = consecutive_hysteresis

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

    @property
    def loss_scale(self):
        return self.cur_scale

    def snapshot(self):
        return {"cur_scale": float(self.cur_scale), "cur_iter": self.cur_iter,
                "last_overflow_iter": self.last_overflow_iter, "cur_hysteresis": self.cur_hysteresis}


def scaler_from_config(config):
    """engine.py:79-99: no "fp16" key -> None; loss_scale == 0 -> dynamic scaler
    with init_scale 2**initial_scale_power (16), scale_factor = config["hysteresis"]
    (2) [sic], scale_window = loss_scale_window (2000), min_scale = min_loss_scale
    (1), delayed_shift 1; else the static scaler."""
    if config is None or "fp16" not in config:
        return None
    ls = config["fp16"]
    assert ls["enabled"], "Must enable fp16 training."
    assert "loss_scale" in ls, "Must have `loss_scale` field set."
    if ls["loss_scale"] == 0:
        return DynamicScalerOracle(
            init_scale=2 ** ls.get("initial_scale_power", 16),
            scale_factor=ls.get("hysteresis", 2),
            scale_window=ls.get("loss_scale_window", 2000),
            min_scale=ls.get("min_loss_scale", 1))
    return StaticScalerOracle(ls["loss_scale"])
