"""TEST INFRASTRUCTURE — the protocol of ``FP16Adam.step`` on the CPU.

Restates patrickstar/ops/fp16_cpu_adam.py:472-628 over the C Adam oracle for
one rank's local chunks:

  * overflow gate (``:287-310``): if any local gradient holds inf/nan (the flag
    is the OR over ranks), every local fp16 chunk is restored from the fp32
    master, the scaler takes ``update_scale(True)`` and the step counter is NOT
    advanced (``:549-558``);
  * otherwise ``state["step"] += 1`` (``:574``), one ``adam_update`` call per
    tensor piece in storage order (``:336-428``) on ONE optimizer object — so
    the reference's call-history dependent beta^t is reproduced — then the fp16
    chunk := cast(fp32 master) (``chunk_io_buff.py:85-128``) and
    ``update_scale(False)`` (``:624-625``);
  * the gradient is first divided by the world size in fp16
    (patrickstar/core/client.py:838) when ``world_size > 1`` and clamped in
    fp16 when gradient clipping is on (``:365-379``, GPU flavour).

  * a torch-managed parameter (``:345-353``: fp32 parameter that is its own
    master, fp32 gradient) is one more adam_update call at its place of the
    visiting order, with no fp16 write-back; its gradient is neither divided by
    the world size nor tested for overflow, and an overflow step leaves it
    untouched (``:301-302``).

Arrays are numpy: fp16 chunks as uint16/float16, states as float32.
"""
import numpy as np

from . import port


class StepOracle:
    def __init__(self, calls, groups, scaler, use_adamw, gradient_clipping=-1, world_size=1,
                 trailing_call_group=None):
        """calls: list of (chunk_index, start, end, group) in visiting order; an
        entry ("torch", k, group) is the k-th torch-managed parameter of the
        ``torch_params`` list given to ``step``.
        groups: list of dicts lr / betas / eps / weight_decay.
        trailing_call_group: when the oracle follows only the first tensors of a
        rank, the group index of the rank's LAST tensor: an empty adam_update
        call with that group's betas is made after the followed ones, so that
        the optimizer object's beta^t history (cpu_adam.h:143-162) is the one the
        full call sequence leaves behind."""
        self.trailing_call_group = trailing_call_group
        self.calls = list(calls)
        self.groups = groups
        self.scaler = scaler
        self.use_adamw = use_adamw
        self.clip = gradient_clipping
        self.world_size = world_size
        g0 = groups[0]
        # create_adam with the constructor's hyper-parameters (fp16_cpu_adam.py:183-193)
        self.adam = port.OracleAdam(g0["lr"], g0["betas"][0], g0["betas"][1], g0["eps"],
                                    g0["weight_decay"], use_adamw)
        self.step_count = 0
        self.skipped = 0

    def _prepared_grad(self, g16):
        g = g16.copy()
        if self.world_size > 1:
            port.div_world_f16(g.view(np.uint16), self.world_size)
        if self.clip > 0:
            c = self.clip
            if self.scaler is not None:
                c = c * self.scaler.loss_scale
            c = np.float32(min(65504.0, c))
            g = np.clip(g.astype(np.float32), -c, c).astype(np.float16)
        return g

    def step(self, h16, p32, exp_avg, exp_avg_sq, overflow=None, torch_params=None):
        """h16 / p32 / exp_avg / exp_avg_sq: lists of per-chunk arrays (in place).
        overflow: the flag after the all-reduce; None = derive from h16.
        torch_params: list of (param fp32, grad fp32, exp_avg, exp_avg_sq) flat
        arrays of the torch-managed parameters (updated in place)."""
        dynamic = self.scaler is not None and getattr(self.scaler, "dynamic", False)
        if overflow is None:
            overflow = dynamic and any(port.has_inf_or_nan_f16(h.view(np.uint16)) for h in h16)
        if not dynamic:
            overflow = False
        if overflow:
            # every local parameter's fp16 slot := cast(fp32 master).  (The reference
            # copies chunk-wise, gaps included; gaps hold zeros on both sides there,
            # so restoring the parameters' own elements is the same thing.)
            for call in self.calls:
                if call[0] == "torch":
                    continue
                c, s, e, _ = call
                out = np.empty(e - s, dtype=np.uint16)
                port.cast_fp32_to_fp16(np.ascontiguousarray(p32[c][s:e]), out)
                h16[c].view(np.uint16)[s:e] = out
            self.scaler.update_scale(True)
            self.skipped += 1
            return True
        self.step_count += 1
        loss_scale = self.scaler.loss_scale if self.scaler is not None else -1
        for call in self.calls:
            if call[0] == "torch":
                _, k, g = call
                hp = self.groups[g]
                tp, tg, tm, tv = torch_params[k]
                if self.clip > 0:
                    # clamp_ on the fp32 gradient itself (fp16_cpu_adam.py:365-379)
                    c_ = self.clip * (self.scaler.loss_scale if self.scaler is not None else 1)
                    c_ = np.float32(min(65504.0, c_))
                    tg = np.clip(tg, -c_, c_).astype(np.float32)
                self.adam.adam_update(self.step_count, hp["lr"], hp["betas"][0], hp["betas"][1], hp["eps"],
                                      hp["weight_decay"], True, tp, np.ascontiguousarray(tg), tm, tv, loss_scale)
                continue
            c, s, e, g = call
            hp = self.groups[g]
            grad = self._prepared_grad(h16[c][s:e].view(np.float16))
            p = np.ascontiguousarray(p32[c][s:e])
            m = np.ascontiguousarray(exp_avg[c][s:e])
            v = np.ascontiguousarray(exp_avg_sq[c][s:e])
            self.adam.adam_update(self.step_count, hp["lr"], hp["betas"][0], hp["betas"][1], hp["eps"],
                                  hp["weight_decay"], True, p, grad, m, v, loss_scale)
            p32[c][s:e] = p
            exp_avg[c][s:e] = m
            exp_avg_sq[c][s:e] = v
            out = np.empty(e - s, dtype=np.uint16)
            port.cast_fp32_to_fp16(p, out)
            h16[c].view(np.uint16)[s:e] = out
        if self.trailing_call_group is not None:
            hp = self.groups[self.trailing_call_group]
            e32, e16 = np.zeros(0, dtype=np.float32), np.zeros(0, dtype=np.float16)
            self.adam.adam_update(self.step_count, hp["lr"], hp["betas"][0], hp["betas"][1], hp["eps"],
                                  hp["weight_decay"], True, e32, e16, e32.copy(), e32.copy(), loss_scale)
        if self.scaler is not None:
            self.scaler.update_scale(False)
        return False
