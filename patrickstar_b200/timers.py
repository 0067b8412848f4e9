"""Section timers for the optimizer step, on CUDA events.

The reference times the step with wall-clock sections that synchronise the
stream at every stop (patrickstar/utils/global_timer.py:51-66; keys ADAM,
ADAM_prepare_data, ADAM_compute, ... in patrickstar/ops/fp16_cpu_adam.py:340-467).
Here a section is a pair of CUDA events recorded on the step's stream: starting
and stopping a section never synchronises; ``summary()`` does, once, when the
numbers are read.
"""
from collections import OrderedDict

import torch

# the reference's key names where a phase still exists in the fused step
ADAM = "ADAM"
ADAM_COMPUTE = "ADAM_compute"                # the fused chunk-step kernel (includes the fp16 write-back,
                                             # which the reference times as ADAM_param_fp32_to_fp16)
ADAM_OVERFLOW_SCAN = "ADAM_overflow_scan"    # no counterpart: the reference checks per parameter in backward
ADAM_OFFLOAD = "ADAM_offload_pipeline"       # replaces ADAM_prepare_data / ADAM_release_data chunk moves


class PhaseTimer:
    def __init__(self):
        self._open = {}
        self._pairs = OrderedDict()
        self._bytes = OrderedDict()   # key -> bytes moved, the reference's DataMoveCnter (global_timer.py:94-126)

    def update_bytes(self, key, nbytes):
        """Account ``nbytes`` of memory traffic to a section (host-side bookkeeping only)."""
        self._bytes[key] = self._bytes.get(key, 0) + int(nbytes)

    def bandwidth(self):
        """{key: GB/s} for the sections that were given byte counts; synchronises the device."""
        times = self.summary()
        return OrderedDict((k, b / (times[k][1] * 1e-3) / 1e9) for k, b in self._bytes.items()
                           if k in times and times[k][1] > 0)

    def start_profile(self, key):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self._open[key] = e

    def finish_profile(self, key):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self._pairs.setdefault(key, []).append((self._open.pop(key), e))

    def summary(self):
        """{key: (calls, total ms)}; synchronises the device."""
        torch.cuda.synchronize()
        return OrderedDict((k, (len(v), sum(a.elapsed_time(b) for a, b in v))) for k, v in self._pairs.items())

    def reset(self):
        self._open.clear()
        self._pairs.clear()
        self._bytes.clear()
