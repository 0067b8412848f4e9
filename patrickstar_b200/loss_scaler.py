"""Loss scalers with device-resident state.

Mirror of ``patrickstar/fp16/loss_scaler.py``: ``LossScaler`` (:46-76) and
``DynamicLossScaler`` (:79-190) keep their names, constructor arguments,
methods and state-machine semantics.  The state (``cur_scale``, ``cur_iter``,
``last_overflow_iter``, ``cur_hysteresis``) lives in a 64-byte block in GPU
memory and is advanced by a one-thread kernel, so an optimizer step needs no
device-to-host synchronisation; reading ``loss_scale`` / ``cur_scale`` from
Python copies the block back (and therefore synchronises).
"""
import ctypes as C

import torch

from ._lib import ScalerState, check, lib


def _stream_ptr(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class _ScaleByDeviceState(torch.autograd.Function):
    """loss * cur_scale with the scale read on the device by the kernel
    (``ps_scale_loss``): forward scales the loss, backward scales the incoming
    gradient by the same factor.  fp32 CUDA tensors."""

    @staticmethod
    def forward(ctx, loss, scaler):
        ctx.scaler = scaler
        return scaler._scale_on_device(loss)

    @staticmethod
    def backward(ctx, grad_out):
        return ctx.scaler._scale_on_device(grad_out), None


class _DeviceScaler:
    """Shared plumbing: the 64-byte ps_scaler_state block and the overflow flag."""

    def __init__(self, init: ScalerState, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError(
                "patrickstar_b200 loss scalers keep their state on a CUDA device; no device found")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._state = torch.zeros(C.sizeof(ScalerState), dtype=torch.uint8, device=self.device)
        # int32 overflow flag, OR-ed into by the scan kernels
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._host_init = init
        with torch.cuda.device(self.device):
            check(lib.ps_scaler_init(self._state.data_ptr(), C.byref(init), _stream_ptr(self.device)),
                  "ps_scaler_init")

    # --- device handles used by FP16Adam -----------------------------------
    @property
    def state_ptr(self):
        return self._state.data_ptr()

    @property
    def flag_ptr(self):
        return self._flag.data_ptr()

    @property
    def flag_tensor(self):
        return self._flag

    @property
    def scale_tensor(self):
        """0-dim float64 view of cur_scale on the device (no sync)."""
        return self._state[:8].view(torch.float64)[0]

    def read_state(self) -> ScalerState:
        out = ScalerState()
        with torch.cuda.device(self.device):
            check(lib.ps_scaler_read(self._state.data_ptr(), C.byref(out), _stream_ptr(self.device)),
                  "ps_scaler_read")
        return out

    def load_state(self, st: ScalerState):
        with torch.cuda.device(self.device):
            check(lib.ps_scaler_init(self._state.data_ptr(), C.byref(st), _stream_ptr(self.device)),
                  "ps_scaler_init")

    # --- reference API -------------------------------------------------------
    @property
    def loss_scale(self):
        return self.cur_scale

    @property
    def cur_scale(self):
        v = self.read_state().cur_scale
        return int(v) if float(v).is_integer() and self._int_scale else v

    def _scale_on_device(self, x):
        x = x.contiguous()
        out = torch.empty_like(x)
        with torch.cuda.device(self.device):
            check(lib.ps_scale_loss(x.data_ptr(), out.data_ptr(), x.numel(), self._state.data_ptr(),
                                    _stream_ptr(self.device)), "ps_scale_loss")
        return out

    def scale_loss(self, loss):
        """``loss * self.loss_scale`` as a differentiable device-side product: the
        scale never travels to the host.  fp32 CUDA losses go through the
        ``ps_scale_loss`` kernel; any other dtype is multiplied by the scale's
        device tensor."""
        if loss.is_cuda and loss.dtype == torch.float32 and loss.device == self.device:
            return _ScaleByDeviceState.apply(loss, self)
        return loss * self.scale_tensor.to(device=loss.device, dtype=loss.dtype)

    def backward(self, loss, retain_graph=False):
        """loss_scaler.py:188-190 — scaled backward; the scale is multiplied in on
        the device, without reading it back."""
        self.scale_loss(loss).backward(retain_graph=retain_graph)

    def state_dict(self):
        st = self.read_state()
        return {name: getattr(st, name) for name, _ in ScalerState._fields_}

    def load_state_dict(self, d):
        st = ScalerState()
        for name, _ in ScalerState._fields_:
            setattr(st, name, d[name])
        self.load_state(st)


class LossScaler(_DeviceScaler):
    """Static loss scale (loss_scaler.py:46-76): never reports an overflow and
    never changes."""

    def __init__(self, scale=1, device=None):
        self._int_scale = isinstance(scale, int)
        st = ScalerState(cur_scale=float(scale), scale_factor=1.0, min_scale=float(scale), cur_iter=0,
                         last_overflow_iter=-1, scale_window=1, delayed_shift=1, cur_hysteresis=1,
                         consecutive_hysteresis=0, dynamic=0)
        super().__init__(st, device)

    def has_overflow(self, param):
        return False

    @staticmethod
    def _has_inf_or_nan(x):
        return False

    def update_scale(self, overflow):
        pass


class DynamicLossScaler(_DeviceScaler):
    """Dynamic loss scale (loss_scaler.py:79-190).  Same constructor and the same
    transitions as the reference; see ``update_scale``."""

    def __init__(self, init_scale=2 ** 32, scale_factor=2.0, scale_window=1000, min_scale=1,
                 delayed_shift=1, consecutive_hysteresis=False, device=None):
        self._int_scale = isinstance(init_scale, int)
        self.scale_factor = scale_factor
        self.scale_window = scale_window
        self.min_scale = min_scale
        self.delayed_shift = delayed_shift
        self.consecutive_hysteresis = consecutive_hysteresis
        st = ScalerState(cur_scale=float(init_scale), scale_factor=float(scale_factor),
                         min_scale=float(min_scale), cur_iter=0, last_overflow_iter=-1,
                         scale_window=int(scale_window), delayed_shift=int(delayed_shift),
                         cur_hysteresis=int(delayed_shift),
                         consecutive_hysteresis=int(bool(consecutive_hysteresis)), dynamic=1)
        super().__init__(st, device)

    @property
    def cur_iter(self):
        return int(self.read_state().cur_iter)

    @property
    def last_overflow_iter(self):
        return int(self.read_state().last_overflow_iter)

    @property
    def cur_hysteresis(self):
        return int(self.read_state().cur_hysteresis)

    def accumulate_overflow(self, grad):
        """Device-side form of ``has_overflow``: ORs "grad holds an inf or nan" into
        the flag without synchronising.  ``grad`` is a CUDA fp16 tensor."""
        if grad is None or grad.numel() == 0:
            return
        if grad.dtype != torch.float16 or not grad.is_cuda:
            raise TypeError("overflow scan needs a CUDA fp16 gradient, got %s on %s" % (grad.dtype, grad.device))
        g = grad if grad.is_contiguous() else grad.contiguous()
        with torch.cuda.device(self.device):
            check(lib.ps_overflow_scan_buffer(g.data_ptr(), g.numel(), self.flag_ptr,
                                              _stream_ptr(self.device)), "ps_overflow_scan_buffer")

    def has_overflow(self, param):
        """loss_scaler.py:127-131 — True when ``param.grad`` holds an inf or nan.
        Returns a Python bool like the reference, which costs a device sync; the
        optimizer itself uses ``accumulate_overflow`` and never syncs."""
        return DynamicLossScaler._has_inf_or_nan(param.grad)

    @staticmethod
    def _has_inf_or_nan(x):
        """loss_scaler.py:133-155.  The reference sums the tensor in fp32 and tests
        the sum; for fp16 gradients that is "any element is inf or nan", which is
        what the scan kernel tests."""
        if x is None or x.numel() == 0:
            return False
        if not x.is_cuda:
            raise TypeError("patrickstar_b200 checks gradients on the GPU only")
        if x.dtype != torch.float16:
            # not a chunk gradient (the reference's fp32 grads of torch-managed
            # params): the reference's own formulation, literally
            cpu_sum = float(x.float().sum())
            return cpu_sum == float("inf") or cpu_sum == -float("inf") or cpu_sum != cpu_sum
        g = x.contiguous()
        flag = torch.zeros(1, dtype=torch.int32, device=x.device)
        with torch.cuda.device(x.device):
            check(lib.ps_overflow_scan_buffer(g.data_ptr(), g.numel(), flag.data_ptr(),
                                              _stream_ptr(x.device)), "ps_overflow_scan_buffer")
        return bool(flag.item())

    def update_scale(self, overflow):
        """loss_scaler.py:158-182 as a one-thread kernel.  ``overflow`` is a bool,
        or None to consume (and clear) the device flag."""
        with torch.cuda.device(self.device):
            if overflow is None:
                check(lib.ps_scaler_update(self.state_ptr, self.flag_ptr, 0, _stream_ptr(self.device)),
                      "ps_scaler_update")
            else:
                check(lib.ps_scaler_update(self.state_ptr, None, int(bool(overflow)),
                                           _stream_ptr(self.device)), "ps_scaler_update")
