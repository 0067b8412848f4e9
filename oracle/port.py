"""TEST INFRASTRUCTURE — ctypes binding of ``adam_oracle.c`` (the C restatement
of patrickstar/ops/csrc/adam/cpu_adam.cpp and csrc/includes/cpu_adam.h)."""
import ctypes as C

import numpy as np

from . import build

_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build.build_port())
        L.ps_oracle_adam_create.restype = C.c_void_p
        L.ps_oracle_adam_create.argtypes = [C.c_float] * 5 + [C.c_int]
        L.ps_oracle_adam_destroy.argtypes = [C.c_void_p]
        L.ps_oracle_adam_update.restype = C.c_int
        L.ps_oracle_adam_update.argtypes = ([C.c_void_p, C.c_size_t] + [C.c_float] * 5 + [C.c_int]
                                            + [C.c_void_p] * 4 + [C.c_size_t, C.c_int, C.c_float])
        L.ps_oracle_adam_get_state.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_uint64)]
        L.ps_oracle_cast_fp32_to_fp16.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.ps_oracle_has_inf_or_nan_f16.restype = C.c_int
        L.ps_oracle_has_inf_or_nan_f16.argtypes = [C.c_void_p, C.c_size_t]
        L.ps_oracle_div_world_f16.argtypes = [C.c_void_p, C.c_size_t, C.c_int]
        _lib = L
    return _lib


def _ptr(a):
    """Address of a numpy array or a CPU torch tensor."""
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data
    assert a.device.type == "cpu" and a.is_contiguous()
    return a.data_ptr()


def _numel(a):
    return a.size if isinstance(a, np.ndarray) else a.numel()


def _is_half(a):
    return (a.dtype == np.float16) if isinstance(a, np.ndarray) else (a.element_size() == 2)


class OracleAdam:
    """One Adam_Optimizer object (cpu_adam.h:85-206): create_adam / adam_update."""

    def __init__(self, alpha=1e-3, betta1=0.9, betta2=0.999, eps=1e-8, weight_decay=0.0, adamw_mode=True):
        self._h = lib().ps_oracle_adam_create(alpha, betta1, betta2, eps, weight_decay, int(adamw_mode))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ps_oracle_adam_destroy(self._h)
            self._h = None

    def adam_update(self, step, lr, beta1, beta2, epsilon, weight_decay, bias_correction, params, grads,
                    exp_avg, exp_avg_sq, loss_scale):
        """ds_adam_step (cpu_adam.cpp:700-742).  Arrays: fp32 params / exp_avg /
        exp_avg_sq (in place), fp16 or fp32 grads."""
        n = _numel(params)
        assert _numel(grads) == n and _numel(exp_avg) == n and _numel(exp_avg_sq) == n
        return lib().ps_oracle_adam_update(self._h, step, lr, beta1, beta2, epsilon, weight_decay,
                                           int(bool(bias_correction)), _ptr(params), _ptr(grads),
                                           _ptr(exp_avg), _ptr(exp_avg_sq), n, int(_is_half(grads)),
                                           float(loss_scale))

    def state(self):
        out = (C.c_float * 4)()
        step = C.c_uint64()
        lib().ps_oracle_adam_get_state(self._h, out, C.byref(step))
        return {"betta1_t": out[0], "betta2_t": out[1], "bias_correction1": out[2],
                "bias_correction2": out[3], "step": step.value}


def cast_fp32_to_fp16(src, dst):
    """chunk_io_buff.py:85-128 — fp16 param chunk := cast(fp32 master chunk)."""
    assert _numel(src) == _numel(dst)
    lib().ps_oracle_cast_fp32_to_fp16(_ptr(src), _ptr(dst), _numel(src))


def has_inf_or_nan_f16(g):
    """loss_scaler.py:133-155 on an fp16 gradient."""
    return bool(lib().ps_oracle_has_inf_or_nan_f16(_ptr(g), _numel(g)))


def div_world_f16(g, world_size):
    """client.py:838 — in-place fp16 `payload /= world_size`."""
    lib().ps_oracle_div_world_f16(_ptr(g), _numel(g), int(world_size))
