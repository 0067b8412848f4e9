"""ctypes binding of the C ABI declared in ``include/ps_b200.h``.

The shared library is built in-tree by ``patrickstar_b200.build`` (nvcc,
sm_100a only).  There is no fallback of any kind: if the library is missing the
import of this module raises, and every compute entry point reports
``PS_ERR_CUDA`` when no CUDA device is present.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libps_b200.so")

PS_OK = 0
PS_ERR_INVALID = -1
PS_ERR_UNKNOWN_ID = -2
PS_ERR_ALIGN = -3
PS_ERR_CUDA = -4
PS_ERR_TABLE = -5
PS_ERR_LIMIT = -6

PS_MAX_GROUPS = 15
PS_MAX_SLOTS = PS_MAX_GROUPS + 1
PS_STATIC_MAX_CHUNKS = 256
PS_STATIC_MAX_SEGMENTS = 4096


class PSError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code, where, detail=""):
        self.code = code
        super().__init__("%s failed: %s (%d)%s" % (where, _strerror(code), code, detail))


# numpy dtypes that mirror the C structs byte for byte
CHUNK_DESC_DTYPE = np.dtype(
    [("p32", "<u8"), ("exp_avg", "<u8"), ("exp_avg_sq", "<u8"), ("h16", "<u8"),
     ("numel", "<u4"), ("seg_begin", "<u4"), ("seg_end", "<u4"), ("reserved", "<u4")])
SEGMENT_DTYPE = np.dtype([("start", "<u4"), ("end", "<u4"), ("slot", "<u4"), ("reserved", "<u4")])
TENSOR_DESC_DTYPE = np.dtype([("p32", "<u8"), ("grad", "<u8"), ("exp_avg", "<u8"), ("exp_avg_sq", "<u8"),
                              ("numel", "<u8"), ("slot", "<u4"), ("reserved", "<u4")])
OFFLOAD_CHUNK_DTYPE = np.dtype([("p32_host", "<u8"), ("exp_avg_host", "<u8"), ("exp_avg_sq_host", "<u8"),
                                ("numel", "<u4"), ("desc_index", "<u4")])
assert TENSOR_DESC_DTYPE.itemsize == 48
assert CHUNK_DESC_DTYPE.itemsize == 48 and SEGMENT_DTYPE.itemsize == 16 and OFFLOAD_CHUNK_DTYPE.itemsize == 32


class GroupHyper(C.Structure):
    _fields_ = [("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("weight_decay", C.c_float), ("adamw_mode", C.c_int32), ("reserved", C.c_int32 * 2)]


class StepPlan(C.Structure):
    _fields_ = [("clip", C.c_double), ("groups", GroupHyper * PS_MAX_GROUPS), ("n_groups", C.c_int32),
                ("first_group", C.c_int32), ("last_group", C.c_int32), ("n_calls", C.c_int32),
                ("grad_divisor", C.c_float), ("bias_correction", C.c_int32)]


class ScalerState(C.Structure):
    _fields_ = [("cur_scale", C.c_double), ("scale_factor", C.c_double), ("min_scale", C.c_double),
                ("cur_iter", C.c_int64), ("last_overflow_iter", C.c_int64), ("scale_window", C.c_int64),
                ("delayed_shift", C.c_int32), ("cur_hysteresis", C.c_int32),
                ("consecutive_hysteresis", C.c_int32), ("dynamic", C.c_int32)]


class HyperSlot(C.Structure):
    _fields_ = [("loss_scale", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float),
                ("beta1_minus1", C.c_float), ("beta2_minus1", C.c_float), ("bias2_sqrt", C.c_float),
                ("eps", C.c_float), ("step_size", C.c_float), ("weight_decay", C.c_float),
                ("w_decay", C.c_float), ("clip", C.c_float), ("grad_divisor", C.c_float),
                ("adamw_mode", C.c_int32), ("inv_loss_scale", C.c_float), ("inv_grad_divisor", C.c_float),
                ("reserved", C.c_int32)]


class StepCtrl(C.Structure):
    _fields_ = [("skip", C.c_int32), ("error", C.c_int32), ("step", C.c_uint64),
                ("n_skipped", C.c_uint64), ("native_step", C.c_uint64), ("betta1", C.c_float),
                ("betta2", C.c_float), ("betta1_t", C.c_float), ("betta2_t", C.c_float),
                ("slots", HyperSlot * PS_MAX_SLOTS)]


assert C.sizeof(StepPlan) == 512 and C.sizeof(ScalerState) == 64
assert C.sizeof(HyperSlot) == 64 and C.sizeof(StepCtrl) == 48 + 64 * PS_MAX_SLOTS

# name -> (restype, argtypes); every name declared in include/ps_b200.h
_p = C.c_void_p
SIGNATURES = {
    "ps_version": (C.c_int, []),
    "ps_strerror": (C.c_char_p, [C.c_int]),
    "ps_last_cuda_error": (C.c_int, []),
    "ps_launch_count": (C.c_uint64, []),
    "ps_tune": (C.c_int, [C.c_char_p, C.c_int]),
    "ps_adam_create": (C.c_int, [C.c_int, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float,
                                 C.c_int, C.c_int]),
    "ps_adam_destroy": (C.c_int, [C.c_int]),
    "ps_adam_get_state": (C.c_int, [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_uint64)]),
    "ps_adam_update": (C.c_int, [C.c_int, C.c_size_t, C.c_float, C.c_float, C.c_float, C.c_float,
                                 C.c_float, C.c_int, _p, _p, _p, _p, C.c_size_t, C.c_int, C.c_float,
                                 _p, _p]),
    "ps_table_check": (C.c_int, [_p, C.c_uint32, _p, C.c_uint32, C.c_uint32, C.c_uint32]),
    "ps_piece_table_check": (C.c_int, [_p, C.c_uint32, C.c_uint32, C.c_uint32]),
    "ps_pow_table_fill": (C.c_int, [C.c_float, C.c_float, C.c_uint64, C.c_uint64, _p]),
    "ps_ctrl_init": (C.c_int, [_p, C.c_uint64, C.c_float, C.c_float, _p]),
    "ps_scaler_init": (C.c_int, [_p, C.POINTER(ScalerState), _p]),
    "ps_overflow_scan": (C.c_int, [_p, C.c_uint32, C.c_uint32, _p, _p]),
    "ps_overflow_scan_buffer": (C.c_int, [_p, C.c_size_t, _p, _p]),
    "ps_grad_handoff": (C.c_int, [_p, _p, C.c_size_t, _p, _p]),
    "ps_step_begin": (C.c_int, [_p, _p, _p, C.POINTER(StepPlan), _p, C.c_uint64, _p]),
    "ps_scaler_update": (C.c_int, [_p, _p, C.c_int, _p]),
    "ps_chunk_step": (C.c_int, [_p, C.c_uint32, C.c_uint32, _p, _p, _p]),
    "ps_chunk_step_static": (C.c_int, [_p, C.c_uint32, C.c_uint32, _p, C.c_uint32, _p, C.c_uint32,
                                       C.c_int, _p]),
    "ps_offload_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int]),
    "ps_offload_destroy": (C.c_int, [_p]),
    "ps_offload_step": (C.c_int, [_p, _p, C.c_uint32, _p, _p, _p, _p, _p]),
    "ps_offload_last_cuda_error": (C.c_int, []),
    "ps_chunk_step_fused": (C.c_int, [_p, C.c_uint32, C.c_uint32, _p, _p, _p, _p, _p, C.c_int, _p]),
    "ps_chunk_step_p2p": (C.c_int, [_p, C.c_uint32, C.c_uint32, _p, _p, _p, _p, C.c_int, _p]),
    "ps_fused_pipe_create": (C.c_int, [C.POINTER(C.c_void_p)]),
    "ps_fused_pipe_destroy": (C.c_int, [_p]),
    "ps_chunk_step_fused_staged": (C.c_int, [_p, _p, C.c_uint32, C.c_uint32, _p, _p, _p, _p, _p, C.c_int, _p, _p]),
    "ps_copy_pipe_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int]),
    "ps_copy_pipe_destroy": (C.c_int, [_p]),
    "ps_chunk_step_copy": (C.c_int, [_p, _p, _p, C.c_uint32, C.c_uint32, _p, _p, _p, _p, _p, C.c_int, C.c_int, _p, _p, _p]),
    "ps_restore_fp16": (C.c_int, [_p, C.c_uint32, C.c_uint32, _p, _p]),
    "ps_tensor_table_step": (C.c_int, [_p, C.c_uint32, C.c_uint32, _p, _p, _p]),
    "ps_p2p_reduce_probe": (C.c_int, [_p, _p, _p, C.c_int, _p, C.c_size_t, _p]),
    "ps_multimem_reduce_probe": (C.c_int, [_p, _p, C.c_size_t, _p]),
    "ps_scaler_read": (C.c_int, [_p, C.POINTER(ScalerState), _p]),
    "ps_ctrl_read": (C.c_int, [_p, C.POINTER(StepCtrl), _p]),
    "ps_scale_loss": (C.c_int, [_p, _p, C.c_size_t, _p, _p]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "patrickstar_b200: %s is missing. Build it with `python -m patrickstar_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback." % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def _strerror(code):
    return lib.ps_strerror(code).decode()


def check(code, where):
    """Raise PSError for a negative status."""
    if code != PS_OK:
        detail = ""
        if code == PS_ERR_CUDA:
            detail = " [cudaError %d]" % lib.ps_last_cuda_error()
        raise PSError(code, where, detail)


def launch_count():
    return int(lib.ps_launch_count())


def tune(key, value):
    check(lib.ps_tune(key.encode(), int(value)), "ps_tune")
