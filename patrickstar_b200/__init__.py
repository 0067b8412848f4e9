"""patrickstar_b200 — PatrickStar's per-chunk mixed-precision optimizer step on B200.

Public names mirror the reference's for this path:

    from patrickstar_b200 import FP16Adam, DynamicLossScaler, LossScaler, initialize_engine
    from patrickstar_b200 import cpu_adam_op      # create_adam / adam_update / destroy_adam

Everything that computes goes through ``libps_b200.so`` (hand-written sm_100a
CUDA behind a C ABI, ``include/ps_b200.h``).  There is no CPU or PyTorch
fallback: importing a compute name without the built library raises.
"""
__version__ = "0.1.0"

_LAZY = {
    "FP16Adam": ("fp16_adam", "FP16Adam"),
    "LossScaler": ("loss_scaler", "LossScaler"),
    "DynamicLossScaler": ("loss_scaler", "DynamicLossScaler"),
    "ChunkClient": ("client", "ChunkClient"),
    "ChunkLayout": ("chunk_list", "ChunkLayout"),
    "initialize_engine": ("engine", "initialize_engine"),
    "ChunkStepEngine": ("engine", "ChunkStepEngine"),
    "cpu_adam_op": ("cpu_adam_op", None),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        m = importlib.import_module("." + mod, __name__)
        return m if attr is None else getattr(m, attr)
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
