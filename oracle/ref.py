"""TEST INFRASTRUCTURE — loader of the reference's own CPU Adam, compiled
unmodified into ``oracle/_ref`` by ``oracle/build.py``.  The module exposes the
reference's pybind functions ``create_adam`` / ``adam_update`` / ``destroy_adam``
(patrickstar/ops/csrc/adam/cpu_adam.cpp:751-756) on CPU torch tensors."""
import importlib.util
import os

from . import build


def _cpu_has_avx512():
    try:
        with open("/proc/cpuinfo") as f:
            return "avx512f" in f.read()
    except OSError:
        return False


def available(simd="avx256"):
    return os.path.exists(build.ref_path(simd))


def load(simd=None):
    """Import the compiled reference module.  ``simd``: "avx256", "avx512" or
    None (avx512 when the host CPU has it, else avx256; the two builds give
    bit-identical results).  Raises FileNotFoundError when it was never built."""
    import torch  # noqa: F401  (the module links against libtorch)

    if simd is None:
        simd = "avx512" if (_cpu_has_avx512() and available("avx512")) else "avx256"
    path = build.ref_path(simd)
    if not os.path.exists(path):
        raise FileNotFoundError("%s not built; run `python oracle/build.py` where the reference "
                                "checkout is present" % path)
    name = "cpu_adam_ref_%s" % simd
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
