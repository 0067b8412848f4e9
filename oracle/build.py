"""TEST INFRASTRUCTURE — build recipe for the parity oracle.  Not part of the product.

Two artefacts, both written under ``oracle/_ref/`` (git-ignored):

* ``libps_oracle.so`` — this repository's plain-C restatement of the reference
  CPU Adam (``oracle/adam_oracle.c``), built with ``gcc``.
* ``cpu_adam_ref_avx256.so`` / ``cpu_adam_ref_avx512.so`` — the reference's own
  ``patrickstar/ops/csrc/adam/cpu_adam.cpp`` compiled unmodified from where it
  lies in the reference checkout (no source is copied), as the torch/pybind
  extension module it is, with the SIMD define forced (the reference's builder,
  ``patrickstar/ops/op_builder/builder.py:312-328``, would pick the
  non-bit-identical scalar path on a non-Intel host) and ``-std=c++17``
  instead of the reference's ``-std=c++14`` (``op_builder/cpu_adam.py:74``)
  because current torch headers need it.  ``ref_link_stubs.cpp`` replaces the
  cuBLAS/cuRAND/stream calls of the reference's ``Context`` singleton at link
  time so the module can be constructed on a host without a GPU.

The reference checkout is only present on the build machine; elsewhere the
prebuilt files are used as they are and ``build_ref`` is a no-op.

Run ``python oracle/build.py`` to build everything that can be built.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# the reference checkout: $PS_REFERENCE_ROOT, else a directory "reference" beside this repository
REFERENCE_ROOT = os.environ.get("PS_REFERENCE_ROOT",
                                os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
REF_CSRC = os.path.join(REFERENCE_ROOT, "patrickstar", "ops", "csrc")

_SIMD = {
    "avx256": ["-mavx2", "-mfma", "-mf16c", "-D__AVX256__"],
    "avx512": ["-mavx512f", "-mavx2", "-mfma", "-mf16c", "-D__AVX512__"],
}


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: %s\n%s" % (" ".join(cmd), r.stderr[-4000:]))


def port_path():
    return os.path.join(OUT, "libps_oracle.so")


def ref_path(simd):
    return os.path.join(OUT, "cpu_adam_ref_%s.so" % simd)


def build_port(force=False):
    """gcc build of the C restatement.  -ffp-contract=off: every rounding in the
    source is the one that is executed (fused multiply-adds are spelled fmaf)."""
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(HERE, "adam_oracle.c")
    out = port_path()
    if force or _stale(out, [src]):
        _run(["gcc", "-O3", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-mavx2", "-mfma",
              "-mf16c", "-ffp-contract=off", "-fno-fast-math", src, "-o", out, "-lm"])
    return out


def reference_available():
    return os.path.exists(os.path.join(REF_CSRC, "adam", "cpu_adam.cpp"))


def build_ref(simd="avx256", force=False):
    """Compile the reference's cpu_adam.cpp in place into oracle/_ref/.  Returns
    the path of the built module, or None when the reference checkout is absent
    and nothing was prebuilt."""
    out = ref_path(simd)
    if not reference_available():
        return out if os.path.exists(out) else None
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(REF_CSRC, "adam", "cpu_adam.cpp")
    stubs = os.path.join(HERE, "ref_link_stubs.cpp")
    hdrs = [os.path.join(REF_CSRC, "includes", h) for h in ("cpu_adam.h", "context.h")]
    if not (force or _stale(out, [src, stubs] + hdrs)):
        return out
    from torch.utils import cpp_extension as ce

    cuda_home = ce.CUDA_HOME or "/usr/local/cuda"
    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    lib = []
    for p in ce.library_paths():
        lib += ["-L" + p, "-Wl,-rpath," + p]
    common = (["-O3", "-std=c++17", "-fPIC", "-fopenmp", "-Wno-reorder", "-g0"] + _SIMD[simd]
              + ["-DTORCH_EXTENSION_NAME=cpu_adam_ref_%s" % simd, "-DTORCH_API_INCLUDE_EXTENSION_H",
                 "-I" + os.path.join(REF_CSRC, "includes"), "-I" + os.path.join(cuda_home, "include"),
                 "-I" + sysconfig.get_paths()["include"]] + inc)
    _run(["g++"] + common + ["-shared", src, stubs, "-o", out, "-Wl,-Bsymbolic"] + lib
         + ["-L" + os.path.join(cuda_home, "lib64"), "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch",
            "-ltorch_python", "-lcudart"])
    return out


def build_all(force=False):
    built = [build_port(force)]
    for simd in ("avx256", "avx512"):
        p = build_ref(simd, force)
        if p:
            built.append(p)
    return built


if __name__ == "__main__":
    for p in build_all(force="--force" in sys.argv):
        print(p)
