"""In-tree build of the CUDA library: ``python -m patrickstar_b200.build``.

One translation unit, nvcc, sm_100a only.  The output ``libps_b200.so`` sits
beside the package so that it is found without installation.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SOURCES = [os.path.join(HERE, "csrc", "ps_kernels.cu"), os.path.join(HERE, "csrc", "ps_offload.cu")]
HEADER = os.path.join(ROOT, "include", "ps_b200.h")
OUT = os.path.join(HERE, "libps_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # IEEE arithmetic on both sides: no fast-math on the device, no contraction on the host
    "-Xcompiler", "-fPIC,-ffp-contract=off", "-shared",
]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def build(force=False, verbose=False):
    srcs = [s for s in SOURCES if os.path.exists(s)]
    deps = srcs + [HEADER]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps):
        return OUT
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [
        "-I" + os.path.join(ROOT, "include")] + srcs + ["-o", OUT]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), r.stderr[-6000:]))
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
