"""Generates the golden fixtures of tests/golden/ by RUNNING THE REFERENCE.

Needs the reference checkout (PS_REFERENCE_ROOT, default: a directory "reference"
beside this repository) and
the compiled reference module (``python oracle/build.py``).  Run from the
repository root:  ``python tests/golden/make_golden.py``

Outputs
  adam_cases.npz      inputs and outputs of the reference's cpu_adam_op.adam_update
                      (AVX build) for a grid of small cases
  scaler_traj.json    trajectories of the reference's DynamicLossScaler (imported
                      from patrickstar/fp16/loss_scaler.py) under seeded overflow patterns
  config0_checksums.json  bit checksums of p / m / v after each of the 5 steps of the
                      single-chunk 64 Mi-element case, from the reference build
"""
import importlib.util
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE_ROOT = os.environ.get("PS_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))


def checksum(t):
    """(xor, sum mod 2^64) over the 32-bit (or 16-bit) patterns of a tensor."""
    a = t.numpy()
    bits = a.view(np.uint32 if a.dtype.itemsize == 4 else np.uint16)
    return [int(np.bitwise_xor.reduce(bits)), int(bits.astype(np.uint64).sum(dtype=np.uint64))]


def config0_inputs(n, seed=0, steps=5, scale=8.0):
    """Single-chunk case: draws in this order from one CPU generator."""
    g = torch.Generator().manual_seed(seed)
    p = torch.randn(n, generator=g) * 0.02
    m = torch.randn(n, generator=g) * 1e-4
    v = (torch.randn(n, generator=g) * 1e-6).abs()
    grads = [(torch.randn(n, generator=g) * 1e-3 * scale).half() for _ in range(steps)]
    return p, m, v, grads


def adam_cases(mod):
    out = {}
    meta = []
    gen = torch.Generator().manual_seed(1234)
    case = 0
    for adamw in (False, True):
        for wd in (0.0, 0.01):
            for ghalf in (True, False):
                for scale in (8.0, -1.0):
                    for hist in ("seq", "two_calls"):
                        n = 1024
                        p = torch.randn(n, generator=gen) * 0.02
                        m = torch.randn(n, generator=gen) * 1e-4
                        v = (torch.randn(n, generator=gen) * 1e-6).abs()
                        steps = [10, 11, 12] if hist == "seq" else [1, 2, 3]
                        gs = []
                        for _ in steps:
                            g = torch.randn(n, generator=gen) * 1e-3 * (scale if scale > 0 else 1.0)
                            gs.append(g.half() if ghalf else g)
                        key = "c%02d" % case
                        out[key + "_p0"], out[key + "_m0"], out[key + "_v0"] = p.numpy().copy(), m.numpy().copy(), v.numpy().copy()
                        mod.create_adam(100 + case, 1e-3, 0.9, 0.999, 1e-6, wd, adamw, False)
                        for i, (s, g) in enumerate(zip(steps, gs)):
                            out["%s_g%d" % (key, i)] = g.numpy().copy()
                            if hist == "seq":
                                mod.adam_update(100 + case, s, 1e-3, 0.9, 0.999, 1e-6, wd, True, p, g, m, v, scale)
                            else:
                                # two tensors per step on one optimizer object: halves of the arrays
                                h = n // 2
                                mod.adam_update(100 + case, s, 1e-3, 0.9, 0.999, 1e-6, wd, True,
                                                p[:h], g[:h].contiguous(), m[:h], v[:h], scale)
                                mod.adam_update(100 + case, s, 1e-3, 0.9, 0.999, 1e-6, wd, True,
                                                p[h:], g[h:].contiguous(), m[h:], v[h:], scale)
                        mod.destroy_adam(100 + case)
                        out[key + "_p"], out[key + "_m"], out[key + "_v"] = p.numpy().copy(), m.numpy().copy(), v.numpy().copy()
                        meta.append({"key": key, "adamw": adamw, "wd": wd, "ghalf": ghalf, "scale": scale,
                                     "hist": hist, "steps": steps, "n": n, "lr": 1e-3, "betas": [0.9, 0.999],
                                     "eps": 1e-6})
                        case += 1
    out["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    return out


def scaler_trajectories():
    spec = importlib.util.spec_from_file_location(
        "ref_loss_scaler", os.path.join(REFERENCE_ROOT, "patrickstar", "fp16", "loss_scaler.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    cases = []
    rng = np.random.RandomState(7)
    patterns = {
        "every17_200": [(i % 17 == 16) for i in range(200)],
        "random_p10_300": [bool(x) for x in (rng.rand(300) < 0.10)],
        "bursts_120": [(i % 40) in (5, 6, 7) for i in range(120)],
        "none_50": [False] * 50,
    }
    configs = [
        dict(init_scale=2 ** 3, scale_factor=2, scale_window=1000, min_scale=1),
        dict(init_scale=2 ** 16, scale_factor=2, scale_window=20, min_scale=1),
        dict(init_scale=2 ** 16, scale_factor=2.0, scale_window=10, min_scale=4, delayed_shift=2),
        dict(init_scale=2 ** 10, scale_factor=2.0, scale_window=8, min_scale=1, delayed_shift=3,
             consecutive_hysteresis=True),
        dict(init_scale=1000, scale_factor=3, scale_window=7, min_scale=1),
        dict(init_scale=2 ** 32, scale_factor=2.0, scale_window=1000, min_scale=1),
    ]
    for cfg in configs:
        for pname, pat in patterns.items():
            s = mod.DynamicLossScaler(**cfg)
            traj = []
            for ov in pat:
                s.update_scale(ov)
                traj.append([float(s.cur_scale), s.cur_iter, s.last_overflow_iter, s.cur_hysteresis])
            cases.append({"config": cfg, "pattern": pname, "overflow": [int(b) for b in pat], "traj": traj})
    return cases


def config0_checksums(mod):
    n = 64 * 1024 * 1024
    p, m, v, grads = config0_inputs(n)
    res = {"n": n, "inputs": {"p": checksum(p), "m": checksum(m), "v": checksum(v),
                              "g": [checksum(g) for g in grads]}, "steps": []}
    mod.create_adam(900, 1e-3, 0.9, 0.999, 1e-6, 0.0, False, False)
    for i, g in enumerate(grads):
        mod.adam_update(900, 10 + i, 1e-3, 0.9, 0.999, 1e-6, 0.0, True, p, g, m, v, 8.0)
        res["steps"].append({"step": 10 + i, "p": checksum(p), "m": checksum(m), "v": checksum(v),
                             "p16": checksum(p.half()),
                             "sample_idx": [0, 1, 12345, n // 2, n - 1],
                             "sample_p_bits": [int(p.view(torch.int32)[j]) for j in (0, 1, 12345, n // 2, n - 1)]})
    mod.destroy_adam(900)
    return res


def main():
    mod = ref.load("avx256")
    np.savez_compressed(os.path.join(HERE, "adam_cases.npz"), **adam_cases(mod))
    with open(os.path.join(HERE, "scaler_traj.json"), "w") as f:
        json.dump(scaler_trajectories(), f)
    with open(os.path.join(HERE, "config0_checksums.json"), "w") as f:
        json.dump(config0_checksums(mod), f, indent=1)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
