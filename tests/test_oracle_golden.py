"""The oracle is pinned here: the C restatement and the Python scaler
restatement against golden vectors produced by running the reference
(tests/golden/make_golden.py), and against the compiled reference itself where
it is present (oracle/_ref)."""
import json
import os

import numpy as np
import pytest
import torch

from helpers import checksum, config0_inputs, n_bit_mismatch
from oracle import port, ref
from oracle.scaler_oracle import DynamicScalerOracle, scaler_from_config


def _cases(golden_dir):
    z = np.load(os.path.join(golden_dir, "adam_cases.npz"))
    meta = json.loads(bytes(z["meta"]).decode())
    return z, meta


def _run_port(z, c):
    k = c["key"]
    p, m, v = z[k + "_p0"].copy(), z[k + "_m0"].copy(), z[k + "_v0"].copy()
    o = port.OracleAdam(c["lr"], c["betas"][0], c["betas"][1], c["eps"], c["wd"], c["adamw"])
    for i, s in enumerate(c["steps"]):
        g = z["%s_g%d" % (k, i)]
        if c["hist"] == "seq":
            o.adam_update(s, c["lr"], *c["betas"], c["eps"], c["wd"], True, p, g, m, v, c["scale"])
        else:
            h = c["n"] // 2
            for sl in (slice(0, h), slice(h, None)):
                pp, mm, vv = p[sl].copy(), m[sl].copy(), v[sl].copy()
                o.adam_update(s, c["lr"], *c["betas"], c["eps"], c["wd"], True, pp,
                              np.ascontiguousarray(g[sl]), mm, vv, c["scale"])
                p[sl], m[sl], v[sl] = pp, mm, vv
    return p, m, v


def test_port_matches_reference_golden_vectors(golden_dir):
    z, meta = _cases(golden_dir)
    assert len(meta) == 32
    for c in meta:
        p, m, v = _run_port(z, c)
        k = c["key"]
        assert n_bit_mismatch(p, z[k + "_p"]) == 0, c
        assert n_bit_mismatch(m, z[k + "_m"]) == 0, c
        assert n_bit_mismatch(v, z[k + "_v"]) == 0, c


def test_scaler_oracle_matches_reference_trajectories(golden_dir):
    with open(os.path.join(golden_dir, "scaler_traj.json")) as f:
        cases = json.load(f)
    assert len(cases) == 24
    for c in cases:
        s = DynamicScalerOracle(**c["config"])
        for ov, want in zip(c["overflow"], c["traj"]):
            s.update_scale(bool(ov))
            got = [float(s.cur_scale), s.cur_iter, s.last_overflow_iter, s.cur_hysteresis]
            assert got == want, (c["config"], c["pattern"])


def test_scaler_from_config_quirks():
    # engine.py:90-97: "hysteresis" lands in scale_factor, delayed_shift stays 1
    s = scaler_from_config({"fp16": {"enabled": True, "loss_scale": 0, "initial_scale_power": 3,
                                     "loss_scale_window": 1000, "hysteresis": 2, "min_loss_scale": 1}})
    assert (s.cur_scale, s.scale_factor, s.scale_window, s.min_scale, s.delayed_shift) == (8, 2, 1000, 1, 1)
    for _ in range(3):
        s.update_scale(True)
    assert s.cur_scale == 1
    s.update_scale(True)
    assert s.cur_scale == 1  # pinned at min_scale
    d = scaler_from_config({"fp16": {"enabled": True, "loss_scale": 0}})
    assert (d.cur_scale, d.scale_window) == (2 ** 16, 2000)
    st = scaler_from_config({"fp16": {"enabled": True, "loss_scale": 128}})
    assert st.loss_scale == 128 and not st.dynamic
    assert scaler_from_config({}) is None
    with pytest.raises(AssertionError):
        scaler_from_config({"fp16": {"enabled": False, "loss_scale": 0}})
    with pytest.raises(AssertionError):
        scaler_from_config({"fp16": {"enabled": True}})


def test_port_helpers():
    x = torch.tensor([0.1, -2.5, 65504.0, 65520.0, 1e-8, float("inf")])
    out = np.zeros(6, dtype=np.uint16)
    port.cast_fp32_to_fp16(x.numpy(), out)
    assert (out.view(np.float16) == x.half().numpy()).all()
    g = torch.randn(1000).half().numpy()
    assert not port.has_inf_or_nan_f16(g.view(np.uint16))
    for bad in (np.inf, -np.inf, np.nan):
        h = g.copy()
        h[777] = bad
        assert port.has_inf_or_nan_f16(h.view(np.uint16))
        # the reference's own formulation (loss_scaler.py:138-153)
        s = float(torch.from_numpy(h).float().sum())
        assert s in (float("inf"), -float("inf")) or s != s
    h = (torch.randn(4096) * 100).half()
    want = (h.float() / 8).half()
    a = h.numpy().copy()
    port.div_world_f16(a.view(np.uint16), 8)
    assert (a.view(np.uint16) == want.numpy().view(np.uint16)).all()


@pytest.mark.skipif(not ref.available("avx256"), reason="compiled reference (oracle/_ref) not present")
def test_port_matches_compiled_reference_random():
    mod = ref.load("avx256")
    gen = torch.Generator().manual_seed(99)
    oid = 4000
    for n in (16, 4096, 65536 + 32):
        for adamw, wd in ((False, 0.0), (False, 0.02), (True, 0.0), (True, 0.02)):
            for ghalf in (True, False):
                p = torch.randn(n, generator=gen) * 0.02
                m = torch.randn(n, generator=gen) * 1e-4
                v = (torch.randn(n, generator=gen) * 1e-6).abs()
                pr, mr, vr = p.clone(), m.clone(), v.clone()
                o = port.OracleAdam(2e-3, 0.8, 0.99, 1e-7, wd, adamw)
                mod.create_adam(oid, 2e-3, 0.8, 0.99, 1e-7, wd, adamw, False)
                for step in (1, 2, 3, 7, 8):  # 3 -> 7 breaks the running product
                    g = torch.randn(n, generator=gen) * 1e-3 * 64
                    g = g.half() if ghalf else g
                    o.adam_update(step, 2e-3, 0.8, 0.99, 1e-7, wd, True, p, g, m, v, 64.0)
                    mod.adam_update(oid, step, 2e-3, 0.8, 0.99, 1e-7, wd, True, pr, g.clone(), mr, vr, 64.0)
                mod.destroy_adam(oid)
                oid += 1
                assert n_bit_mismatch(p.numpy(), pr.numpy()) == 0
                assert n_bit_mismatch(m.numpy(), mr.numpy()) == 0
                assert n_bit_mismatch(v.numpy(), vr.numpy()) == 0


@pytest.mark.skipif(not ref.available("avx256") or not ref.available("avx512"),
                    reason="both compiled reference builds needed")
def test_reference_avx_builds_agree():
    if not ref._cpu_has_avx512():
        pytest.skip("host CPU has no AVX-512")
    a, b = ref.load("avx256"), ref.load("avx512")
    p, m, v, grads = config0_inputs(1 << 16)
    pa, ma, va = p.clone(), m.clone(), v.clone()
    a.create_adam(5000, 1e-3, 0.9, 0.999, 1e-6, 0.0, False, False)
    b.create_adam(5000, 1e-3, 0.9, 0.999, 1e-6, 0.0, False, False)
    for i, g in enumerate(grads):
        a.adam_update(5000, 10 + i, 1e-3, 0.9, 0.999, 1e-6, 0.0, True, pa, g, ma, va, 8.0)
        b.adam_update(5000, 10 + i, 1e-3, 0.9, 0.999, 1e-6, 0.0, True, p, g, m, v, 8.0)
    assert n_bit_mismatch(pa.numpy(), p.numpy()) == 0 and n_bit_mismatch(va.numpy(), v.numpy()) == 0


def test_port_full_chunk_checksums_match_reference(golden_dir):
    """Single-chunk 64 Mi-element case, 5 steps: the port's results have the bit
    checksums the reference build produced."""
    with open(os.path.join(golden_dir, "config0_checksums.json")) as f:
        gold = json.load(f)
    n = gold["n"]
    p, m, v, grads = config0_inputs(n)
    if checksum(p) != gold["inputs"]["p"] or checksum(grads[0]) != gold["inputs"]["g"][0]:
        pytest.skip("this torch build draws a different random stream than the fixture's")
    o = port.OracleAdam(1e-3, 0.9, 0.999, 1e-6, 0.0, False)
    for i, g in enumerate(grads):
        o.adam_update(10 + i, 1e-3, 0.9, 0.999, 1e-6, 0.0, True, p, g, m, v, 8.0)
        want = gold["steps"][i]
        assert checksum(p) == want["p"] and checksum(m) == want["m"] and checksum(v) == want["v"]
        assert checksum(p.half()) == want["p16"]
