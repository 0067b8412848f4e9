"""The C-ABI library loads and exports every symbol include/ps_b200.h declares;
host-only entry points behave (no compute call is made here: no GPU needed)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from patrickstar_b200 import build
    build.build()
    from patrickstar_b200 import _lib
    return _lib


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ps_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ps_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(L):
    names = declared_functions()
    assert len(names) >= 20
    raw = C.CDLL(L.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), "symbol %s declared in ps_b200.h is not exported" % n
        assert n in L.SIGNATURES, "symbol %s has no ctypes signature in _lib.py" % n
    for n in L.SIGNATURES:
        assert n in names, "%s bound in _lib.py but not declared in ps_b200.h" % n


def test_struct_sizes_match_header_constants(L):
    text = open(os.path.join(ROOT, "include", "ps_b200.h")).read()
    assert int(re.search(r"#define PS_MAX_GROUPS (\d+)", text).group(1)) == L.PS_MAX_GROUPS
    assert int(re.search(r"#define PS_STATIC_MAX_CHUNKS (\d+)", text).group(1)) == L.PS_STATIC_MAX_CHUNKS
    assert int(re.search(r"#define PS_STATIC_MAX_SEGMENTS (\d+)", text).group(1)) == L.PS_STATIC_MAX_SEGMENTS
    assert C.sizeof(L.StepCtrl) == 48 + 64 * (L.PS_MAX_GROUPS + 1)


def test_host_only_entry_points(L):
    lib = L.lib
    assert lib.ps_version() >= 100
    assert lib.ps_strerror(0) == b"ok"
    assert b"unknown optimizer" in lib.ps_strerror(L.PS_ERR_UNKNOWN_ID)
    assert lib.ps_adam_create(4242, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, 0) == 0
    out = (C.c_float * 4)()
    step = C.c_uint64()
    assert lib.ps_adam_get_state(4242, out, C.byref(step)) == 0
    assert (out[0], out[1], step.value) == (1.0, 1.0, 0)
    assert lib.ps_adam_destroy(4242) == 0
    assert lib.ps_adam_destroy(4242) == L.PS_ERR_UNKNOWN_ID
    assert lib.ps_adam_get_state(4242, out, C.byref(step)) == L.PS_ERR_UNKNOWN_ID
    assert lib.ps_tune(b"unroll", 3) == L.PS_ERR_INVALID
    assert lib.ps_tune(b"nonsense", 1) == L.PS_ERR_INVALID
    assert lib.ps_tune(b"unroll", 2) == 0


def test_pow_table_is_the_libm_pow_of_the_reference(L):
    """IncrementStep's pow branch: float(pow(double(float beta), step))
    (patrickstar/ops/csrc/includes/cpu_adam.h:147-156)."""
    import math
    tab = np.zeros((300, 2), dtype=np.float32)
    assert L.lib.ps_pow_table_fill(0.9, 0.999, 0, 300, tab.ctypes.data) == 0
    b1, b2 = float(np.float32(0.9)), float(np.float32(0.999))
    for t in (0, 1, 2, 10, 150, 299):
        assert tab[t, 0] == np.float32(math.pow(b1, t))
        assert tab[t, 1] == np.float32(math.pow(b2, t))


def test_host_clock_matches_oracle_history(L):
    """ps_adam_update advances the optimizer's beta^t history before it looks at
    the tensors (as ds_adam_step does); with n == 0 that is all it does, so the
    host state machine can be compared with the oracle's without a GPU."""
    from oracle import port
    lib = L.lib
    seq = [(1, 0.9, 0.999), (2, 0.9, 0.999), (2, 0.9, 0.999), (3, 0.9, 0.999), (7, 0.9, 0.999),
           (8, 0.9, 0.999), (8, 0.8, 0.99), (9, 0.8, 0.99), (9, 0.9, 0.999), (10, 0.9, 0.999)]
    o = port.OracleAdam(1e-3, 0.9, 0.999, 1e-8, 0.0, True)
    assert lib.ps_adam_create(4343, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, 0) == 0
    empty32 = np.zeros(0, dtype=np.float32)
    empty16 = np.zeros(0, dtype=np.float16)
    out = (C.c_float * 4)()
    step = C.c_uint64()
    for s, b1, b2 in seq:
        o.adam_update(s, 1e-3, b1, b2, 1e-8, 0.0, True, empty32, empty16, empty32, empty32, -1)
        assert lib.ps_adam_update(4343, s, 1e-3, b1, b2, 1e-8, 0.0, 1, None, None, None, None, 0, 1, -1.0,
                                  None, None) == 0
        assert lib.ps_adam_get_state(4343, out, C.byref(step)) == 0
        st = o.state()
        got = [np.float32(x) for x in out]
        want = [np.float32(st[k]) for k in ("betta1_t", "betta2_t", "bias_correction1", "bias_correction2")]
        assert got == want and step.value == st["step"], (s, b1, b2)
    lib.ps_adam_destroy(4343)


def test_compute_entry_points_refuse_without_arguments(L):
    lib = L.lib
    assert lib.ps_overflow_scan(None, 1, 16, None, None) == L.PS_ERR_INVALID
    assert lib.ps_chunk_step(None, 1, 16, None, None, None) == L.PS_ERR_INVALID
    assert lib.ps_step_begin(None, None, None, None, None, 0, None) == L.PS_ERR_INVALID
    assert lib.ps_adam_update(123456, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, None, None, None, None, 0, 1, -1.0,
                              None, None) == L.PS_ERR_UNKNOWN_ID


def test_package_import_is_lazy_and_fails_loudly_without_library(tmp_path, monkeypatch):
    """No fallback: with the shared library missing, importing a compute name raises."""
    from patrickstar_b200 import _lib
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "missing.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib._load()


def test_table_check_looks_at_the_first_element_field(L):
    """Host-only: ps_chunk_desc.reserved (first element of a piece) must be a
    multiple of 2048 and lie below numel."""
    d = np.zeros(1, dtype=L.CHUNK_DESC_DTYPE)
    s = np.zeros(1, dtype=L.SEGMENT_DTYPE)
    d["p32"], d["exp_avg"], d["exp_avg_sq"], d["h16"] = 256, 512, 768, 1024
    d["numel"], d["seg_begin"], d["seg_end"] = 8192, 0, 1
    s["start"], s["end"], s["slot"] = 0, 8192, 0
    chk = lambda: L.lib.ps_table_check(d.ctypes.data, 1, s.ctypes.data, 1, 1, 8192)
    assert chk() == 0
    for bad in (1, 8, 2047, 2056, 8192, 10240):
        d["reserved"] = bad
        assert chk() == L.PS_ERR_TABLE, bad
    for good in (0, 2048, 6144):
        d["reserved"] = good
        assert chk() == 0, good
    # the allocation-free entry point takes whole chunks only and says so before it touches a device
    d["reserved"] = 2048
    slots = (L.HyperSlot * 1)()
    rc = L.lib.ps_chunk_step_static(d.ctypes.data, 1, 8192, s.ctypes.data, 1, C.cast(slots, C.c_void_p), 1, 0, None)
    assert rc == L.PS_ERR_TABLE


def test_piece_table_check(L):
    """Host-only: descriptors of a piece [reserved, numel) of a chunk."""
    d = np.zeros(2, dtype=L.CHUNK_DESC_DTYPE)
    d["p32"], d["exp_avg"], d["exp_avg_sq"], d["h16"] = 256, 512, 768, 1024
    d["numel"], d["reserved"] = [2048, 5000], [0, 4096]
    d["seg_begin"], d["seg_end"] = 0, 3
    chk = lambda: L.lib.ps_piece_table_check(d.ctypes.data, 2, 3, 8192)
    assert chk() == 0
    d["reserved"][1] = 4100
    assert chk() == L.PS_ERR_TABLE
    d["reserved"][1] = 6144
    assert chk() == L.PS_ERR_TABLE      # at or beyond numel
    d["reserved"][1] = 4096
    d["seg_end"][0] = 4
    assert chk() == L.PS_ERR_TABLE      # segment range outside the table
    d["seg_end"][0] = 3
    d["exp_avg"][1] = 520
    assert chk() == L.PS_ERR_ALIGN


def test_tuning_knobs_accept_only_their_values(L):
    """ps_tune: every knob takes its documented values and refuses others."""
    ok = {"unroll": (1, 2, 4), "scan_unroll": (1, 2, 4), "blocks_per_sm": (0, 2, 32), "bulk": (0, 2, 3, 4),
          "fused_depth": (2, 4, 8), "fused_min_blocks": (2, 3, 4), "fused_blocks_per_sm": (0, 4),
          "pull_blocks_per_sm": (1, 2), "staged_blocks_per_sm": (1, 2), "p2p_unroll": (0, 1, 2),
          "p2p_min_blocks": (2, 3, 4), "p2p_blocks_per_sm": (0, 4)}
    bad = {"unroll": (0, 3), "bulk": (1, 5), "fused_depth": (1, 3, 16), "fused_min_blocks": (1, 5), "p2p_unroll": (3,),
           "blocks_per_sm": (-1, 33)}
    defaults = {"unroll": 2, "scan_unroll": 4, "blocks_per_sm": 0, "bulk": 0, "fused_depth": 4, "fused_min_blocks": 2,
                "fused_blocks_per_sm": 0, "pull_blocks_per_sm": 2, "staged_blocks_per_sm": 1, "p2p_unroll": 0,
                "p2p_min_blocks": 2, "p2p_blocks_per_sm": 0}
    try:
        for key, values in ok.items():
            for v in values:
                assert L.lib.ps_tune(key.encode(), v) == 0, (key, v)
        for key, values in bad.items():
            for v in values:
                assert L.lib.ps_tune(key.encode(), v) == L.PS_ERR_INVALID, (key, v)
        assert L.lib.ps_tune(b"no_such_knob", 1) == L.PS_ERR_INVALID
        assert L.lib.ps_tune(None, 1) == L.PS_ERR_INVALID
    finally:
        for key, v in defaults.items():
            assert L.lib.ps_tune(key.encode(), v) == 0
