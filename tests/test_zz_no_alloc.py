"""ps_chunk_step_static — the chunk step for callers that may not allocate.

Some users of this library cannot call cudaMalloc: a chunk manager that owns
the whole GPU through its own pool and accounts for every byte, or a caller on
a path where cudaMalloc's device-wide synchronisation is not acceptable.  They
have no device memory for the tables ps_chunk_step reads, so this entry point
stages them from host memory into an array inside the library.  The test calls
it through the C ABI twice in a row on one copy of the data, runs the regular
entry points (ps_step_begin + ps_chunk_step) on an identical copy, and demands
bit-equal fp32 master / momentum / variance and fp16 params — the same bar as
the other chunk-step tests.  The second call also proves that nothing stale
from the first one survives in the shared array (it uses fewer chunks, other
segments and a skip step).

Collected last on purpose (file name), so a run that stops at the first failure
has already run everything else.  Passes alone in a fresh process too.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tables(chunks, segs):
    from patrickstar_b200._lib import CHUNK_DESC_DTYPE, SEGMENT_DTYPE
    d = np.zeros(len(chunks), dtype=CHUNK_DESC_DTYPE)
    for i, (p, m, v, h, numel, sb, se) in enumerate(chunks):
        d[i] = (p.data_ptr(), m.data_ptr(), v.data_ptr(), h.data_ptr(), numel, sb, se, 0)
    s = np.zeros(len(segs), dtype=SEGMENT_DTYPE)
    for i, (a, b, slot) in enumerate(segs):
        s[i] = (a, b, slot, 0)
    return d, s


def _regular_step(lib, L, d, s, max_numel, plan, ctrl_dev, scaler_dev, flag_dev, pow_dev, pow_len, stream):
    """The existing path: tables uploaded to device memory, ps_step_begin, ps_chunk_step."""
    d_dev = torch.from_numpy(d.view(np.uint8).copy()).to(DEV)
    s_dev = torch.from_numpy(s.view(np.uint8).copy()).to(DEV)
    L.check(lib.ps_step_begin(ctrl_dev.data_ptr(), scaler_dev.data_ptr(), flag_dev.data_ptr(), C.byref(plan),
                              pow_dev.data_ptr(), pow_len, stream), "ps_step_begin")
    L.check(lib.ps_chunk_step(d_dev.data_ptr(), len(d), max_numel, s_dev.data_ptr(), ctrl_dev.data_ptr(),
                              stream), "ps_chunk_step")
    out = L.StepCtrl()
    L.check(lib.ps_ctrl_read(ctrl_dev.data_ptr(), C.byref(out), stream), "ps_ctrl_read")
    return out


def test_static_variant_matches_regular_entry_point_twice():
    from patrickstar_b200 import _lib as L
    lib = L.lib
    stream = C.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)
    cs = 50000
    gen = torch.Generator().manual_seed(77)

    def make_set():
        out = []
        for _ in range(3):
            p = torch.randn(cs, generator=gen) * 0.02
            m = torch.randn(cs, generator=gen) * 1e-4
            v = (torch.randn(cs, generator=gen) * 1e-6).abs()
            out.append((p, m, v))
        return out

    host = make_set()
    A = [[t.to(DEV) for t in c] + [torch.zeros(cs, dtype=torch.float16, device=DEV)] for c in host]
    B = [[t.clone() for t in c] for c in A]

    # regular path state: control block, dynamic scaler (scale 16), flag, pow table
    ctrl_dev = torch.zeros(C.sizeof(L.StepCtrl), dtype=torch.uint8, device=DEV)
    scaler_dev = torch.zeros(C.sizeof(L.ScalerState), dtype=torch.uint8, device=DEV)
    flag_dev = torch.zeros(1, dtype=torch.int32, device=DEV)
    L.check(lib.ps_ctrl_init(ctrl_dev.data_ptr(), 0, 0.9, 0.999, stream), "ps_ctrl_init")
    init = L.ScalerState(cur_scale=16.0, scale_factor=2.0, min_scale=1.0, cur_iter=0, last_overflow_iter=-1,
                         scale_window=1000, delayed_shift=1, cur_hysteresis=1, consecutive_hysteresis=0,
                         dynamic=1)
    L.check(lib.ps_scaler_init(scaler_dev.data_ptr(), C.byref(init), stream), "ps_scaler_init")
    pow_host = np.zeros((2, 64, 2), dtype=np.float32)
    for g, (b1, b2) in enumerate(((0.9, 0.999), (0.8, 0.99))):
        L.check(lib.ps_pow_table_fill(b1, b2, 0, 64, pow_host[g].ctypes.data), "ps_pow_table_fill")
    pow_dev = torch.from_numpy(pow_host).to(DEV)
    plan = L.StepPlan()
    plan.groups[0] = L.GroupHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-6, weight_decay=0.01, adamw_mode=1)
    plan.groups[1] = L.GroupHyper(lr=2e-3, beta1=0.8, beta2=0.99, eps=1e-8, weight_decay=0.0, adamw_mode=1)
    plan.n_groups, plan.first_group, plan.last_group, plan.n_calls = 2, 0, 1, 5
    plan.grad_divisor, plan.bias_correction, plan.clip = 0.0, 1, 0.0

    def grads(n_chunks, poison=False):
        gs = [(torch.randn(cs, generator=gen) * 1e-3 * 16).half() for _ in range(n_chunks)]
        if poison:
            gs[0][123] = float("nan")
        return gs

    # Nothing may be allocated by the two calls below: neither through torch's pool
    # (memory_allocated / memory_reserved) nor behind its back (cudaMemGetInfo).  The
    # first-call set-up (symbol address look-up) is made here, before the baseline.
    warm_d, warm_s = _tables([(A[0][0], A[0][1], A[0][2], A[0][3], 0, 0, 0)], [(0, 1, 0)])
    warm_slots = (L.HyperSlot * 1)()
    L.check(lib.ps_chunk_step_static(warm_d.ctypes.data, 1, 16, warm_s.ctypes.data, 1,
                                     C.cast(warm_slots, C.c_void_p), 1, 1, stream), "warm-up")
    torch.cuda.synchronize()
    seen = []

    def mem_probe():
        return (torch.cuda.memory_allocated(DEV), torch.cuda.memory_reserved(DEV), torch.cuda.mem_get_info(DEV)[0])

    # ---- call 1: three chunks, two groups, ragged segments ---------------------
    segs1 = [(0, 20001, 0), (20001, 49999, 2),      # chunk 0 (first piece -> slot 0)
             (0, 7, 2), (7, 50000, 1),               # chunk 1
             (16, 40000, 1)]                         # chunk 2: a hole before 16 and after 40000
    ranges1 = [(0, 2), (2, 4), (4, 5)]
    numels1 = [49999, 50000, 40000]
    gs = grads(3)
    for X in (A, B):
        for k in range(3):
            X[k][3].copy_(gs[k])
    dA, sA = _tables([(A[k][0], A[k][1], A[k][2], A[k][3], numels1[k], *ranges1[k]) for k in range(3)], segs1)
    ctrl = _regular_step(lib, L, dA, sA, max(numels1), plan, ctrl_dev, scaler_dev, flag_dev, pow_dev, 64, stream)
    assert ctrl.skip == 0 and ctrl.step == 1
    dB, sB = _tables([(B[k][0], B[k][1], B[k][2], B[k][3], numels1[k], *ranges1[k]) for k in range(3)], segs1)
    slots = (L.HyperSlot * 3)(*[ctrl.slots[i] for i in range(3)])
    # tables in PINNED host memory, overwritten the moment the call returns: the entry point
    # must have taken its copy by then (a caller with its own pool keeps tables pinned)
    dB_pin = torch.from_numpy(dB.view(np.uint8).copy()).pin_memory()
    sB_pin = torch.from_numpy(sB.view(np.uint8).copy()).pin_memory()
    slots_pin = torch.frombuffer(bytearray(bytes(slots)), dtype=torch.uint8).pin_memory()
    torch.cuda.synchronize()
    before = mem_probe()
    L.check(lib.ps_chunk_step_static(dB_pin.data_ptr(), 3, max(numels1), sB_pin.data_ptr(), len(segs1),
                                     slots_pin.data_ptr(), 3, 0, stream), "ps_chunk_step_static")
    dB_pin.fill_(0xFF), sB_pin.fill_(0xFF), slots_pin.fill_(0xFF)
    torch.cuda.synchronize()
    seen.append((before, mem_probe()))
    for k in range(3):
        for j in range(4):
            assert torch.equal(A[k][j].view(torch.uint8), B[k][j].view(torch.uint8)), ("call 1", k, j)

    # ---- call 2, right after: two chunks, other segments, an overflow (skip) step ----
    segs2 = [(0, 50000, 0), (8, 30000, 2)]
    ranges2 = [(0, 1), (1, 2)]
    numels2 = [50000, 30000]
    plan.n_calls, plan.last_group = 2, 1
    gs = grads(2, poison=True)
    for X in (A, B):
        for k in range(2):
            X[k][3].copy_(gs[k])
    dA, sA = _tables([(A[k][0], A[k][1], A[k][2], A[k][3], numels2[k], *ranges2[k]) for k in range(2)], segs2)
    dA_dev = torch.from_numpy(dA.view(np.uint8).copy()).to(DEV)
    L.check(lib.ps_overflow_scan(dA_dev.data_ptr(), 2, max(numels2), flag_dev.data_ptr(), stream), "scan")
    ctrl = _regular_step(lib, L, dA, sA, max(numels2), plan, ctrl_dev, scaler_dev, flag_dev, pow_dev, 64, stream)
    assert ctrl.skip == 1 and ctrl.step == 1  # the poisoned step is skipped
    dB, sB = _tables([(B[k][0], B[k][1], B[k][2], B[k][3], numels2[k], *ranges2[k]) for k in range(2)], segs2)
    torch.cuda.synchronize()
    before = mem_probe()
    L.check(lib.ps_chunk_step_static(dB.ctypes.data, 2, max(numels2), sB.ctypes.data, len(segs2),
                                     C.cast(slots, C.c_void_p), 3, int(ctrl.skip), stream),
            "ps_chunk_step_static")
    torch.cuda.synchronize()
    seen.append((before, mem_probe()))
    for k in range(3):
        for j in range(4):
            assert torch.equal(A[k][j].view(torch.uint8), B[k][j].view(torch.uint8)), ("call 2", k, j)
    # the skip restored fp16 params from the master inside the segments only
    assert torch.equal(B[0][3].view(torch.int16), B[0][0].half().view(torch.int16))
    assert torch.equal(B[1][3][8:30000].view(torch.int16), B[1][0][8:30000].half().view(torch.int16))
    assert torch.isnan(gs[0][123]) and not torch.isnan(B[0][3][123])
    # the property in the entry point's name: no device memory appeared or went away
    for before, after in seen:
        assert after[0] == before[0] and after[1] == before[1], (before, after)
        assert after[2] >= before[2], ("free device memory shrank across the call", before, after)


def test_static_variant_rejects_sizes_beyond_its_maximum():
    from patrickstar_b200 import _lib as L
    lib = L.lib
    d = np.zeros(L.PS_STATIC_MAX_CHUNKS + 1, dtype=L.CHUNK_DESC_DTYPE)
    s = np.zeros(1, dtype=L.SEGMENT_DTYPE)
    slots = (L.HyperSlot * 1)()
    rc = lib.ps_chunk_step_static(d.ctypes.data, L.PS_STATIC_MAX_CHUNKS + 1, 16, s.ctypes.data, 1,
                                  C.cast(slots, C.c_void_p), 1, 0, None)
    assert rc == L.PS_ERR_LIMIT
    s2 = np.zeros(L.PS_STATIC_MAX_SEGMENTS + 1, dtype=L.SEGMENT_DTYPE)
    rc = lib.ps_chunk_step_static(d.ctypes.data, 1, 16, s2.ctypes.data, L.PS_STATIC_MAX_SEGMENTS + 1,
                                  C.cast(slots, C.c_void_p), 1, 0, None)
    assert rc == L.PS_ERR_LIMIT
    assert b"maximum" in lib.ps_strerror(rc)
