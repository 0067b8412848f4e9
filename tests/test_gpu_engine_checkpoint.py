"""Drop-in surface on a small model: initialize_engine -> forward / backward / step,
and optimizer checkpoint round trip (modelled on the reference's
unitest/test_optimizer_init.py and unitest/test_checkpoint.py:116-180)."""
import copy

import numpy as np
import pytest
import torch

from helpers import n_bit_mismatch
from oracle.scaler_oracle import DynamicScalerOracle
from oracle.step_oracle import StepOracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CONFIG = {
    "optimizer": {"type": "Adam", "params": {"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-6,
                                             "weight_decay": 0, "use_hybrid_adam": True}},
    "fp16": {"enabled": True, "loss_scale": 0, "initial_scale_power": 10, "loss_scale_window": 1000,
             "hysteresis": 2, "min_loss_scale": 1},
    "default_chunk_size": 4096,
}


def model_func():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(32, 48), torch.nn.Tanh(), torch.nn.Linear(48, 16))


def test_initialize_engine_trains_and_matches_oracle():
    from patrickstar_b200 import DynamicLossScaler, FP16Adam, initialize_engine
    engine, opt = initialize_engine(model_func, 0, CONFIG)
    assert isinstance(opt, FP16Adam) and isinstance(engine.loss_scaler, DynamicLossScaler)
    assert engine.loss_scaler.loss_scale == 1024 and engine.loss_scaler.scale_factor == 2
    client = engine.client
    lay = client.layout
    # the reference's packing: a module's parameters are never split (32*48+48 = 1584, 48*16+16 = 784)
    assert lay.pack == "no_split" and lay.n_data_chunks == 1
    for name, p in engine.module.named_parameters():
        assert p.dtype == torch.float16 and p.data_ptr() == client.fp16_view(lay.tensor(name)).data_ptr()
    n_local = len(client.local_ids)
    P = [client.chunk_state(k)[0].cpu().numpy().copy() for k in range(n_local)]
    M = [np.zeros_like(x) for x in P]
    V = [np.zeros_like(x) for x in P]
    so = DynamicScalerOracle(2 ** 10, 2, 1000, 1)
    calls = [(client.local_ids.index(c.chunk_id), c.start, c.end, c.group) for c in lay.calls_of_rank(0)]
    orc = StepOracle(calls, [{"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-6, "weight_decay": 0}], so, False)
    gen = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn(64, 32, device=DEV, dtype=torch.float16, generator=gen)
    y = torch.randn(64, 16, device=DEV, dtype=torch.float16, generator=gen)
    losses = []
    for it in range(12):
        out = engine(x)
        loss = torch.nn.functional.mse_loss(out.float(), y.float())
        losses.append(float(loss.detach()))
        engine.backward(loss)               # scaled backward + grads into the fp16 slots
        H = [client.fp16_chunk(c).cpu().numpy().copy() for c in client.local_ids]
        opt.step()
        orc.step(H, P, M, V)
        torch.cuda.synchronize()
        for k, c in enumerate(client.local_ids):
            dp, dm, dv = client.chunk_state(k)
            assert n_bit_mismatch(dp.cpu().numpy(), P[k]) == 0, it
            assert n_bit_mismatch(dm.cpu().numpy(), M[k]) == 0, it
            assert n_bit_mismatch(dv.cpu().numpy(), V[k]) == 0, it
            assert n_bit_mismatch(client.fp16_chunk(c).cpu().numpy(), H[k]) == 0, it
    assert losses[-1] < losses[0]
    assert opt.step_count + opt.skipped_steps == 12


def test_constructor_validation_like_the_reference():
    from patrickstar_b200 import ChunkClient, FP16Adam
    c = ChunkClient(rank=0, default_chunk_size=64, world_size=1, device=DEV, pack="flat")
    c.append_tensor("w", 64)
    c.allocate()
    for kw, msg in ((dict(lr=-1.0), "Invalid learning rate"), (dict(eps=-1e-8), "Invalid epsilon"),
                    (dict(betas=(1.0, 0.9)), "index 0"), (dict(betas=(0.9, 1.5)), "index 1"),
                    (dict(weight_decay=-0.1), "Invalid weight_decay")):
        with pytest.raises(ValueError, match=msg):
            FP16Adam(c, c.params.values(), **kw)
    with pytest.raises(ValueError, match="not registered"):
        FP16Adam(c, [torch.nn.Parameter(torch.zeros(4, device=DEV))])


def test_optimizer_checkpoint_round_trip():
    """state_dict / load_state_dict (fp16_cpu_adam.py:630-694) — resuming reproduces
    the uninterrupted run bit for bit, loss-scaler state and beta^t history included
    (both are missing from the reference's checkpoint)."""
    from patrickstar_b200 import ChunkClient, DynamicLossScaler, FP16Adam
    cs = 5000

    def build():
        c = ChunkClient(rank=0, default_chunk_size=cs, world_size=1, device=DEV, pack="flat")
        c.append_tensor_list([("a", 3000, 0), ("b", 4500, 1), ("c", 2000, 0)])
        c.allocate()
        s = DynamicLossScaler(init_scale=64, scale_factor=2, scale_window=4, min_scale=1)
        g0 = [c.params["a"], c.params["c"]]
        o = FP16Adam(c, [{"params": g0, "weight_decay": 0.01}, {"params": [c.params["b"]], "weight_decay": 0.0}],
                     loss_scaler=s, lr=1e-3, use_adamw=True)
        return c, s, o

    def grads(step):
        g = torch.Generator().manual_seed(50 + step)
        x = (torch.randn(2 * cs, generator=g) * 1e-2).half()
        if step == 4:
            x[123] = float("inf")
        return x

    def init(c):
        g = torch.Generator().manual_seed(3)
        for k in range(2):
            for t, sd in zip(c.chunk_state(k), (0.02, 1e-4, 1e-6)):
                t.copy_((torch.randn(cs, generator=g) * sd).abs() if sd == 1e-6 else torch.randn(cs, generator=g) * sd)

    ca, sa, oa = build()
    init(ca)
    for step in range(10):
        ca.fp16[:2 * cs].copy_(grads(step))
        oa.step()
        if step == 5:
            sd = copy.deepcopy(oa.state_dict())
            master = [ca.chunk_state(k)[0].clone() for k in range(2)]
    assert set(sd["state"][0]) >= {"step", "exp_avg", "exp_avg_sq", "betas", "lr", "weight_decay", "eps"}
    assert sd["state"][0]["exp_avg"].shape == (3000,) and sd["state"][0]["step"] == 5  # one of 6 skipped
    # through the on-disk format the reference uses for it (torch.save of the dict)
    import io
    buf = io.BytesIO()
    torch.save(sd, buf)
    buf.seek(0)
    sd = torch.load(buf, weights_only=False)
    cb, sb, ob = build()
    for k in range(2):
        cb.chunk_state(k)[0].copy_(master[k])
    ob.load_state_dict(sd)
    for step in range(6, 10):
        cb.fp16[:2 * cs].copy_(grads(step))
        ob.step()
    torch.cuda.synchronize()
    for k in range(2):
        n_used = ca.layout.chunk_numel(k)   # the checkpoint holds the tensors, not the unused chunk tail
        for ta, tb in zip(ca.chunk_state(k), cb.chunk_state(k)):
            assert torch.equal(ta[:n_used].view(torch.int32), tb[:n_used].view(torch.int32))
        assert torch.equal(ca.fp16_chunk(k)[:n_used].view(torch.int16), cb.fp16_chunk(k)[:n_used].view(torch.int16))
    assert oa.step_count == ob.step_count == 9
    assert sa.read_state().cur_scale == sb.read_state().cur_scale
    assert sa.cur_iter == sb.cur_iter == 10


def test_grad_handoff_copies_and_flags():
    """ps_grad_handoff through the C ABI: bit copy at every alignment, flag set
    exactly when an inf/nan is present (the per-parameter check + copy of the
    reference's backward hook, patrickstar/core/hook.py:212-216)."""
    import ctypes as C
    from patrickstar_b200._lib import check, lib
    stream = C.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)
    gen = torch.Generator().manual_seed(9)
    for n in (0, 1, 7, 8, 9, 1000, 4099, 1 << 18):
        for so, do in ((0, 0), (3, 3), (1, 5), (8, 0), (2, 11)):
            for bad in (None, float("inf"), float("nan"), -float("inf")):
                src = (torch.randn(n + 32, generator=gen) * 10).half()
                pos = None
                if bad is not None and n:
                    pos = int(torch.randint(0, n, (1,), generator=gen))
                    src[so + pos] = bad
                src_d = src.to(DEV)
                dst_d = torch.full((n + 32,), 7.0, dtype=torch.float16, device=DEV)
                flag = torch.zeros(1, dtype=torch.int32, device=DEV)
                check(lib.ps_grad_handoff(src_d.data_ptr() + 2 * so, dst_d.data_ptr() + 2 * do, n, flag.data_ptr(),
                                          stream), "ps_grad_handoff")
                out = dst_d.cpu()
                assert torch.equal(out[do:do + n].view(torch.int16), src[so:so + n].view(torch.int16))
                assert (out[:do] == 7).all() and (out[do + n:] == 7).all()
                assert int(flag.item()) == int(pos is not None), (n, so, do, bad)


def test_engine_step_skips_on_overflow_seen_in_backward():
    from patrickstar_b200 import initialize_engine
    engine, opt = initialize_engine(model_func, 0, CONFIG)
    x = torch.randn(8, 32, device=DEV, dtype=torch.float16)
    before = [client_p.clone() for client_p in engine.client.chunk_state(0)]
    out = engine(x)
    loss = out.float().sum() * float("inf")      # every gradient becomes inf / nan
    engine.backward(loss)
    engine.step()                                 # no second scan: the flag came from the hand-off
    assert opt.skipped_steps == 1 and opt.step_count == 0
    assert engine.loss_scaler.loss_scale == 512
    for a, b in zip(before, engine.client.chunk_state(0)):
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    # the skipped step restored the fp16 params from the master
    for name, p in engine.module.named_parameters():
        assert torch.isfinite(p).all()
    out = engine(x)
    engine.backward(out.float().pow(2).mean())
    engine.step()
    assert opt.step_count == 1 and opt.skipped_steps == 1
