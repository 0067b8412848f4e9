"""Parity at the benchmark configurations' full sizes.

The CPU oracle cannot follow 16-24 chunks of 64 Mi elements for many steps in a
test's time, so these tests combine
  * bit-exact comparison with the oracle on the chunks it does follow,
  * size-independent properties over ALL chunks (identical inputs give
    identical bits; fp16 slot == half(fp32 master); every step's skip decision
    and the loss-scale trajectory against the scaler oracle).
"""
import numpy as np
import pytest
import torch

from helpers import checksum, n_bit_mismatch
from oracle.scaler_oracle import DynamicScalerOracle
from oracle.step_oracle import StepOracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CHUNK = 64 * 1024 * 1024


def _free_gib():
    free, _ = torch.cuda.mem_get_info()
    return free / 2 ** 30


def test_dynamic_loss_scale_16_chunks_200_steps():
    """16 chunks x 64 Mi elements, DynamicLossScaler(2^3, window 1000, hysteresis
    key 2, min 1) as initialize_engine builds it, 200 steps, every 17th step a
    seeded injection of 1-8 inf/nan into one random chunk.  All chunks receive
    the same gradients.  Chunk 0 holds the first tensor the optimizer visits in
    a step, which sees another beta^t than the later ones
    (patrickstar/ops/csrc/includes/cpu_adam.h:143-162); chunks 1..15 must stay
    bit-identical to each other.  Chunks 0 and 1 are followed by the oracle for
    all 200 steps."""
    if _free_gib() < 24:
        pytest.skip("needs ~20 GiB of free device memory")
    from patrickstar_b200 import ChunkClient, FP16Adam
    from patrickstar_b200.engine import build_loss_scaler, parse_config
    n_chunks, steps = 16, 200
    cfg = {"optimizer": {"type": "Adam", "params": {"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-6,
                                                     "weight_decay": 0}},
           "fp16": {"enabled": True, "loss_scale": 0, "initial_scale_power": 3, "loss_scale_window": 1000,
                    "hysteresis": 2, "min_loss_scale": 1}, "default_chunk_size": CHUNK}
    parsed = parse_config(cfg)
    client = ChunkClient(rank=0, default_chunk_size=parsed["default_chunk_size"], world_size=1, device=DEV,
                         pack="flat")
    client.append_tensor_list([("w%d" % i, CHUNK, 0) for i in range(n_chunks)])
    client.allocate()
    scaler = build_loss_scaler(parsed, DEV)
    op = parsed["optim_params"]
    opt = FP16Adam(client, client.params.values(), loss_scaler=scaler, lr=op["lr"], betas=op["betas"],
                   eps=op["eps"], weight_decay=op["weight_decay"], use_adamw=False)
    gen = torch.Generator(device=DEV).manual_seed(0)
    p0 = torch.empty(CHUNK, device=DEV).normal_(0, 0.02, generator=gen)
    m0 = torch.empty(CHUNK, device=DEV).normal_(0, 1e-4, generator=gen)
    v0 = torch.empty(CHUNK, device=DEV).normal_(0, 1e-6, generator=gen).abs_()
    for k in range(n_chunks):
        p, m, v = client.chunk_state(k)
        p.copy_(p0), m.copy_(m0), v.copy_(v0)
    P = [p0.cpu().numpy(), p0.cpu().numpy()]
    M = [m0.cpu().numpy(), m0.cpu().numpy()]
    V = [v0.cpu().numpy(), v0.cpu().numpy()]
    del p0, m0, v0
    so = DynamicScalerOracle(2 ** 3, 2, 1000, 1)
    # the oracle follows the first two of the 16 tensors; the others only matter through the
    # beta^t history they leave in the optimizer object (trailing_call_group)
    orc = StepOracle([(0, 0, CHUNK, 0), (1, 0, CHUNK, 0)],
                     [{"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-6, "weight_decay": 0}],
                     so, False, trailing_call_group=0)
    rng = np.random.RandomState(0)
    pinned = torch.empty(CHUNK, dtype=torch.float16).pin_memory()
    second = np.empty(CHUNK, dtype=np.float16)
    tmp = torch.empty(CHUNK, device=DEV)
    skips = []
    for step in range(steps):
        tmp.normal_(0, 1e-3, generator=gen).mul_(float(so.loss_scale))
        g = tmp.half()
        for cid in range(n_chunks):
            client.fp16_chunk(cid).copy_(g)
        inject = step % 17 == 16
        if inject:
            victim = int(rng.randint(n_chunks))
            for pos in rng.randint(0, CHUNK, size=rng.randint(1, 9)):
                client.fp16_chunk(victim)[int(pos)] = float(rng.choice([np.inf, -np.inf, np.nan]))
        pinned.copy_(g)
        torch.cuda.synchronize()
        second[:] = pinned.numpy()
        H = [pinned.numpy(), second]
        opt.step()
        skipped = orc.step(H, P, M, V, overflow=inject)
        skips.append(skipped)
        st = scaler.read_state()  # bit-exact scale trajectory, every step
        assert (st.cur_scale, st.cur_iter, st.last_overflow_iter, st.cur_hysteresis) == \
            (float(so.cur_scale), so.cur_iter, so.last_overflow_iter, so.cur_hysteresis), step
        assert opt.read_ctrl().skip == int(inject), step
    assert sum(skips) == 11 and opt.step_count == steps - 11 == orc.step_count
    assert scaler.loss_scale == 1  # 8 -> 4 -> 2 -> 1, then pinned at min_scale
    torch.cuda.synchronize()
    for k in (0, 1):
        p, m, v = client.chunk_state(k)
        assert n_bit_mismatch(p.cpu().numpy(), P[k]) == 0, k
        assert n_bit_mismatch(m.cpu().numpy(), M[k]) == 0, k
        assert n_bit_mismatch(v.cpu().numpy(), V[k]) == 0, k
        assert n_bit_mismatch(client.fp16_chunk(k).cpu().numpy(), H[k]) == 0, k
    p, m, v = client.chunk_state(1)
    ref = [checksum(t) for t in (p, m, v, client.fp16_chunk(1))]
    for k in range(2, n_chunks):
        pk, mk, vk = client.chunk_state(k)
        assert [checksum(t) for t in (pk, mk, vk, client.fp16_chunk(k))] == ref, k
    assert [checksum(t) for t in client.chunk_state(0)] != ref[:3]  # the first-call quirk is real


def test_gpt2_xl_layout_adamw_two_groups():
    """GPT-2 1.5B (48 layers, hidden 1600, vocab 50257) packed in module order into
    24 chunks of 64 Mi elements, AdamW with weight decay 0.01 on the weights and 0
    on biases / LayerNorm (two param groups whose segments straddle chunk
    boundaries), fp16 grads ~ N(0, 1e-3) * 2^12.  Chunks 0, 1, 12 and 23 are
    followed by the oracle; all chunks are checked for fp16 == half(master)."""
    if _free_gib() < 30:
        pytest.skip("needs ~26 GiB of free device memory")
    from patrickstar_b200 import ChunkClient, FP16Adam, LossScaler
    from patrickstar_b200.model_layouts import model_specs
    specs = model_specs("gpt2_1.5b")
    client = ChunkClient(rank=0, default_chunk_size=CHUNK, world_size=1, device=DEV, pack="flat")
    client.append_tensor_list([(n, int(np.prod(s)), g) for n, s, g in specs], [s for _, s, _ in specs])
    client.allocate()
    lay = client.layout
    assert lay.n_data_chunks == 24
    decay = [client.params[n] for n, _, g in specs if g == 0]
    no_decay = [client.params[n] for n, _, g in specs if g == 1]
    opt = FP16Adam(client, [{"params": decay, "weight_decay": 0.01}, {"params": no_decay, "weight_decay": 0.0}],
                   loss_scaler=LossScaler(2.0 ** 12), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, use_adamw=True)
    followed = [0, 1, 12, 23]
    gen = torch.Generator(device=DEV).manual_seed(2)
    P, M, V = {}, {}, {}
    for k in range(24):
        p, m, v = client.chunk_state(k)
        p.normal_(0, 0.02, generator=gen)
        m.normal_(0, 1e-4, generator=gen)
        v.normal_(0, 1e-6, generator=gen).abs_()
        if k in followed:
            P[k], M[k], V[k] = p.cpu().numpy(), m.cpu().numpy(), v.cpu().numpy()
    calls_all = lay.calls_of_rank(0)
    assert calls_all[0].chunk_id == 0
    idx = {c: i for i, c in enumerate(followed)}
    calls = [(idx[p.chunk_id], p.start, p.end, p.group) for p in calls_all if p.chunk_id in idx]
    assert len({g for _, _, _, g in calls}) == 2 and len(calls) > 40
    groups = [{"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-8, "weight_decay": 0.01},
              {"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-8, "weight_decay": 0.0}]
    from oracle.scaler_oracle import StaticScalerOracle
    orc = StepOracle(calls, groups, StaticScalerOracle(2.0 ** 12), True)
    tmp = torch.empty(CHUNK, device=DEV)
    for step in range(2):
        H = {}
        for k in range(24):
            tmp.normal_(0, 1e-3 * 4096, generator=gen)
            client.fp16_chunk(k).copy_(tmp.half())
            if k in followed:
                H[k] = client.fp16_chunk(k).cpu().numpy()
        opt.step()
        orc.step([H[k] for k in followed], [P[k] for k in followed], [M[k] for k in followed],
                 [V[k] for k in followed])
        torch.cuda.synchronize()
        for k in followed:
            p, m, v = client.chunk_state(k)
            n_used = lay.chunk_numel(k)
            assert n_bit_mismatch(p.cpu().numpy(), P[k]) == 0, (step, k)
            assert n_bit_mismatch(m.cpu().numpy(), M[k]) == 0, (step, k)
            assert n_bit_mismatch(v.cpu().numpy(), V[k]) == 0, (step, k)
            assert n_bit_mismatch(client.fp16_chunk(k)[:n_used].cpu().numpy(), H[k][:n_used]) == 0, (step, k)
        for k in range(24):
            n_used = lay.chunk_numel(k)
            p = client.chunk_state(k)[0]
            assert torch.equal(client.fp16_chunk(k)[:n_used].view(torch.int16), p[:n_used].half().view(torch.int16)), k
    assert opt.step_count == 2
