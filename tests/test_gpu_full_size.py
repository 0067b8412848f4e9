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
    seeded injection of 1-8 inf/nan into one random chunk.  Every chunk has its
    own state and receives its own gradients every step.  Four chunks spread over
    the table are followed by the oracle for all 200 steps, bit for bit: the first
    (its tensor makes the first adam_update call of a step, which sees another
    beta^t than the later ones, patrickstar/ops/csrc/includes/cpu_adam.h:143-162),
    the victim of the first injection, one mid-table chunk and the last.  As an
    extra, chunks 6 and 7 are given identical states and gradients and must stay
    bit-identical to each other; all chunks must end with fp16 == half(master)."""
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
    # the injection plan is drawn up front so that the first victim can be followed
    rng = np.random.RandomState(0)
    plan = {}
    for step in range(steps):
        if step % 17 == 16:
            victim = int(rng.randint(n_chunks))
            where = [int(x) for x in rng.randint(0, CHUNK, size=rng.randint(1, 9))]
            what = [float(rng.choice([np.inf, -np.inf, np.nan])) for _ in where]
            plan[step] = (victim, where, what)
    first_victim = plan[16][0]
    followed = sorted({0, first_victim if first_victim not in (0, 15) else 3, 9 if first_victim != 9 else 10, 15})
    assert len(followed) == 4
    gen = torch.Generator(device=DEV).manual_seed(0)
    P, M, V = {}, {}, {}
    for k in range(n_chunks):
        p, m, v = client.chunk_state(k)
        p.normal_(0, 0.02, generator=gen)
        m.normal_(0, 1e-4, generator=gen)
        v.normal_(0, 1e-6, generator=gen).abs_()
        if k == 7:
            for dst, src in zip((p, m, v), client.chunk_state(6)):
                dst.copy_(src)
        if k in followed:
            P[k], M[k], V[k] = p.cpu().numpy(), m.cpu().numpy(), v.cpu().numpy()
    so = DynamicScalerOracle(2 ** 3, 2, 1000, 1)
    # the oracle makes the followed tensors' adam_update calls in visiting order; the calls in
    # between only repeat what the second call already leaves in the optimizer object's beta^t
    # history, and the last followed tensor is the rank's last one
    orc = StepOracle([(i, 0, CHUNK, 0) for i in range(len(followed))],
                     [{"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-6, "weight_decay": 0}], so, False)
    pinned = [torch.empty(CHUNK, dtype=torch.float16).pin_memory() for _ in followed]
    tmp = torch.empty(CHUNK, device=DEV)
    skips = []
    for step in range(steps):
        for cid in range(n_chunks):
            if cid == 7:
                client.fp16_chunk(7).copy_(client.fp16_chunk(6))
                continue
            tmp.normal_(0, 1e-3, generator=gen).mul_(float(so.loss_scale))
            client.fp16_chunk(cid).copy_(tmp)      # fp32 -> fp16, round to nearest even
        inject = step in plan
        if inject:
            victim, where, what = plan[step]
            for pos, val in zip(where, what):
                client.fp16_chunk(victim)[pos] = val
            if victim == 6:
                client.fp16_chunk(7).copy_(client.fp16_chunk(6))
        for buf, k in zip(pinned, followed):
            buf.copy_(client.fp16_chunk(k))
        torch.cuda.synchronize()
        H = [buf.numpy() for buf in pinned]
        opt.step()
        skipped = orc.step(H, [P[k] for k in followed], [M[k] for k in followed], [V[k] for k in followed],
                           overflow=inject)
        skips.append(skipped)
        st = scaler.read_state()  # bit-exact scale trajectory, every step
        assert (st.cur_scale, st.cur_iter, st.last_overflow_iter, st.cur_hysteresis) == \
            (float(so.cur_scale), so.cur_iter, so.last_overflow_iter, so.cur_hysteresis), step
        assert opt.read_ctrl().skip == int(inject), step
        if step in (0, 16, 17, 100):   # early divergence would show here, not only at the end
            for i, k in enumerate(followed):
                assert n_bit_mismatch(client.chunk_state(k)[0].cpu().numpy(), P[k]) == 0, (step, k)
                assert n_bit_mismatch(client.fp16_chunk(k).cpu().numpy(), H[i]) == 0, (step, k)
    assert sum(skips) == 11 and opt.step_count == steps - 11 == orc.step_count
    assert scaler.loss_scale == 1  # 8 -> 4 -> 2 -> 1, then pinned at min_scale
    torch.cuda.synchronize()
    for i, k in enumerate(followed):
        p, m, v = client.chunk_state(k)
        assert n_bit_mismatch(p.cpu().numpy(), P[k]) == 0, k
        assert n_bit_mismatch(m.cpu().numpy(), M[k]) == 0, k
        assert n_bit_mismatch(v.cpu().numpy(), V[k]) == 0, k
        assert n_bit_mismatch(client.fp16_chunk(k).cpu().numpy(), H[i]) == 0, k
    six = [checksum(t) for t in (*client.chunk_state(6), client.fp16_chunk(6))]
    seven = [checksum(t) for t in (*client.chunk_state(7), client.fp16_chunk(7))]
    assert six == seven
    sums = {tuple(checksum(client.chunk_state(k)[0])) for k in range(n_chunks)}
    assert len(sums) == n_chunks - 1      # every chunk went its own way (6 and 7 together)
    for k in range(n_chunks):
        p = client.chunk_state(k)[0]
        assert torch.equal(client.fp16_chunk(k).view(torch.int16), p.half().view(torch.int16)), k


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
