"""GPU parity of the optimizer step's remaining features against the CPU oracle:
the bulk-async staged kernel variant, NaN-preserving gradient clipping, the
world-size division as torch computes it, torch-managed (fp32-gradient)
parameters inside the step, per-step re-placement of chunk states, the restore
entry point and the device-side loss scaling.  Same bar as the other chunk-step
tests: bit-exact fp32 master / momentum / variance and fp16 params."""
import numpy as np
import pytest
import torch

from helpers import n_bit_mismatch
from oracle.scaler_oracle import DynamicScalerOracle, StaticScalerOracle
from oracle.step_oracle import StepOracle
from test_gpu_chunk_step import compare, fill_states, groups_of, make_client, oracle_calls

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("stages", [2, 4])
def test_bulk_staged_variant_two_groups_ragged(stages):
    """The chunk step with cp.async.bulk + mbarrier staging through shared memory
    (``ps_tune("bulk", 2..4)``) on two param groups that straddle chunk boundaries
    and a ragged last tensor, with a skipped step in the middle."""
    from patrickstar_b200 import DynamicLossScaler, FP16Adam, _lib
    cs = 3 * 2048 + 512     # full staged tiles and a ragged last tile per chunk
    specs = [("a", cs - 100, 0), ("b", 700, 1), ("c", 2 * cs + 5, 0), ("d", 33, 1), ("e", cs - 77, 0)]
    client = make_client(specs, cs)
    g0 = [client.params[n] for n, _, g in specs if g == 0]
    g1 = [client.params[n] for n, _, g in specs if g == 1]
    scaler = DynamicLossScaler(init_scale=32, scale_factor=2, scale_window=1000, min_scale=1)
    opt = FP16Adam(client, [{"params": g0, "weight_decay": 0.01}, {"params": g1, "weight_decay": 0.0}],
                   loss_scaler=scaler, lr=1e-3, eps=1e-6, use_adamw=True)
    P, M, V = fill_states(client, 21)
    so = DynamicScalerOracle(32, 2, 1000, 1)
    orc = StepOracle(oracle_calls(client), groups_of(opt), so, True)
    gen = torch.Generator().manual_seed(22)
    _lib.tune("bulk", stages)
    try:
        for step in range(4):
            H = []
            for k, cid in enumerate(client.local_ids):
                g = (torch.randn(cs, generator=gen) * 1e-3 * so.loss_scale).half()
                if step == 2 and k == 1:
                    g[cs // 2] = float("-inf")
                client.fp16_chunk(cid).copy_(g)
                H.append(g.numpy().copy())
            opt.step()
            assert orc.step(H, P, M, V) == (step == 2)
            compare(client, H, P, M, V, "bulk=%d step %d" % (stages, step))
        assert opt.read_ctrl().error == 0   # no bounded wait ran out
    finally:
        _lib.tune("bulk", 0)
    assert opt.step_count == 3 and opt.skipped_steps == 1


def test_clipping_keeps_nan_with_static_scaler():
    """fp16_cpu_adam.py:365-379: ``clamp_`` propagates NaN.  With a static scaler
    there is no overflow gate, so a NaN gradient must reach the parameters (a
    visible failure) instead of being clamped to -clip."""
    from patrickstar_b200 import FP16Adam, LossScaler
    cs = 4096
    client = make_client([("w", cs, 0)], cs)
    opt = FP16Adam(client, client.params.values(), loss_scaler=LossScaler(4.0), gradient_clipping=0.01, lr=1e-3)
    P, M, V = fill_states(client, 31)
    orc = StepOracle(oracle_calls(client), groups_of(opt), StaticScalerOracle(4.0), False, gradient_clipping=0.01)
    g = (torch.randn(cs, generator=torch.Generator().manual_seed(32)) * 0.1).half()
    g[5] = float("nan")
    g[9] = float("inf")       # clamps to +clip
    g[2049] = float("nan")    # in the second tile
    H = [g.numpy().copy()]
    client.fp16_chunk(0).copy_(g)
    opt.step()
    assert orc.step(H, P, M, V) is False
    torch.cuda.synchronize()
    p = client.chunk_state(0)[0].cpu().numpy()
    assert np.isnan(p[5]) and np.isnan(p[2049]) and np.isfinite(p[9])
    assert np.isnan(P[0][5]) and np.isnan(P[0][2049]) and np.isfinite(P[0][9])
    ok = ~np.isnan(P[0])
    assert (np.isnan(p) == ~ok).all()
    assert (p[ok].view(np.uint32) == P[0][ok].view(np.uint32)).all()
    h = client.fp16_chunk(0).cpu().numpy()
    assert (h[ok].view(np.uint16) == H[0][ok].view(np.uint16)).all() and np.isnan(h[5])


@pytest.mark.parametrize("world", [2, 3, 5, 6, 7, 8])
def test_world_divisor_is_torch_cuda_division(world):
    """patrickstar/core/client.py:838 runs ``payload /= world_size`` on a CUDA fp16
    tensor.  The kernel's folded division (and the oracle's) must be what torch
    computes there, bit for bit, for every world size - also the ones that are
    not powers of two, where the true quotient can differ by an fp16 ulp."""
    from patrickstar_b200 import FP16Adam, LossScaler
    from oracle import port
    cs = 1 << 16                      # every fp16 bit pattern once
    client = make_client([("w", cs, 0)], cs)
    opt = FP16Adam(client, client.params.values(), loss_scaler=LossScaler(1.0), lr=1.0, betas=(0.0, 0.0), eps=0.0)
    bits = torch.arange(cs, dtype=torch.int32).to(torch.int16)
    g = bits.view(torch.float16)
    want = g.to(DEV)
    want /= world                     # the reference's own operation, on the device
    want = want.cpu()
    mine = g.numpy().copy()
    port.div_world_f16(mine.view(np.uint16), world)
    finite = torch.isfinite(g).numpy()
    assert (mine.view(np.uint16)[finite] == want.numpy().view(np.uint16)[finite]).all(), "oracle != torch"
    # through the kernel: with beta1 = beta2 = 0, eps = 0, lr = 1 one step gives
    # exp_avg = g / world exactly (fp32 of the fp16 quotient)
    client.fp16_chunk(0).copy_(g)
    p, m, v = client.chunk_state(0)
    p.zero_(), m.zero_(), v.zero_()
    opt.step(grad_divisor=world)
    torch.cuda.synchronize()
    got = m.cpu().numpy()
    assert (got[finite] == want.float().numpy()[finite]).all(), "kernel != torch"


def test_torch_managed_fp32_grad_params_inside_the_step():
    """fp16_cpu_adam.py:345-353: a TORCH_BASED parameter (fp32, its own master, fp32
    gradient; the reference keeps the embedding weights so) is updated inside the
    same step, at its place of the visiting order.  Here the embedding-like tensor
    is registered FIRST, so it makes the first adam_update call of every step and
    takes the call-history dependent beta^t of that call
    (patrickstar/ops/csrc/includes/cpu_adam.h:143-162); a second one sits between
    the chunk tensors.  An overflow step must leave both untouched."""
    from patrickstar_b200 import ChunkClient, DynamicLossScaler, FP16Adam
    cs = 8192
    client = ChunkClient(rank=0, default_chunk_size=cs, world_size=1, device=DEV, pack="flat")
    emb = torch.nn.Parameter(torch.randn(1001, 7, generator=torch.Generator().manual_seed(40)) * 0.02)
    mid = torch.nn.Parameter(torch.randn(333, generator=torch.Generator().manual_seed(41)) * 0.02)
    client.append_torch_param("emb", emb)
    client.append_tensor_list([("a", cs + 100, 0), ("b", 500, 0)])
    client.append_torch_param("mid", mid)
    client.append_tensor_list([("c", cs - 9, 0)])
    client.allocate()
    assert emb.is_cuda and emb.dtype == torch.float32
    params = [emb, client.params["a"], client.params["b"], mid, client.params["c"]]
    scaler = DynamicLossScaler(init_scale=16, scale_factor=2, scale_window=1000, min_scale=1)
    opt = FP16Adam(client, params, loss_scaler=scaler, gradient_clipping=0.5, lr=1e-3, eps=1e-6, weight_decay=0.01,
                   use_adamw=True)
    P, M, V = fill_states(client, 42)
    seq = opt._call_sequence()
    assert [k for k, _ in seq][:2] == ["torch", "chunk"] and seq[0][1] == 0
    calls = []
    for kind, x in seq:
        calls.append(("torch", x, 0) if kind == "torch" else (client.local_ids.index(x.chunk_id), x.start, x.end, x.group))
    assert ("torch", 1, 0) in calls[2:-1]
    so = DynamicScalerOracle(16, 2, 1000, 1)
    orc = StepOracle(calls, groups_of(opt), so, True, gradient_clipping=0.5)
    T = [[t.detach().cpu().numpy().reshape(-1).copy(), None, np.zeros(t.numel(), np.float32),
          np.zeros(t.numel(), np.float32)] for t in (emb, mid)]
    gen = torch.Generator().manual_seed(43)
    for step in range(4):
        H = []
        for k, cid in enumerate(client.local_ids):
            g = (torch.randn(cs, generator=gen) * 1e-3 * so.loss_scale).half()
            if step == 1 and k == 0:
                g[17] = float("nan")
            client.fp16_chunk(cid).copy_(g)
            H.append(g.numpy().copy())
        for row, t in zip(T, (emb, mid)):
            g32 = torch.randn(t.shape, generator=gen) * 1e-3 * so.loss_scale
            if step == 2:
                g32.view(-1)[3] = 1e4      # beyond the clip: clamped in fp32
            t.grad = g32.to(DEV)
            row[1] = g32.numpy().reshape(-1).copy()
        opt.step()
        assert orc.step(H, P, M, V, torch_params=T) == (step == 1)
        compare(client, H, P, M, V, "step %d" % step)
        for row, t in zip(T, (emb, mid)):
            st = opt.state[t]
            assert n_bit_mismatch(t.detach().cpu().numpy().reshape(-1), row[0]) == 0, step
            assert n_bit_mismatch(st["exp_avg"].cpu().numpy().reshape(-1), row[2]) == 0, step
            assert n_bit_mismatch(st["exp_avg_sq"].cpu().numpy().reshape(-1), row[3]) == 0, step
    assert opt.step_count == 3 and opt.skipped_steps == 1
    sd = opt.state_dict()
    assert sd["state"][0]["exp_avg"].shape == emb.shape


def test_rebalance_moves_chunk_states_when_memory_runs_short():
    """patrickstar/core/memtracer/memtracer.py:190-214 + fp16_cpu_adam.py:523-528:
    the number of chunks that keep their state in HBM is re-derived from the free
    memory before a step.  A faked ``mem_get_info`` plays a device that runs short
    (two of five chunks must leave) and recovers; the trajectory stays bit-exact
    across both moves."""
    from patrickstar_b200 import ChunkClient, DynamicLossScaler, FP16Adam
    cs = 1 << 14
    per_chunk = 12 * cs
    c = ChunkClient(rank=0, default_chunk_size=cs, world_size=1, device=DEV, pack="flat",
                    config={"mem_tracer": {"margin_use_ratio": 1.0}})
    c.append_tensor_list([("w%d" % i, cs - (3 if i == 4 else 0), i % 2) for i in range(5)])
    c.mem_get_info = lambda dev: (1 << 40, 1 << 40)
    c.allocate(state_budget_bytes="auto")
    assert c.n_resident == 5
    g0 = [p for n, p in c.params.items() if c.layout.tensor(n).group == 0]
    g1 = [p for n, p in c.params.items() if c.layout.tensor(n).group == 1]
    so = DynamicScalerOracle(8, 2, 1000, 1)
    opt = FP16Adam(c, [{"params": g0}, {"params": g1, "weight_decay": 0.1}],
                   loss_scaler=DynamicLossScaler(init_scale=8, scale_factor=2, scale_window=1000, min_scale=1),
                   lr=1e-3, eps=1e-6, use_adamw=True)
    P, M, V = fill_states(c, 51)
    orc = StepOracle(oracle_calls(c), groups_of(opt), so, True)
    gen = torch.Generator().manual_seed(52)

    def one_step(tag):
        H = []
        for cid in c.local_ids:
            g = (torch.randn(cs, generator=gen) * 1e-3 * so.loss_scale).half()
            c.fp16_chunk(cid).copy_(g)
            H.append(g.numpy().copy())
        opt.step()
        orc.step(H, P, M, V)
        compare(c, H, P, M, V, tag)

    one_step("all resident")
    # the device is short: what the states hold now plus what is free makes room for 3 chunks
    c.mem_get_info = lambda dev: (3 * per_chunk + 100 - per_chunk * c.n_resident, 1 << 40)
    assert opt.rebalance() is True
    assert c.n_resident == 3 and opt._offload is not None and len(c.p32_host) == 2 and c.p32_host[0].is_pinned()
    one_step("two chunks on the host")
    one_step("two chunks on the host, again")
    assert opt.rebalance() is False          # nothing changed: no move
    c.mem_get_info = lambda dev: (1 << 40, 1 << 40)
    assert opt.rebalance() is True
    assert c.n_resident == 5 and opt._offload is None and c.p32_host is None
    one_step("back in HBM")
    assert opt.step_count == 4


def test_restore_fp16_entry_point():
    """ps_restore_fp16: fp16 slot := half(fp32 master) inside the segments only
    (fp16_cpu_adam.py:298-309), without a control block."""
    from patrickstar_b200 import FP16Adam
    cs = 5000
    client = make_client([("a", 3000, 0), ("b", cs + 1234, 0)], cs)
    opt = FP16Adam(client, client.params.values(), lr=1e-3)
    P, _, _ = fill_states(client, 61)
    junk = torch.full((cs,), 7.0, dtype=torch.float16)
    for cid in client.local_ids:
        client.fp16_chunk(cid).copy_(junk)
    opt.restore_fp16()
    torch.cuda.synchronize()
    for k, cid in enumerate(client.local_ids):
        n_used = client.layout.chunk_numel(cid)
        want = torch.from_numpy(P[k]).half()
        got = client.fp16_chunk(cid).cpu()
        assert torch.equal(got[:n_used].view(torch.int16), want[:n_used].view(torch.int16))
        assert (got[n_used:] == 7.0).all()      # outside every segment: untouched


def test_scale_loss_runs_on_the_device_state():
    """DynamicLossScaler.backward (loss_scaler.py:188-190) multiplies by the scale
    held in the device state block: value and gradient follow a scale change
    without any host read."""
    from patrickstar_b200 import DynamicLossScaler
    sc = DynamicLossScaler(init_scale=2 ** 10, scale_factor=2, scale_window=1000, min_scale=1, device=DEV)
    w = torch.tensor([1.5, -2.0, 0.25], device=DEV, requires_grad=True)
    loss = (w * w).sum()
    scaled = sc.scale_loss(loss)
    assert float(scaled.detach()) == float(loss.detach()) * 1024
    sc.backward((w * w).sum())
    assert torch.equal(w.grad, 2 * w.detach() * 1024)
    sc.update_scale(True)            # overflow: 1024 -> 512, on the device
    w.grad = None
    sc.backward((w * w).sum())
    assert torch.equal(w.grad, 2 * w.detach() * 512)
    half_loss = (w.half() * 2).sum()
    assert sc.scale_loss(half_loss).dtype == torch.float16


def test_engine_follows_free_memory_step_by_step():
    """initialize_engine with use_hybrid_adam (the default) places chunk states by the memory
    that is free and re-decides before every step (fp16_cpu_adam.py:523-528).  Two identical
    engines train on the same batch; one of them is told, through a faked ``mem_get_info``,
    that memory runs short from iteration 3 on and recovers at iteration 7.  Its chunk states
    move to pinned host memory and back, and every parameter stays bit-identical to the
    undisturbed engine's."""
    from patrickstar_b200 import initialize_engine

    def model_func():
        torch.manual_seed(3)
        return torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.Tanh(), torch.nn.Linear(40, 40),
                                   torch.nn.Tanh(), torch.nn.Linear(40, 40), torch.nn.Tanh(),
                                   torch.nn.Linear(40, 8))

    cfg = {"optimizer": {"type": "AdamW", "params": {"lr": 1e-3, "eps": 1e-6, "weight_decay": 0.01}},
           "fp16": {"enabled": True, "loss_scale": 0, "initial_scale_power": 8, "loss_scale_window": 1000,
                    "hysteresis": 2, "min_loss_scale": 1},
           "default_chunk_size": 2048, "client": {"mem_tracer": {"margin_use_ratio": 1.0}}}
    a, _ = initialize_engine(model_func, 0, cfg)
    b, _ = initialize_engine(model_func, 0, cfg)
    n_local = len(b.client.local_ids)
    assert n_local >= 3 and a.client._budget == "auto" and a.client.n_resident == b.client.n_resident == n_local
    per_chunk = 12 * 2048
    gen = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn(16, 24, device=DEV, dtype=torch.float16, generator=gen)
    y = torch.randn(16, 8, device=DEV, generator=gen)
    seen = []
    for it in range(10):
        if it == 3:     # room for one chunk's state only
            b.client.mem_get_info = lambda dev: (per_chunk + 8 - per_chunk * b.client.n_resident, 1 << 40)
        if it == 7:
            b.client.mem_get_info = lambda dev: (1 << 40, 1 << 40)
        for eng in (a, b):
            loss = torch.nn.functional.mse_loss(eng(x).float(), y)
            eng.backward(loss)
            eng.step()
        seen.append(b.client.n_resident)
        for pa, pb in zip(a.module.parameters(), b.module.parameters()):
            assert torch.equal(pa.data.view(torch.int16), pb.data.view(torch.int16)), it
    assert seen == [n_local] * 3 + [1] * 4 + [n_local] * 3, seen
    for k in range(n_local):
        for ta, tb in zip(a.client.chunk_state(k), b.client.chunk_state(k)):
            assert torch.equal(ta.cpu().view(torch.int32), tb.cpu().view(torch.int32)), k
    assert a.optimizer.step_count == b.optimizer.step_count == 10
