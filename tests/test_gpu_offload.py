"""Offload tier: chunks whose fp32 state lives in pinned host memory are streamed
through staging slots; results must equal the all-resident run and the oracle
bit for bit, over several steps (slot reuse across steps) and through a skipped
step."""
import pytest
import torch

from oracle.scaler_oracle import DynamicScalerOracle
from oracle.step_oracle import StepOracle
from test_gpu_chunk_step import compare, fill_states, groups_of, make_client, oracle_calls

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_resident", [0, 2, 4])
@pytest.mark.parametrize("piece", [2048, 1 << 24])
def test_offloaded_chunks_match_oracle(n_resident, piece):
    from patrickstar_b200 import DynamicLossScaler, FP16Adam
    cs = 30000
    sizes = [cs, 12345, cs - 12345 + 777, 2 * cs, 999, 3 * cs - 1776 - 13]
    specs = [("t%d" % i, n, i % 2) for i, n in enumerate(sizes)]
    client = make_client(specs, cs, budget=n_resident * 12 * cs)
    n_local = len(client.local_ids)
    assert client.n_resident == n_resident and n_local == 7
    g0 = [p for n, p in client.params.items() if client.layout.tensor(n).group == 0]
    g1 = [p for n, p in client.params.items() if client.layout.tensor(n).group == 1]
    scaler = DynamicLossScaler(init_scale=8, scale_factor=2, scale_window=1000, min_scale=1)
    opt = FP16Adam(client, [{"params": g0, "weight_decay": 0.01}, {"params": g1, "weight_decay": 0.0}],
                   loss_scaler=scaler, lr=1e-3, eps=1e-6, use_adamw=True)
    assert (opt._offload is not None) == (n_resident < n_local)
    if opt._offload is not None:
        opt.configure_offload(n_slots=2, piece_elems=piece)
    P, M, V = fill_states(client, 21)
    so = DynamicScalerOracle(8, 2, 1000, 1)
    orc = StepOracle(oracle_calls(client), groups_of(opt), so, True)
    gen = torch.Generator().manual_seed(22)
    for step in range(5):
        H = []
        for cid in client.local_ids:
            g = (torch.randn(cs, generator=gen) * 1e-3 * so.loss_scale).half()
            if step == 2 and cid == 5:
                g[4321] = float("-inf")
            client.fp16_chunk(cid).copy_(g)
            H.append(g.numpy().copy())
        opt.step()
        skipped = orc.step(H, P, M, V)
        assert skipped == (step == 2)
        compare(client, H, P, M, V, "step %d" % step)
    assert opt.step_count == 4 and opt.skipped_steps == 1


def test_more_slots_than_chunks_and_three_slots():
    from patrickstar_b200 import FP16Adam, LossScaler
    cs = 8192
    client = make_client([("w%d" % i, cs, 0) for i in range(5)], cs, budget=0)
    opt = FP16Adam(client, client.params.values(), loss_scaler=LossScaler(4.0), lr=1e-3)
    opt.configure_offload(n_slots=3, piece_elems=4096)
    P, M, V = fill_states(client, 31)
    from oracle.scaler_oracle import StaticScalerOracle
    orc = StepOracle(oracle_calls(client), groups_of(opt), StaticScalerOracle(4.0), False)
    gen = torch.Generator().manual_seed(32)
    for step in range(3):
        H = []
        for cid in client.local_ids:
            g = (torch.randn(cs, generator=gen) * 1e-3 * 4).half()
            client.fp16_chunk(cid).copy_(g)
            H.append(g.numpy().copy())
        opt.step()
        orc.step(H, P, M, V)
        compare(client, H, P, M, V, "step %d" % step)
