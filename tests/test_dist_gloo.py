"""World-size-2 test of the multi-rank path on CPU (gloo): ownership, the
in-place group collectives of patrickstar_b200/comm.py, the flag all-reduce and
the order reduce-scatter -> /world + step -> all-gather.  The rank-local step is
played by the CPU oracle here (the CUDA kernels need a GPU; their multi-GPU run
is in the gpu-marked tests)."""
import os
import sys
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORLD = 2
CS = 4096
N_CHUNKS = 6


def _grads(rank, step):
    g = torch.Generator().manual_seed(100 * step + rank)
    return (torch.randn(N_CHUNKS * CS, generator=g) * 1e-3 * 8 * WORLD).half()


def _worker(rank, port, q):
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=WORLD)
        from oracle.scaler_oracle import DynamicScalerOracle
        from oracle.step_oracle import StepOracle
        from patrickstar_b200 import comm
        from patrickstar_b200.chunk_list import ChunkLayout

        lay = ChunkLayout(CS, WORLD, "flat")
        lay.append_tensor_list([("w%d" % i, CS + (i % 3) * 100, i % 2) for i in range(5)])
        lay.freeze()
        assert lay.n_chunks == N_CHUNKS and lay.n_groups_comm == 3
        local = lay.local_chunk_ids(rank)
        assert local == [rank, rank + 2, rank + 4]
        calls = [(local.index(p.chunk_id), p.start, p.end, p.group) for p in lay.calls_of_rank(rank)]
        groups = [{"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-6, "weight_decay": 0.01},
                  {"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-6, "weight_decay": 0.0}]
        scaler = DynamicScalerOracle(8, 2, 1000, 1)
        orc = StepOracle(calls, groups, scaler, True, world_size=WORLD)
        gen = torch.Generator().manual_seed(7 + rank)
        P = [(torch.randn(CS, generator=gen) * 0.02).numpy() for _ in local]
        M = [(torch.randn(CS, generator=gen) * 1e-4).numpy() for _ in local]
        V = [(torch.randn(CS, generator=gen) * 1e-6).abs().numpy() for _ in local]
        fp16 = torch.zeros(N_CHUNKS * CS, dtype=torch.float16)
        results = []
        for step in range(3):
            fp16.copy_(_grads(rank, step))
            if step == 1 and rank == 1:
                fp16[3 * CS + 17] = float("inf")     # overflow on ONE rank must skip on BOTH
            exact = sum(_grads(r, step).double() for r in range(WORLD))
            for g in range(lay.n_groups_comm):
                buf = fp16[g * WORLD * CS:(g + 1) * WORLD * CS]
                comm.reduce_scatter_group(buf, rank, WORLD, CS)
            # the reduce-scatter result is the fp16-rounded sum of this rank's slices
            if step != 1:
                for c in local:
                    got = fp16[c * CS:(c + 1) * CS].double()
                    want = exact[c * CS:(c + 1) * CS]
                    ulp = torch.maximum(want.abs() * 2.0 ** -10, torch.full_like(want, 2.0 ** -24))
                    assert ((got - want).abs() <= ulp).all()
            H = [fp16[c * CS:(c + 1) * CS].numpy() for c in local]   # views: updated in place
            from oracle import port as oport
            flag = torch.tensor([int(any(oport.has_inf_or_nan_f16(h.view(np.uint16)) for h in H))],
                                dtype=torch.int32)
            comm.all_reduce_flag(flag)
            skipped = orc.step(H, P, M, V, overflow=bool(flag.item()))
            assert skipped == (step == 1)
            for g in range(lay.n_groups_comm):
                buf = fp16[g * WORLD * CS:(g + 1) * WORLD * CS]
                comm.all_gather_group(buf, rank, WORLD, CS)
            results.append(fp16.clone())
        q.put((rank, [r.numpy().view(np.uint16).copy() for r in results], orc.step_count,
               float(scaler.cur_scale), [p.copy() for p in P]))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        q.put((rank, "ERROR: " + traceback.format_exc(), None, None, None))


@pytest.mark.timeout(300)
def test_two_rank_chunk_step_over_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, port, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(WORLD):
        rank, res, steps, scale, P = q.get(timeout=240)
        assert not isinstance(res, str), res
        out[rank] = (res, steps, scale, P)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # both ranks hold the same full fp16 param buffer after every all-gather
    for a, b in zip(out[0][0], out[1][0]):
        assert (a == b).all()
    # both skipped exactly the poisoned step and agree on the scale
    assert out[0][1] == out[1][1] == 2
    assert out[0][2] == out[1][2] == 4.0
    # the gathered fp16 params are each owner's fp32 master rounded to fp16
    final = out[0][0][-1]
    for rank in range(WORLD):
        for k, c in enumerate([rank, rank + 2, rank + 4]):
            want = torch.from_numpy(out[rank][3][k]).half().numpy().view(np.uint16)
            numel = CS if c < 5 else 5 * CS + 300 - 5 * CS
            assert (final[c * CS:c * CS + numel] == want[:numel]).all()
