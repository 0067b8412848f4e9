"""Worker of the multi-GPU chunk-step test.  Launched by
tests/test_gpu_multi.py with torch.distributed.run, one rank per GPU (NCCL)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


SCAN = os.environ.get("PS_TEST_SCAN", "local")
FUSED = ("fused", "p2p", "staged", "copy", "copy_pull")  # the forms over symmetric memory
TRANSPORT = {"fused": "multimem", "p2p": "p2p", "staged": "staged", "copy": "copy", "copy_pull": "copy_pull"}


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from helpers import n_bit_mismatch
    from oracle.scaler_oracle import DynamicScalerOracle
    from oracle.step_oracle import StepOracle
    from patrickstar_b200 import ChunkClient, DynamicLossScaler, FP16Adam

    cs = 1 << 15
    n_tensors = 3 * world + 1          # -> padded with dummy chunks
    client = ChunkClient(rank=local, default_chunk_size=cs, world_size=world, device=dev, pack="flat",
                         symmetric=(SCAN in FUSED))
    client.append_tensor_list([("w%d" % i, cs - (7 if i == n_tensors - 1 else 0), i % 2)
                               for i in range(n_tensors)])
    n_off = int(os.environ.get("PS_TEST_OFFLOAD", "0"))     # local chunks kept in pinned host memory
    client.allocate(state_budget_bytes=None if n_off == 0 else (4 - n_off) * 12 * cs)
    lay = client.layout
    assert len(client.local_ids) == 4 and client.n_resident == 4 - n_off
    assert lay.n_chunks % world == 0 and client.rank == rank
    g0 = [p for n, p in client.params.items() if lay.tensor(n).group == 0]
    g1 = [p for n, p in client.params.items() if lay.tensor(n).group == 1]
    scaler = DynamicLossScaler(init_scale=8, scale_factor=2, scale_window=1000, min_scale=1, device=dev)
    opt = FP16Adam(client, [{"params": g0, "weight_decay": 0.01}, {"params": g1, "weight_decay": 0.0}],
                   loss_scaler=scaler, lr=1e-3, eps=1e-6, use_adamw=True)
    gen = torch.Generator().manual_seed(500 + rank)
    P, M, V = [], [], []
    for k in range(len(client.local_ids)):
        p = torch.randn(cs, generator=gen) * 0.02
        m = torch.randn(cs, generator=gen) * 1e-4
        v = (torch.randn(cs, generator=gen) * 1e-6).abs()
        for dst, src in zip(client.chunk_state(k), (p, m, v)):
            dst.copy_(src)
        P.append(p.numpy().copy()), M.append(m.numpy().copy()), V.append(v.numpy().copy())
    so = DynamicScalerOracle(8, 2, 1000, 1)
    calls = [(client.local_ids.index(p.chunk_id), p.start, p.end, p.group) for p in lay.calls_of_rank(rank)]
    groups = [{"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-6, "weight_decay": 0.01},
              {"lr": 1e-3, "betas": (0.9, 0.999), "eps": 1e-6, "weight_decay": 0.0}]
    orc = StepOracle(calls, groups, so, True, world_size=world)
    for step in range(4):
        grads = (torch.randn(lay.n_chunks * cs, generator=gen) * 1e-3 * so.loss_scale * world).half()
        poisoned = step == 2
        if poisoned and rank == world - 1:
            grads[cs + 5] = float("nan")          # one rank's local gradient overflows
        client.fp16.copy_(grads)
        allg = [torch.empty_like(grads, device=dev) for _ in range(world)]
        dist.all_gather(allg, grads.to(dev))
        exact = sum(t.double() for t in allg)
        mag = sum(t.double().abs() for t in allg)
        if SCAN in FUSED:
            # what the fused kernel's reduction returns for this rank's chunks
            dist.barrier()
            reduced = opt.reduced_gradients("p2p" if SCAN in ("p2p", "copy", "copy_pull") else "multimem")
            torch.cuda.synchronize()
            dist.barrier()
        else:
            # what the reduce-scatter leaves in this rank's chunks (computed with NCCL itself,
            # so that its summation order is not part of the parity claim)
            probe = client.fp16.clone()
            for g in range(lay.n_groups_comm):
                buf = probe[g * world * cs:(g + 1) * world * cs]
                dist.reduce_scatter_tensor(buf[rank * cs:(rank + 1) * cs], buf, op=dist.ReduceOp.SUM)
            reduced = [probe[c * cs:(c + 1) * cs] for c in client.local_ids]
        H = []
        for k, c in enumerate(client.local_ids):
            got = reduced[k]
            if not poisoned:
                want = exact[c * cs:(c + 1) * cs]
                if SCAN in ("fused", "staged"):
                    # the switch accumulates in fp32 and converts the sum to fp16 by truncation
                    # (measured: errors up to 0.9 ulp, always toward zero): less than one fp16
                    # ulp of the exact sum, inside the (world - 1) / 2 ulp a ring of fp16
                    # additions may be off by for world >= 3
                    tol = 2.0 ** -10 * want.abs() + 2.0 ** -24
                elif SCAN in ("p2p", "copy", "copy_pull"):
                    # fp32 accumulation in rank order (each addition within 2^-24 relative of
                    # the partial sum), one rounding to fp16
                    tol = 2.0 ** -11 * want.abs() + world * 2.0 ** -23 * mag[c * cs:(c + 1) * cs] + 2.0 ** -25
                else:
                    # NCCL adds the `world` fp16 contributions in an order of its own, rounding
                    # to fp16 after every addition: (world - 1) roundings of at most half an ulp
                    # of a partial sum that never exceeds sum |x_r|
                    tol = (world - 1) * 2.0 ** -11 * mag[c * cs:(c + 1) * cs] + 2.0 ** -24
                bad = (got.double() - want).abs() > tol
                if bad.any():
                    i = int(bad.nonzero()[0])
                    raise AssertionError("reduced gradients outside fp16 rounding: chunk %d elem %d of %d bad: got %r "
                                         "exact %r contributions %r" % (c, i, int(bad.sum()), float(got[i]), float(want[i]),
                                                                        [float(t[c * cs + i]) for t in allg]))
            H.append(got.cpu().numpy().copy())
        if SCAN in FUSED:
            opt.step_fused_collectives(TRANSPORT[SCAN])
        else:
            opt.step_with_collectives(scan=SCAN)
        skipped = orc.step(H, P, M, V, overflow=poisoned)
        assert skipped == poisoned
        torch.cuda.synchronize()
        for k, c in enumerate(client.local_ids):
            dp, dm, dv = client.chunk_state(k)
            assert n_bit_mismatch(dp.cpu().numpy(), P[k]) == 0, (step, "p32", k)
            assert n_bit_mismatch(dm.cpu().numpy(), M[k]) == 0, (step, "exp_avg", k)
            assert n_bit_mismatch(dv.cpu().numpy(), V[k]) == 0, (step, "exp_avg_sq", k)
            # inside the chunk's used elements; the unused tail of a chunk keeps the reduced
            # gradients after an NCCL reduce-scatter and the local ones after the fused kernel
            n_used = lay.chunk_numel(c)
            assert n_bit_mismatch(client.fp16_chunk(c)[:n_used].cpu().numpy(), H[k][:n_used]) == 0, (step, "fp16", k)
        # after the all-gather every rank holds every owner's chunk (its used elements)
        mine = torch.cat([client.fp16_chunk(c) for c in client.local_ids])
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        for r in range(world):
            for k, c in enumerate(lay.local_chunk_ids(r)):
                n_used = lay.chunk_numel(c)
                theirs = client.fp16_chunk(c)[:n_used]
                owners = gathered[r][k * cs:k * cs + n_used]
                assert torch.equal(theirs.view(torch.int16), owners.view(torch.int16)), (step, "all-gather", r, c)
    assert opt.step_count == 3 and opt.skipped_steps == 1 and scaler.loss_scale == 4
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("dist_worker ok: world %d" % world)


if __name__ == "__main__":
    main()
