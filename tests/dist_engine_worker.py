"""Worker of the data-parallel engine test: initialize_engine on every rank, each
rank trains on its own batch; engine.step() runs reduce-scatter, the rank-local
fused step and all-gather.  Launched by tests/test_gpu_multi.py."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from patrickstar_b200 import initialize_engine

    def model_func():
        torch.manual_seed(0)   # same initial weights on every rank
        return torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.Tanh(), torch.nn.Linear(96, 96),
                                   torch.nn.Tanh(), torch.nn.Linear(96, 96), torch.nn.Tanh(),
                                   torch.nn.Linear(96, 8))

    config = {"optimizer": {"type": "AdamW", "params": {"lr": 2e-3, "eps": 1e-6, "weight_decay": 0.01}},
              "fp16": {"enabled": True, "loss_scale": 0, "initial_scale_power": 8, "loss_scale_window": 1000,
                       "hysteresis": 2, "min_loss_scale": 1},
              "default_chunk_size": 10240,
              "client": {"opts": {"fused_collectives": os.environ.get("PS_TEST_COLLECTIVES", "auto")}}}
    engine, opt = initialize_engine(model_func, local, config)
    client = engine.client
    want = config["client"]["opts"]["fused_collectives"]
    assert engine.collectives == {"auto": "p2p" if world <= 3 else "multimem"}.get(want, want), engine.collectives
    assert (client.symm_handle is not None) == (engine.collectives != "nccl")
    assert client.world_size == world and client.layout.n_chunks % world == 0
    assert client.layout.n_data_chunks >= 3      # several communication groups
    gen = torch.Generator(device=dev).manual_seed(100 + rank)   # a different batch on every rank
    x = torch.randn(32, 64, device=dev, dtype=torch.float16, generator=gen)
    w_true = torch.randn(64, 8, device=dev, generator=torch.Generator(device=dev).manual_seed(7))
    y = (x.float() @ w_true).tanh()
    losses = []
    for it in range(30):
        out = engine(x)
        loss = torch.nn.functional.mse_loss(out.float(), y)
        if it == 5 and rank == world - 1:
            loss = loss * float("inf")           # one rank overflows: every rank must skip
        losses.append(float(loss.detach()))
        engine.backward(loss)
        if engine.collectives == "nccl":
            # every communication group that holds parameters was reduce-scattered from the
            # backward hand-off already; step() only waits for those
            with_data = {c // world for c in range(client.layout.n_data_chunks)}
            assert set(opt._rs_fired) == with_data, (sorted(opt._rs_fired), sorted(with_data))
        else:
            assert not opt._rs_fired
        engine.step()
        assert not opt._rs_fired and not opt._handed
        # after the all-gather every rank holds the same fp16 parameters
        mine = client.fp16.clone()
        ref = mine.clone()
        dist.broadcast(ref, src=0)
        used = torch.zeros_like(mine, dtype=torch.bool)
        for t in client.layout.tensors:
            s = t.flat_start(client.layout.chunk_size)
            used[s:s + t.numel] = True
        assert torch.equal(mine[used].view(torch.int16), ref[used].view(torch.int16)), it
        assert torch.isfinite(mine[used]).all(), it
    assert opt.step_count == 29 and opt.skipped_steps == 1
    assert engine.loss_scaler.loss_scale == 128
    finite = [l for l in losses if l == l and l != float("inf")]
    assert finite[-1] < 0.5 * finite[0], (finite[0], finite[-1])
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("dist_engine_worker ok: world %d, loss %.4f -> %.4f" % (world, finite[0], finite[-1]))


if __name__ == "__main__":
    main()
