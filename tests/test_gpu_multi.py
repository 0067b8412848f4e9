"""Multi-GPU chunk step (reduce-scatter -> scan -> flag all-reduce -> step ->
all-gather) on real GPUs over NCCL, one process per GPU, checked rank by rank
against the oracle fed the actual post-reduce-scatter gradients."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# every form at 2 ranks; at 4 and 8 ranks the forms the benchmark picks there plus one NCCL form
COMBOS = [(2, "local"), (2, "reduced"), (2, "fused"), (2, "p2p"), (2, "staged"), (2, "copy"), (2, "copy_pull"),
          (4, "reduced"), (4, "fused"), (4, "p2p"), (4, "staged"), (4, "copy"), (4, "copy_pull"),
          (8, "local"), (8, "fused"), (8, "staged"), (8, "copy")]


@pytest.mark.parametrize("world,scan", COMBOS, ids=["%d-%s" % c for c in COMBOS])
def test_chunk_step_with_collectives(world, scan):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    env = dict(os.environ, PS_TEST_SCAN=scan)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(29700 + world),
           os.path.join(ROOT, "tests", "dist_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    if r.returncode != 0:
        err = "\n".join(ln for ln in (r.stdout + r.stderr).splitlines() if "Warning" not in ln)
        raise AssertionError(err[-6000:])
    assert "dist_worker ok" in r.stdout


@pytest.mark.parametrize("scan", ["local", "reduced"])
def test_chunk_step_with_collectives_and_offloaded_chunks(scan):
    """Hybrid placement on several GPUs: two of each rank's four chunks keep their
    fp32 state in pinned host memory and are streamed around the kernel between
    their reduce-scatter and their all-gather."""
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    env = dict(os.environ, PS_TEST_SCAN=scan, PS_TEST_OFFLOAD="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", "29731", os.path.join(ROOT, "tests", "dist_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    if r.returncode != 0:
        err = "\n".join(ln for ln in (r.stdout + r.stderr).splitlines() if "Warning" not in ln)
        raise AssertionError(err[-6000:])
    assert "dist_worker ok" in r.stdout


@pytest.mark.parametrize("collectives", ["nccl", "auto", "multimem"])
def test_data_parallel_engine_end_to_end(collectives):
    """initialize_engine on 2 ranks with different batches: forward, scaled backward
    with the gradient hand-off inside backward, step with the chunk collectives the
    config asks for (client.opts.fused_collectives); ranks stay in sync, an overflow
    on one rank skips the step on both, the loss goes down.  In the NCCL form every
    group's reduce-scatter must have been fired from the hand-off, before step()."""
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", "29741", os.path.join(ROOT, "tests", "dist_engine_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, PS_TEST_COLLECTIVES=collectives))
    if r.returncode != 0:
        err = "\n".join(ln for ln in (r.stdout + r.stderr).splitlines() if "Warning" not in ln)
        raise AssertionError(err[-6000:])
    assert "dist_engine_worker ok" in r.stdout
