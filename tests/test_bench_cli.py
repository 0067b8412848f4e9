"""bench.py's reference arm runs on the host cores alone (no GPU) and prints the
contract's JSON line."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--chunks", "2",
                        "--chunk-size", "65536", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "adam_updated_params_per_sec" and d["unit"] == "params/s"
    assert d["value"] > 0 and d["higher_is_better"] is True and d["gpu_launches"] == 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "params/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["steps"] == 2 and d["warmup"] == 1


def test_reference_arm_other_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--chunks", "1", "--chunk-size", "4096", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_nvlink_byte_formula_is_the_documented_one():
    """One formula for the NVLink bytes of a multi-GPU step: in-switch forms move world + 1 chunks
    per direction, rank and group; peer, ring and copy-engine forms 2 * (world - 1)."""
    import bench
    for w in (2, 4, 8):
        assert bench.nvlink_chunks_per_group("fused", w) == w + 1
        assert bench.nvlink_chunks_per_group("staged", w) == w + 1
        for form in ("p2p", "nccl", "copy", "copy_pull"):
            assert bench.nvlink_chunks_per_group(form, w) == 2 * (w - 1)
