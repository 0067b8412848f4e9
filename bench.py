#!/usr/bin/env python
"""Benchmark of the chunk optimizer step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the dynamic-loss-scale configuration — 16 chunks of 64 Mi
elements, fp32 master ~ N(0, 0.02), exp_avg ~ N(0, 1e-4), exp_avg_sq = |N(0, 1e-6)|,
fp16 grads = fp16(N(0, 1e-3) * scale), Adam lr 1e-3 betas (0.9, 0.999) eps 1e-6
wd 0, DynamicLossScaler(2**3, window 1000, min 1).  One step = overflow scan of
all chunks + step-begin kernel + the fused chunk step.  With N > 1 every rank
owns 16 chunks of a 16*N chunk list (weak scaling) and a step additionally does
the reduce-scatter of the fp16 grad chunks and the all-gather of the fp16 param
chunks of every communication group.

Prints ONE JSON line on rank 0.  All data is synthetic and seeded.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CHUNK = 64 * 1024 * 1024
CHUNKS_PER_RANK = 16
HYPER = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.0)
SCALER = dict(init_scale=2 ** 3, scale_factor=2, scale_window=1000, min_scale=1)
METRIC = "adam_updated_params_per_sec"
UNIT = "params/s"
BYTES_PER_PARAM = 28  # fp16 grad 2 + fp32 p/m/v read 12 + write 12 + fp16 param 2
# DRAM traffic of chunk_step_kernel per parameter from the ncu capture of the 2-chunk case
# (dram__bytes_read.sum + dram__bytes_write.sum = 3.702 GB for 134,217,728 parameters);
# traffic grows linearly with the number of chunks, so a launch is scaled by its parameters
NCU_DRAM_BYTES_PER_PARAM = 3.702e9 / (2 * 64 * 1024 * 1024)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--chunks", type=int, default=CHUNKS_PER_RANK, help="chunks per rank")
    ap.add_argument("--chunk-size", type=int, default=CHUNK)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--unroll", type=int, default=0, help="kernel tuning knob (0 = library default)")
    ap.add_argument("--blocks-per-sm", type=int, default=-1)
    ap.add_argument("--bulk", type=int, default=-1, help="kernel tuning knob: 1 = bulk-async staged chunk step")
    ap.add_argument("--scan", default="local", choices=["local", "reduced"],
                    help="N > 1: overflow test on local gradients before the reduction (the reference's "
                         "rule) or on the reduced ones")
    ap.add_argument("--collectives", default="auto", choices=["auto", "nccl", "fused", "p2p"],
                    help="N > 1: 'nccl' = NCCL reduce-scatter / all-gather pipelined around the step kernel; "
                         "'fused' = one kernel over NVSwitch multicast memory (multimem); 'p2p' = one kernel "
                         "over peer loads / stores; 'auto' = p2p for 2-3 ranks, fused for more, nccl if "
                         "symmetric memory cannot be set up")
    ap.add_argument("--layout", default="uniform", choices=["uniform", "gpt2_1.5b"],
                    help="N = 1 only: 'gpt2_1.5b' packs the GPT-2 1.5B tensors flat into 64 Mi chunks (24 "
                         "chunks, ~580 tensors, AdamW with two param groups straddling chunk boundaries) "
                         "instead of the uniform one-tensor-per-chunk workload; a side measurement of what "
                         "the segment tables cost")
    ap.add_argument("--offload-chunks", type=int, default=0,
                    help="keep the fp32 state of this many of the rank's chunks in pinned host memory and "
                         "stream them through the double-buffered offload pipeline (hybrid placement); "
                         "prints the offload report instead of the headline line")
    ap.add_argument("--offload-slots", type=int, default=2)
    ap.add_argument("--offload-piece", type=int, default=16 * 1024 * 1024, help="elements per staged piece")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while running."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def wait_first_sample(self, timeout=5.0):
        """nvidia-smi needs a few hundred milliseconds to start; wait for its first line."""
        t_end = time.time() + timeout
        while self.proc is not None and not self.lines and time.time() < t_end:
            time.sleep(0.02)

    def mark_load_begin(self):
        self.t_load = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        t_load = getattr(self, "t_load", 0.0)
        under_load = [ln for ts, ln in self.lines if ts >= t_load]
        for ln in (under_load or [ln for _, ln in self.lines]):
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# CPU baseline / reference arm
# ---------------------------------------------------------------------------
def _load_cpu_impl():
    """The reference's own CPU Adam (oracle/_ref) when it was built, else the C
    port of it."""
    from oracle import port, ref
    try:
        mod = ref.load()
        return "reference", mod
    except (FileNotFoundError, ImportError, OSError):
        port.lib()
        return "port", port


def use_all_host_threads():
    """The CPU arms run on every core the process may use.  (torch.distributed.run exports
    OMP_NUM_THREADS=1 to its workers; the OpenMP runtime shared by torch and the compiled
    reference follows torch.set_num_threads.)"""
    import torch
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_chunk_inputs(n):
    import torch
    g = torch.Generator().manual_seed(0)
    p = torch.randn(n, generator=g) * 0.02
    m = torch.randn(n, generator=g) * 1e-4
    v = (torch.randn(n, generator=g) * 1e-6).abs()
    gr = (torch.randn(n, generator=g) * 1e-3 * 8).half()
    return p, m, v, gr


def cpu_adam_call(kind, impl, handle, step, p, g, m, v):
    if kind == "reference":
        impl.adam_update(handle, step, HYPER["lr"], HYPER["betas"][0], HYPER["betas"][1], HYPER["eps"],
                         HYPER["weight_decay"], True, p, g, m, v, 8.0)
    else:
        handle.adam_update(step, HYPER["lr"], HYPER["betas"][0], HYPER["betas"][1], HYPER["eps"],
                           HYPER["weight_decay"], True, p, g, m, v, 8.0)


def cpu_baseline(n, seconds=10.0, max_calls=2000, warm=3):
    """Times adam_update of the CPU implementation on one chunk with all host
    threads.  Bounded sample: 1 chunk, about `seconds` of calls."""
    import torch
    kind, impl = _load_cpu_impl()
    cores = use_all_host_threads()
    p, m, v, g = cpu_chunk_inputs(n)
    if kind == "reference":
        impl.create_adam(31337, HYPER["lr"], HYPER["betas"][0], HYPER["betas"][1], HYPER["eps"],
                         HYPER["weight_decay"], False, False)
        handle = 31337
    else:
        handle = impl.OracleAdam(HYPER["lr"], HYPER["betas"][0], HYPER["betas"][1], HYPER["eps"],
                                 HYPER["weight_decay"], False)
    for i in range(warm):
        cpu_adam_call(kind, impl, handle, 1 + i, p, g, m, v)
    ts = []
    t_begin = time.perf_counter()
    while len(ts) < max_calls and (time.perf_counter() - t_begin < seconds or len(ts) < 10):
        t0 = time.perf_counter()
        cpu_adam_call(kind, impl, handle, 1 + warm + len(ts), p, g, m, v)
        ts.append(time.perf_counter() - t0)
    calls = len(ts)
    if kind == "reference":
        impl.destroy_adam(31337)
    ts.sort()
    med = ts[len(ts) // 2]
    return {"value": n / med, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": "1 chunk of %d elements, %d adam_update calls (median %.2f ms), all host threads; "
                      "Adam only (26 B/param), no overflow scan, no fp16 write-back" % (n, calls, med * 1e3)}


def run_reference_arm(args):
    """The reference's CPU implementation of the whole step on the host cores:
    per chunk the overflow test `grad.float().sum()` (loss_scaler.py:138), the
    native adam_update, and the fp32 -> fp16 chunk cast (chunk_io_buff.py:123-126)."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, impl = _load_cpu_impl()
    n, nchunks = args.chunk_size, args.chunks
    cores = use_all_host_threads()
    p0, m0, v0, g0 = cpu_chunk_inputs(n)
    # a bounded sample: `sample` chunks stand for the rank's `nchunks` (same distributions)
    sample = min(nchunks, 4)
    P = [p0.clone() for _ in range(sample)]
    M = [m0.clone() for _ in range(sample)]
    V = [v0.clone() for _ in range(sample)]
    G = [g0.clone() for _ in range(sample)]
    H = [torch.empty(n, dtype=torch.float16) for _ in range(sample)]
    if kind == "reference":
        impl.create_adam(31338, HYPER["lr"], HYPER["betas"][0], HYPER["betas"][1], HYPER["eps"],
                         HYPER["weight_decay"], False, False)
        handle = 31338
    else:
        handle = impl.OracleAdam(HYPER["lr"], HYPER["betas"][0], HYPER["betas"][1], HYPER["eps"],
                                 HYPER["weight_decay"], False)

    def one_step(step):
        overflow = False
        for k in range(sample):
            s = float(G[k].float().sum())
            overflow |= (s in (float("inf"), -float("inf")) or s != s)
        for k in range(sample):
            cpu_adam_call(kind, impl, handle, step, P[k], G[k], M[k], V[k])
            H[k].copy_(P[k])
        return overflow

    for i in range(args.warmup):
        one_step(1 + i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        one_step(1 + args.warmup + i)
    dt = time.perf_counter() - t0
    value = sample * n * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args, 1),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": "%d of %d chunks per step (overflow test + adam_update + fp16 cast), "
                                   "all host threads" % (sample, nchunks)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(args, world):
    return {"workload": "dynamic-loss-scale chunk step: %d chunks x %d elements per rank, Adam lr 1e-3 "
                        "betas (0.9,0.999) eps 1e-6 wd 0, DynamicLossScaler(2^3, window 1000, min 1)"
                        % (args.chunks, args.chunk_size),
            "chunks_per_rank": args.chunks, "chunk_elements": args.chunk_size,
            "parallelism": "chunk-sharded x%d" % world,
            "collectives": "none" if world == 1 else "reduce-scatter fp16 grads + all-gather fp16 params per group",
            "l2": "inputs (%.1f GiB per rank) exceed L2; fp16 grad slots rewritten between timed steps"
                  % (args.chunks * args.chunk_size * 14 / 2 ** 30)}


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus %d must be launched with torch.distributed.run "
                             "--nproc-per-node %d" % (args.gpus, args.gpus))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from patrickstar_b200 import ChunkClient, DynamicLossScaler, FP16Adam
    from patrickstar_b200 import _lib

    if args.unroll:
        _lib.tune("unroll", args.unroll)
    if args.blocks_per_sm >= 0:
        _lib.tune("blocks_per_sm", args.blocks_per_sm)
    if args.bulk >= 0:
        _lib.tune("bulk", args.bulk)

    cs, npr = args.chunk_size, args.chunks
    if args.collectives == "auto":
        args.collectives = "nccl" if world == 1 else ("p2p" if world <= 3 else "fused")
    fused = world > 1 and args.collectives in ("fused", "p2p")

    gpt_layout = args.layout != "uniform"
    if gpt_layout and world != 1:
        raise SystemExit("--layout %s is a single-GPU side measurement" % args.layout)

    def make_client(symmetric):
        c = ChunkClient(rank=local_rank, default_chunk_size=cs, world_size=world, device=dev, pack="flat",
                        symmetric=symmetric)
        if gpt_layout:
            from patrickstar_b200.model_layouts import model_specs
            import numpy as np
            specs = model_specs(args.layout)
            c.append_tensor_list([(n, int(np.prod(sh)), g) for n, sh, g in specs])
        else:
            c.append_tensor_list([("chunk%d" % i, cs, 0) for i in range(npr * world)])
        c.allocate()
        return c

    fallback_note = None
    if fused:
        # every rank must take the same path: agree on whether symmetric memory came up
        try:
            client = make_client(True)
            ok = 1
        except Exception as e:  # noqa: BLE001 - any set-up failure means "use NCCL"
            client, ok, fallback_note = None, 0, "symmetric memory unavailable (%s): NCCL collectives" % type(e).__name__
        t = torch.tensor([ok], dtype=torch.int32, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if int(t.item()) == 0:
            fused, args.collectives = False, "nccl"
            fallback_note = fallback_note or "symmetric memory unavailable on another rank: NCCL collectives"
            del client
            torch.cuda.empty_cache()
            client = make_client(False)
    else:
        client = make_client(False)
    scaler = DynamicLossScaler(device=dev, **SCALER)
    if gpt_layout:
        npr = args.chunks = len(client.local_ids)
        lay = client.layout
        decay = [p for n, p in client.params.items() if lay.tensor(n).group == 0]
        no_decay = [p for n, p in client.params.items() if lay.tensor(n).group == 1]
        hyper = dict(HYPER, weight_decay=0.01)
        opt = FP16Adam(client, [{"params": decay}, {"params": no_decay, "weight_decay": 0.0}],
                       loss_scaler=scaler, use_adamw=True, **hyper)
    else:
        opt = FP16Adam(client, client.params.values(), loss_scaler=scaler, use_adamw=False, **HYPER)

    # seeded synthetic state, generated on the device chunk by chunk
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    for k in range(npr):
        p, m, v = client.chunk_state(k)
        p.normal_(0, 0.02, generator=gen)
        m.normal_(0, 1e-4, generator=gen)
        v.normal_(0, 1e-6, generator=gen).abs_()
    # pristine fp16 grads of one communication group (world chunks); copied into
    # every group's slots before each step, outside the timed events
    tmp = torch.empty(world * cs, dtype=torch.float32, device=dev)
    tmp.normal_(0, 1e-3 * 8, generator=gen)
    pristine = tmp.half()
    del tmp

    def refresh_grads():
        for g in range(npr):
            client.fp16_group(g).copy_(pristine)

    def one_step():
        if fused:
            opt.step_fused_collectives("multimem" if args.collectives == "fused" else "p2p")
        elif world > 1:
            opt.step_with_collectives(scan=args.scan)
        else:
            opt.step()

    kernel_ev = []

    def timed_kernel_step():
        """opt.step() with CUDA events around the fused chunk-step launch."""
        if fused:
            # the fused kernel is timed by the step itself (its launch is not a separate method)
            one_step()
            return
        orig = opt._update_resident

        def wrapped(st, first=0, count=None):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            orig(st, first, count)
            b.record()
            kernel_ev.append((a, b, (client.n_resident - first) if count is None else count))
        opt._update_resident = wrapped
        try:
            one_step()
        finally:
            opt._update_resident = orig

    # clocks are sampled from the warm-up on (the GPU is under the same load there), so that
    # a timed region of a few hundred milliseconds still yields several samples
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        sampler.wait_first_sample()
    if world > 1:
        dist.barrier()
    if sampler:
        sampler.mark_load_begin()
    for _ in range(args.warmup):
        refresh_grads()
        one_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches0 = _lib.launch_count()
    step_ev = []
    torch.cuda.synchronize()
    for _ in range(args.steps):
        refresh_grads()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        timed_kernel_step()
        b.record()
        step_ev.append((a, b))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches = _lib.launch_count() - launches0
    step_ms = [a.elapsed_time(b) for a, b in step_ev]
    total_ms = sum(step_ms)
    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    # A timed region shorter than about a second holds one or two nvidia-smi samples.  In that
    # case keep the same load going (untimed, same steps) so that the median SM clock under
    # this load rests on several samples; the sampler runs through the timed region as well.
    n_extra = 0
    if total_ms < 1000.0:
        n_extra = max(1, min(400, int((1000.0 - total_ms) / max(total_ms / args.steps + 1.0, 1.0))))
    for _ in range(n_extra):
        refresh_grads()
        one_step()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    if clocks is not None:
        clocks["untimed_tail_steps"] = n_extra  # samples taken under the same load after the timed steps
    ctrl = opt.read_ctrl()
    assert ctrl.step == args.warmup + args.steps + n_extra and ctrl.n_skipped == 0, (ctrl.step, ctrl.n_skipped)
    params_per_step = opt.params_per_step if gpt_layout else npr * cs * world
    value = params_per_step * args.steps / (total_ms * 1e-3)

    peak, peak_kind = measured_peaks()
    if fused:
        # NVLink-bound: per owned parameter 2 B x (world-1) leave every GPU for the in-switch
        # reduction and 2 B x (world-1) arrive with the multicast store; measured peer-copy
        # bandwidth on this pool is 770 GB/s per direction
        link_bytes = 2 * (world - 1) * npr * cs
        step_s = total_ms / args.steps * 1e-3
        roofline = {"bound": "nvlink", "kernel": "chunk_step_fused_kernel" if args.collectives == "fused" else "chunk_step_p2p_kernel", "achieved": link_bytes / step_s / 1e9,
                    "peak": 770.0, "unit": "GB/s", "frac": link_bytes / step_s / 1e9 / 770.0,
                    "peak_source": "measured peer copy per direction (whole step time, scan and barriers included)",
                    "traffic": None, "algorithmic_bytes_per_launch": link_bytes, "launch_ms": None,
                    "launches_timed": args.steps}
    else:
        kern_ms = [a.elapsed_time(b) for a, b, _ in kernel_ev]
        kern_chunks = sum(c for _, _, c in kernel_ev)
        kern_avg_ms = sum(kern_ms) / len(kern_ms)
        bytes_per_launch = (BYTES_PER_PARAM * params_per_step if gpt_layout
                            else BYTES_PER_PARAM * cs * (kern_chunks / len(kernel_ev)))
        achieved = bytes_per_launch / (kern_avg_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "chunk_step_kernel", "achieved": achieved, "peak": peak,
                    "unit": "GB/s", "frac": achieved / peak, "peak_source": "%s copy bandwidth" % peak_kind,
                    "traffic": NCU_DRAM_BYTES_PER_PARAM * bytes_per_launch / BYTES_PER_PARAM,
                    "traffic_source": "ncu capture of the 2-chunk case, scaled by parameters per launch",
                    "algorithmic_bytes_per_launch": bytes_per_launch,
                    "launch_ms": kern_avg_ms, "launches_timed": len(kernel_ev)}

    local_step = None
    if world > 1:
        # the rank-local part alone (scan of the owned chunks + step-begin + fused
        # step, no collectives), for reading the comm-inclusive number against
        ev = []
        for _ in range(min(args.steps, 5)):
            refresh_grads()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            opt.step()
            b.record()
            ev.append((a, b))
        torch.cuda.synchronize()
        t = torch.tensor([sum(a.elapsed_time(b) for a, b in ev)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        local_step = {"value": params_per_step * len(ev) / (float(t.item()) * 1e-3), "unit": UNIT,
                      "ms_per_step": float(t.item()) / len(ev),
                      "what": "rank-local part only: no reduce-scatter, no all-gather"}

    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, client, opt, pristine, world, rank, dev, one_step)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, world),
            "roofline": roofline,
            "clocks": clocks, "gpu_launches": int(launches),
            "hbm_gbs_whole_step": (BYTES_PER_PARAM + 2) * npr * cs / (total_ms / args.steps * 1e-3) / 1e9
            if world == 1 else None,
        }
        if e2e is not None:
            line["e2e"] = e2e
        if fallback_note:
            line["config"]["note"] = fallback_note
        if gpt_layout:
            line["config"]["workload"] = ("GPT-2 1.5B layout: %d parameters in %d chunks of %d elements, %d "
                                          "segments, AdamW wd 0.01 / 0 in two param groups" % (
                                              params_per_step, npr, cs, len(opt._segs_host)))
        if local_step is not None:
            line["local_step"] = local_step
            line["config"]["overflow_scan"] = "local" if fused else args.scan
            line["config"]["collectives"] = (("fused into the step kernel (multimem ld_reduce / st over NVSwitch)" if args.collectives == "fused"
                                              else "fused into the step kernel (peer loads / stores over NVLink)")
                                             if fused else line["config"]["collectives"])
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(cs)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_e2e(args, client, opt, pristine, world, rank, dev, one_step_fn):
    """The same step through the public API with HOST buffers: every step copies
    the rank's fp16 grads from pinned host memory into the fp16 slots, runs the
    step, and copies the updated fp16 params of the local chunks plus the
    control block back to pinned host memory."""
    import torch
    import torch.distributed as dist
    cs, npr = args.chunk_size, args.chunks
    steps = max(2, min(args.steps, 5))
    host_in = torch.empty(world * cs, dtype=torch.float16).pin_memory()
    host_in.copy_(pristine)
    host_out = torch.empty(npr * cs, dtype=torch.float16).pin_memory()
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    outs = [host_out[k * cs:(k + 1) * cs] for k in range(npr)]
    ins = [host_in[:cs]] * npr

    def e2e_step():
        if world == 1:
            # the public call for host-resident fp16 chunks: copies, scan, step and
            # write-back pipelined chunk by chunk
            opt.step_host_chunks(ins, outs)
            return opt.read_ctrl()  # device -> host read of the step's result (skip flag, step counter)
        evs = []
        with torch.cuda.stream(copy_in):
            for g in range(npr):
                client.fp16_group(g).copy_(host_in, non_blocking=True)
                e = torch.cuda.Event()
                e.record()
                evs.append(e)
        for e in evs:
            main.wait_event(e)
        one_step_fn()
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            for k, cid in enumerate(client.local_ids):
                host_out[k * cs:(k + 1) * cs].copy_(client.fp16_chunk(cid), non_blocking=True)
        main.wait_stream(copy_out)
        return opt.read_ctrl()  # device -> host read of the step's result (skip flag, step counter)

    e2e_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        e2e_step()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return {"value": npr * cs * world * steps / (ms * 1e-3), "unit": UNIT,
            "h2d_bytes_per_step": 2 * npr * world * cs, "d2h_bytes_per_step": 2 * npr * cs + 1072,
            "ms_per_step": ms / steps, "steps": steps,
            "what": "pinned host fp16 grads -> slots, step, fp16 params of local chunks + control block -> pinned host"}


def run_offload(args):
    """Hybrid placement: `--offload-chunks` of the rank's chunks keep master / momentum /
    variance in pinned host memory.  Reports the step time, the three component times of
    the offloaded part measured alone (host->device copies, kernel, device->host copies)
    and overlap efficiency = max(component) / (step time - resident-only time)."""
    import torch
    import torch.distributed as dist
    from patrickstar_b200 import ChunkClient, DynamicLossScaler, FP16Adam
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cs, npr, k_off = args.chunk_size, args.chunks, args.offload_chunks
    client = ChunkClient(rank=local_rank, default_chunk_size=cs, world_size=world, device=dev, pack="flat")
    client.append_tensor_list([("chunk%d" % i, cs, 0) for i in range(npr * world)])
    client.allocate(state_budget_bytes=(npr - k_off) * 12 * cs)
    assert len(client.local_ids) - client.n_resident == k_off
    scaler = DynamicLossScaler(device=dev, **SCALER)
    opt = FP16Adam(client, client.params.values(), loss_scaler=scaler, use_adamw=False, **HYPER)
    if args.offload_slots != 2 or args.offload_piece != 16 * 1024 * 1024:
        opt.configure_offload(n_slots=args.offload_slots, piece_elems=args.offload_piece)
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    tmp = torch.empty(cs, device=dev)
    for k in range(npr):
        for t, (mu, sd) in zip(client.chunk_state(k), ((0, 0.02), (0, 1e-4), (0, 1e-6))):
            tmp.normal_(mu, sd, generator=gen)
            t.copy_(tmp.abs() if sd == 1e-6 else tmp)
    pristine = tmp.normal_(0, 8e-3, generator=gen).half()

    def refresh():
        for c in range(npr * world):
            client.fp16_chunk(c).copy_(pristine)

    def step_fn():
        if world > 1:
            opt.step_with_collectives()
        else:
            opt.step()

    def timed(fn, n):
        ev = []
        for _ in range(n):
            refresh()
            if world > 1:
                dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            ev.append((a, b))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in ev) / n

    for _ in range(args.warmup):
        refresh()
        step_fn()
    torch.cuda.synchronize()

    def over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    step_ms = over_ranks(timed(step_fn, args.steps))
    # components of the offloaded part, each alone on one stream (all ranks at once when N > 1,
    # so that contention for the host's memory and PCIe switches shows)
    staging = [torch.empty(cs, dtype=torch.float32, device=dev) for _ in range(3)]
    off = range(client.n_resident, npr)

    def h2d():
        for k in off:
            for dst, src in zip(staging, client.chunk_state(k)):
                dst.copy_(src, non_blocking=True)

    def d2h():
        for k in off:
            for src, dst in zip(staging, client.chunk_state(k)):
                dst.copy_(src, non_blocking=True)

    h2d_ms, d2h_ms = over_ranks(timed(h2d, 3)), over_ranks(timed(d2h, 3))
    # the same step without the pipeline (resident chunks and, for N > 1, all collectives)
    pipe, opt._offload = opt._offload, None
    n_res_saved = client.n_resident
    resident_ms = over_ranks(timed(step_fn, 3)) if world == 1 else None
    opt._offload = pipe
    client.n_resident = n_res_saved
    kern_ms = k_off * (BYTES_PER_PARAM * cs / 6.2e12) * 1e3  # from the measured 6.2 TB/s of the step kernel
    bound = max(h2d_ms, d2h_ms, kern_ms)
    pipe_ms = step_ms - resident_ms if resident_ms is not None else step_ms
    if rank == 0:
        line = {"workload": "hybrid offload: %d chunks x %d elements per rank, %d resident in HBM, %d in pinned "
                            "host memory, %d staging slots of %d elements" % (
                                npr, cs, npr - k_off, k_off, args.offload_slots, opt._offload.piece_elems),
                "metric": METRIC, "unit": UNIT, "value": world * npr * cs / (step_ms * 1e-3),
                "ms_per_step": step_ms, "offloaded_params_per_s_per_gpu": k_off * cs / (pipe_ms * 1e-3),
                "h2d_ms_alone": h2d_ms, "d2h_ms_alone": d2h_ms, "kernel_ms_offloaded_est": kern_ms,
                "resident_only_ms": resident_ms,
                "h2d_gbs_per_gpu": 12 * k_off * cs / (h2d_ms * 1e-3) / 1e9,
                "d2h_gbs_per_gpu": 12 * k_off * cs / (d2h_ms * 1e-3) / 1e9,
                "overlap_efficiency": bound / pipe_ms,
                "overlap_efficiency_note": "max(component alone) / (step - resident-only step); for N > 1 the "
                                           "denominator is the whole step, collectives included",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "data": "synthetic"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.offload_chunks > 0:
        return run_offload(args)
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
