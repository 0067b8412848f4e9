"""FP16Adam — the mixed-precision chunk optimizer, B200 edition.

Mirror of ``patrickstar/ops/fp16_cpu_adam.py``: same class name, constructor
signature (``:64-77``), validation errors (``:82-91``), ``check_overflow``,
``step``, ``state_dict`` / ``load_state_dict``.  Where the reference walks the
parameters in Python and calls a CPU Adam or ~10 torch kernels per tensor, this
class enqueues, per step and without any host synchronisation,

  1. an overflow scan of the local fp16 chunks (2 B/element),
  2. a one-thread kernel that takes the skip decision, advances the step
     counter and the loss scale, and prepares the per-group constants,
  3. one fused launch over all resident local chunks (28 B/element), plus the
     double-buffered host-offload pipeline for chunks kept in pinned memory.

Differences from the reference that a user can see
  * more than one param group is accepted (the reference asserts exactly one,
    ``:108-110``); with one group the behaviour is the reference's.
  * ``state[p]["step"]`` is not kept per parameter on the host; the step counter
    lives on the device (``step_count`` reads it back).
  * like the reference, hyper-parameters are captured into ``state[p]`` at
    construction (``:112-120``) and the step reads them from there, not from
    ``param_groups``.
  * parameters registered with the client as torch-managed (the reference's
    TORCH_BASED kind: fp32 parameter, fp32 gradient, no fp16 slot, ``:345-353``)
    are updated by the same step, in their place of the visiting order, by one
    extra launch over a table of them; like the reference their gradients are
    neither tested for overflow nor divided by the world size.
"""
import ctypes as C
import logging
from copy import deepcopy

import numpy as np
import torch

from ._lib import (CHUNK_DESC_DTYPE, PS_MAX_GROUPS, SEGMENT_DTYPE, TENSOR_DESC_DTYPE, GroupHyper, ScalerState,
                   StepCtrl, StepPlan, check, lib)
from .loss_scaler import DynamicLossScaler, _DeviceScaler
from .timers import ADAM, ADAM_COMPUTE, ADAM_OFFLOAD, ADAM_OVERFLOW_SCAN, PhaseTimer


logger = logging.getLogger("PatrickStar")   # the reference's logger name (patrickstar/utils/logging.py:36)


class _NoScaler(_DeviceScaler):
    """State block for `loss_scaler=None`: loss_scale -1, no overflow gate
    (fp16_cpu_adam.py:226)."""
    _int_scale = False

    def __init__(self, device):
        st = ScalerState(cur_scale=-1.0, scale_factor=1.0, min_scale=1.0, cur_iter=0,
                         last_overflow_iter=-1, scale_window=1, delayed_shift=1, cur_hysteresis=1,
                         consecutive_hysteresis=0, dynamic=-1)
        super().__init__(st, device)


class FP16Adam(torch.optim.Optimizer):
    optimizer_id = 0

    def __init__(self, client, params, loss_scaler=None, gradient_clipping=-1, lr=1e-3,
                 betas=(0.9, 0.999), eps=1e-8, weight_decay=0, use_adamw=False, amsgrad=False,
                 use_hybrid_adam=True):
        if not 0.0 <= lr:
            raise ValueError("Invalid learning rate: {}".format(lr))
        if not 0.0 <= eps:
            raise ValueError("Invalid epsilon value: {}".format(eps))
        if not 0.0 <= betas[0] < 1.0:
            raise ValueError("Invalid beta parameter at index 0: {}".format(betas[0]))
        if not 0.0 <= betas[1] < 1.0:
            raise ValueError("Invalid beta parameter at index 1: {}".format(betas[1]))
        if not 0.0 <= weight_decay:
            raise ValueError("Invalid weight_decay value: {}".format(weight_decay))
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad)
        super().__init__(params, defaults)
        if len(self.param_groups) > PS_MAX_GROUPS:
            raise ValueError("at most %d param groups are supported" % PS_MAX_GROUPS)
        self.client = client
        self.device = client.device
        self.loss_scaler = loss_scaler
        self.gradient_clipping = gradient_clipping
        self.use_hybrid_adam = use_hybrid_adam
        self.use_adamw = use_adamw
        self.opt_id = FP16Adam.optimizer_id
        FP16Adam.optimizer_id += 1
        self._scaler = loss_scaler if loss_scaler is not None else _NoScaler(self.device)
        if not isinstance(self._scaler, _DeviceScaler):
            raise TypeError("loss_scaler must be a patrickstar_b200 LossScaler / DynamicLossScaler")
        self._dynamic = isinstance(self._scaler, DynamicLossScaler)

        # eager state, as the reference (fp16_cpu_adam.py:112-120); the group
        # index of every tensor in the chunk layout follows param_groups
        name_of = {id(p): n for n, p in client.params.items()}
        torch_name_of = {id(p): n for n, (p, _) in client.torch_params.items()}
        lay = client.layout
        self._torch = []   # [name, param, group index, visiting position] of the torch-managed parameters
        for gi, group in enumerate(self.param_groups):
            for p in group["params"]:
                if id(p) not in name_of and id(p) not in torch_name_of:
                    raise ValueError("FP16Adam got a parameter that is not registered with the client")
                st = self.state[p]
                st["betas"] = group["betas"]
                st["lr"] = group["lr"]
                st["weight_decay"] = group["weight_decay"]
                st["eps"] = group["eps"]
                if id(p) in torch_name_of:
                    # fp16_cpu_adam.py:122-131: momentum and variance of a torch-managed
                    # parameter are plain fp32 tensors of its shape
                    name = torch_name_of[id(p)]
                    st["name"] = name
                    st["exp_avg"] = torch.zeros_like(p.data, dtype=torch.float32, device=self.device)
                    st["exp_avg_sq"] = torch.zeros_like(p.data, dtype=torch.float32, device=self.device)
                    self._torch.append([name, p, gi, client.torch_params[name][1]])
                    continue
                st["name"] = name_of[id(p)]
                lay.set_group(name_of[id(p)], gi)
        self._torch.sort(key=lambda t: t[3])
        self._torch_table_dev = (torch.zeros(max(len(self._torch), 1) * TENSOR_DESC_DTYPE.itemsize,
                                             dtype=torch.uint8, device=self.device) if self._torch else None)
        # backward-side bookkeeping for data-parallel runs: elements handed off per
        # communication group, and the reduce-scatters already fired for complete groups
        self.rs_on_handoff = False
        self._handed = {}
        self._rs_fired = {}
        self._expected = None

        # section timing of the step on CUDA events (off by default; no sync either way)
        self.time_profile = False
        # The reference logs "Gradient overflow! Update loss scale from X to Y." on a skipped step
        # (fp16_cpu_adam.py:549-558).  Here the decision is taken on the device, so the message
        # costs a read-back (a synchronisation) per step and is off unless asked for.
        self.log_overflow = False
        # optional callable(name): called between the phases of the fused multi-GPU step so that
        # a benchmark can drop CUDA events there ("scan", "flag", "kernel", "barrier" = phase done)
        self.phase_marker = None
        self.timer = PhaseTimer()
        self._calls = 0            # number of step() calls, an upper bound of the step counter
        self._pow_len = 0
        self._pow_table = None
        self._ctrl = torch.zeros(C.sizeof(StepCtrl), dtype=torch.uint8, device=self.device)
        b1, b2 = self.param_groups[0]["betas"]
        with torch.cuda.device(self.device):
            check(lib.ps_ctrl_init(self._ctrl.data_ptr(), 0, b1, b2, self._stream()), "ps_ctrl_init")
        self._build_tables()
        self._offload = None
        if client.n_resident < len(client.local_ids):
            from .offload import OffloadPipeline
            self._offload = OffloadPipeline(client, self)

    def configure_offload(self, n_slots=2, piece_elems=16 * 1024 * 1024):
        """Rebuild the offload pipeline with another number of staging slots or
        another piece size (no-op when every local chunk is resident)."""
        if self.client.n_resident >= len(self.client.local_ids):
            return
        from .offload import OffloadPipeline
        self._offload = None
        self._desc_host = self._desc_host[:self._n_local].copy()
        self._offload = OffloadPipeline(self.client, self, n_slots=n_slots, piece_elems=piece_elems)

    # ------------------------------------------------------------------ tables
    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _call_sequence(self):
        """The adam_update calls the reference would make on this rank in one step,
        in its visiting order (the optimizer's parameter order, remote chunks
        skipped; fp16_cpu_adam.py:569-606): ("chunk", piece) and ("torch", index
        into self._torch) entries."""
        c = self.client
        seq = []
        torch_left = list(range(len(self._torch)))
        for piece in c.layout.calls_of_rank(c.rank):
            while torch_left and self._torch[torch_left[0]][3] <= piece.tensor_index:
                seq.append(("torch", torch_left.pop(0)))
            seq.append(("chunk", piece))
        seq.extend(("torch", i) for i in torch_left)
        return seq

    def _build_tables(self):
        c = self.client
        lay = c.layout
        seq = self._call_sequence()
        # the first call of a step sees another beta^t than the later ones (slot 0); when a
        # torch-managed parameter is visited first, no chunk piece carries that slot
        torch_first = bool(seq) and seq[0][0] == "torch"
        local, numels, ranges, segs = lay.build_tables(c.rank, first_call_slot=not torch_first)
        n_local = len(local)
        cs = lay.chunk_size
        desc = np.zeros(n_local, dtype=CHUNK_DESC_DTYPE)
        for k, cid in enumerate(local):
            desc["h16"][k] = c.fp16_chunk(cid).data_ptr()
            desc["numel"][k] = numels[k]
            desc["seg_begin"][k], desc["seg_end"][k] = ranges[k]
            if k < c.n_resident:
                p, m, v = c.chunk_state(k)
                desc["p32"][k], desc["exp_avg"][k], desc["exp_avg_sq"][k] = (
                    p.data_ptr(), m.data_ptr(), v.data_ptr())
        seg_rows = np.zeros(max(len(segs), 1), dtype=SEGMENT_DTYPE)
        if len(segs):
            seg_rows["start"], seg_rows["end"], seg_rows["slot"] = segs[:, 0], segs[:, 1], segs[:, 2]
        # chunks without tensors (dummy padding) take an empty range
        self._desc_host = desc
        self._segs_host = seg_rows
        n_res = c.n_resident
        if n_res:
            check(lib.ps_table_check(desc.ctypes.data, n_res, seg_rows.ctypes.data, len(segs),
                                     len(self.param_groups) + 1, cs), "ps_table_check")
        self._desc_dev = torch.from_numpy(desc.view(np.uint8).copy()).to(self.device)
        self._segs_dev = torch.from_numpy(seg_rows.view(np.uint8).copy()).to(self.device)
        self._n_local = n_local
        self._max_numel = int(max(numels)) if numels else 0
        self._max_numel_resident = int(max(numels[:n_res])) if n_res else 0
        group_of = lambda e: e[1].group if e[0] == "chunk" else self._torch[e[1]][2]
        self._first_group = group_of(seq[0]) if seq else 0
        self._last_group = group_of(seq[-1]) if seq else 0
        self._n_calls = len(seq)
        self._torch_slots = [0 if (torch_first and i == seq[0][1]) else 1 + t[2] for i, t in enumerate(self._torch)]
        self._n_updated = int(sum(numels)) + sum(t[1].numel() for t in self._torch)

    def _ensure_pow_table(self, upto):
        if upto < self._pow_len:
            return
        new_len = max(4096, self._pow_len)
        while new_len <= upto:
            new_len *= 2
        ng = len(self.param_groups)
        host = np.zeros((ng, new_len, 2), dtype=np.float32)
        for gi, group in enumerate(self.param_groups):
            b1, b2 = self.state[group["params"][0]]["betas"] if group["params"] else group["betas"]
            check(lib.ps_pow_table_fill(b1, b2, 0, new_len, host[gi].ctypes.data), "ps_pow_table_fill")
        self._pow_table = torch.from_numpy(host).to(self.device)
        self._pow_len = new_len

    def _plan(self, grad_divisor):
        plan = StepPlan()
        plan.clip = float(self.gradient_clipping) if self.gradient_clipping > 0 else 0.0
        for gi, group in enumerate(self.param_groups):
            st = self.state[group["params"][0]] if group["params"] else group
            b1, b2 = st["betas"]
            plan.groups[gi] = GroupHyper(lr=st["lr"], beta1=b1, beta2=b2, eps=st["eps"],
                                         weight_decay=st["weight_decay"], adamw_mode=int(self.use_adamw))
        plan.n_groups = len(self.param_groups)
        plan.first_group = self._first_group
        plan.last_group = self._last_group
        plan.n_calls = self._n_calls
        plan.grad_divisor = float(grad_divisor)
        plan.bias_correction = 1
        return plan

    # ------------------------------------------------------------ reference API
    def check_overflow(self, param):
        """fp16_cpu_adam.py:279-285 — sticky OR of "param.grad holds inf/nan",
        accumulated in the device flag without a host sync."""
        if self._dynamic and param.grad is not None:
            self._scaler.accumulate_overflow(param.grad)

    @torch.no_grad()
    def handoff_grad(self, param):
        """The backward hook's per-parameter work (patrickstar/core/hook.py:205-230)
        as one kernel: test ``param.grad`` for inf/nan into the device flag and copy
        it into the parameter's fp16 slot, then drop ``param.grad``.  No host sync.
        A step whose gradients all arrived this way may run with ``scan=False``.

        With ``rs_on_handoff`` set (data parallel, NCCL form) the hand-off also
        counts the elements that have arrived per communication group and, once a
        group's gradients are complete, fires that group's reduce-scatter at once
        on the reduce-scatter communicator — the reference's trigger
        (hook.py:218-227 -> patrickstar/core/client.py:812-840) — so that the
        collective overlaps the rest of backward; ``step_with_collectives(scan="done")``
        then only waits for it.  Every rank must hand its gradients off in the same
        order (same model, same graph), as NCCL requires of collectives.

        A torch-managed (fp32) parameter keeps its ``.grad``: the step reads it
        in place."""
        g = param.grad
        if g is None:
            return
        st_p = self.state[param]
        if "exp_avg" in st_p:   # torch-managed: nothing to hand off
            return
        if g.dtype != torch.float16 or not g.is_cuda:
            raise TypeError("handoff_grad needs a CUDA fp16 gradient, got %s on %s" % (g.dtype, g.device))
        g = g.contiguous()
        flag = self._scaler.flag_ptr if self._dynamic else None
        with torch.cuda.device(self.device):
            check(lib.ps_grad_handoff(g.data_ptr(), param.data.data_ptr(), g.numel(), flag, self._stream()),
                  "ps_grad_handoff")
        param.grad = None
        c = self.client
        if self.rs_on_handoff and c.world_size > 1:
            self._count_handoff(st_p["name"])

    def _count_handoff(self, name):
        c = self.client
        lay = c.layout
        if self._expected is None:
            exp = {}
            for t in lay.tensors:
                lay.add_to_comm_groups(t, exp)
            self._expected = exp
        for g, n in lay.add_to_comm_groups(lay.tensor(name), {}).items():
            self._handed[g] = self._handed.get(g, 0) + n
            if self._handed[g] == self._expected[g] and g not in self._rs_fired:
                # the group's gradients are complete on this rank: reduce-scatter now
                self._rs_fired[g] = c.reduce_scatter_group(g, async_op=True)

    @torch.no_grad()
    def step(self, closure=None, grad_divisor=None, scan=True):
        """One optimizer step over this rank's local chunks (fp16_cpu_adam.py:472-628).

        Expects the fp16 slots of the local chunks to hold the (reduce-scattered)
        gradients.  ``grad_divisor`` folds the reference's fp16 `payload /=
        world_size` (patrickstar/core/client.py:838) into the gradient load;
        default: the world size when it is > 1."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        c = self.client
        if grad_divisor is None:
            grad_divisor = c.world_size if c.world_size > 1 else 0
        tp = self.time_profile
        with torch.cuda.device(self.device):
            st = self._stream()
            old_scale = self._scaler.loss_scale if (self.log_overflow and self._dynamic) else None
            if tp:
                self.timer.start_profile(ADAM)
            if self._dynamic:
                if scan and self._n_local:
                    if tp:
                        self.timer.start_profile(ADAM_OVERFLOW_SCAN)
                    check(lib.ps_overflow_scan(self._desc_dev.data_ptr(), self._n_local, self._max_numel,
                                               self._scaler.flag_ptr, st), "ps_overflow_scan")
                    if tp:
                        self.timer.finish_profile(ADAM_OVERFLOW_SCAN)
                        self.timer.update_bytes(ADAM_OVERFLOW_SCAN, 2 * int(self._desc_host["numel"][:self._n_local].sum()))
                c.all_reduce_flag(self._scaler.flag_tensor)
            self._begin(grad_divisor, st)
            if tp:
                self.timer.start_profile(ADAM_COMPUTE)
            self._update_resident(st)
            self._update_torch_params(st)
            if tp:
                self.timer.finish_profile(ADAM_COMPUTE)
                # 28 B per updated parameter (a skipped step moves 6 B; the counter states the update's)
                self.timer.update_bytes(ADAM_COMPUTE, 28 * int(self._desc_host["numel"][:c.n_resident].sum()))
            if self._offload is not None:
                if tp:
                    self.timer.start_profile(ADAM_OFFLOAD)
                self._offload.run()
                if tp:
                    self.timer.finish_profile(ADAM_OFFLOAD)
            if tp:
                self.timer.finish_profile(ADAM)
            if old_scale is not None and self.read_ctrl().skip:
                logger.warning("Gradient overflow! Update loss scale from %s to %s.", old_scale, self._scaler.loss_scale)
        return loss

    def _update_torch_params(self, st):
        """The torch-managed parameters' share of the step (fp16_cpu_adam.py:345-353):
        one launch over a table of (param, fp32 grad, exp_avg, exp_avg_sq) rows that
        is rebuilt every step because autograd hands out a new ``.grad`` each time.
        Parameters without a gradient this step are left out, like every optimizer
        does."""
        if not self._torch:
            return
        rows = np.zeros(len(self._torch), dtype=TENSOR_DESC_DTYPE)
        n = 0
        for i, (name, p, gi, _) in enumerate(self._torch):
            g = p.grad
            if g is None:
                continue
            if g.dtype != torch.float32 or not g.is_cuda or not g.is_contiguous():
                raise TypeError("torch-managed parameter %s needs a contiguous CUDA fp32 gradient" % name)
            state = self.state[p]
            rows[n] = (p.data.data_ptr(), g.data_ptr(), state["exp_avg"].data_ptr(),
                       state["exp_avg_sq"].data_ptr(), p.numel(), self._torch_slots[i], 0)
            n += 1
        if n:
            check(lib.ps_tensor_table_step(rows.ctypes.data, n, len(self.param_groups) + 1,
                                           self._torch_table_dev.data_ptr(), self._ctrl.data_ptr(), st),
                  "ps_tensor_table_step")

    @torch.no_grad()
    def restore_fp16(self):
        """fp16 slot := half(fp32 master) for every resident local chunk, the
        restore of has_overflow_and_reset_param (fp16_cpu_adam.py:298-309) on its
        own (a skipped step does it by itself)."""
        n = self.client.n_resident
        if n:
            with torch.cuda.device(self.device):
                check(lib.ps_restore_fp16(self._desc_dev.data_ptr(), n, self._max_numel_resident,
                                          self._segs_dev.data_ptr(), self._stream()), "ps_restore_fp16")

    def rebalance(self, state_budget_bytes=None):
        """Re-decide which local chunks keep their fp32 state in HBM from the memory
        that is free now (``ChunkClient.rebalance``) and rebuild the device tables
        and the offload pipeline when the split changed.  The reference re-derives
        this before every step (fp16_cpu_adam.py:523-528); call it between steps."""
        if not self.client.rebalance(state_budget_bytes):
            return False
        self._offload = None
        self._build_tables()
        if self.client.n_resident < len(self.client.local_ids):
            from .offload import OffloadPipeline
            self._offload = OffloadPipeline(self.client, self)
        return True

    def _begin(self, grad_divisor, st):
        self._calls += 1
        self._ensure_pow_table(self._calls + 1)
        plan = self._plan(grad_divisor)
        check(lib.ps_step_begin(self._ctrl.data_ptr(), self._scaler.state_ptr, self._scaler.flag_ptr,
                                C.byref(plan), self._pow_table.data_ptr(), self._pow_len, st),
              "ps_step_begin")

    def _update_resident(self, st, first=0, count=None):
        n = self.client.n_resident - first if count is None else count
        if n <= 0:
            return
        off = first * CHUNK_DESC_DTYPE.itemsize
        check(lib.ps_chunk_step(self._desc_dev.data_ptr() + off, n, self._max_numel_resident,
                                self._segs_dev.data_ptr(), self._ctrl.data_ptr(), st), "ps_chunk_step")

    @torch.no_grad()
    def step_host_chunks(self, host_grads, host_params_out):
        """One step for a caller that keeps the fp16 chunks in (pinned) host memory,
        as the reference does for fp16 chunks it has evicted to the CPU
        (patrickstar/ops/chunk_io_buff.py:214-255 copies such a grad chunk to the
        compute device, :85-128 writes the params back).

        host_grads[k] / host_params_out[k]: pinned fp16 host tensors for the k-th
        local chunk.  Pipeline, no host synchronisation: chunk k's gradients are
        copied in on a side stream and scanned as they arrive; after the last one
        the skip decision is taken; then chunk k is updated and its fp16 params
        are copied out on a second side stream while chunk k+1 is updated.
        Single rank, resident chunks only."""
        c = self.client
        if c.world_size != 1 or self._offload is not None:
            raise NotImplementedError("step_host_chunks: single rank, all chunks resident")
        n = self._n_local
        if len(host_grads) != n or len(host_params_out) != n:
            raise ValueError("need one host tensor per local chunk")
        if getattr(self, "_io_streams", None) is None:
            self._io_streams = (torch.cuda.Stream(self.device), torch.cuda.Stream(self.device))
        s_in, s_out = self._io_streams
        main = torch.cuda.current_stream(self.device)
        item = CHUNK_DESC_DTYPE.itemsize
        with torch.cuda.device(self.device):
            st = self._stream()
            s_in.wait_stream(main)
            for k, cid in enumerate(c.local_ids):
                numel = int(self._desc_host["numel"][k])
                with torch.cuda.stream(s_in):
                    c.fp16_chunk(cid)[:numel].copy_(host_grads[k][:numel], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(s_in)
                main.wait_event(ev)
                if self._dynamic and numel:
                    check(lib.ps_overflow_scan(self._desc_dev.data_ptr() + k * item, 1, numel,
                                               self._scaler.flag_ptr, st), "ps_overflow_scan")
            self._begin(0, st)
            for k, cid in enumerate(c.local_ids):
                numel = int(self._desc_host["numel"][k])
                self._update_resident(st, first=k, count=1)
                ev = torch.cuda.Event()
                ev.record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev)
                    host_params_out[k][:numel].copy_(c.fp16_chunk(cid)[:numel], non_blocking=True)
            main.wait_stream(s_out)
        return None

    @torch.no_grad()
    def step_with_collectives(self, scan="local"):
        """The multi-GPU chunk step: per communication group a reduce-scatter of the
        fp16 grad chunks, the rank-local fused step, and an all-gather of the fp16
        param chunks (patrickstar/core/client.py:818-856, 428-497).

        ``scan="local"`` (default) is the reference's rule: the overflow test runs
        on this rank's own gradients BEFORE the reduction (patrickstar/core/hook.py:212)
        and the flag is MAX-all-reduced (fp16_cpu_adam.py:292-297).  The skip
        decision is then known before the first reduce-scatter, so the groups
        pipeline: reduce-scatter of group g+1, update of group g and all-gather of
        group g-1 are in flight together (two communicators, events between
        streams, no host synchronisation).

        ``scan="done"`` is ``"local"`` for a caller whose gradients were already
        tested when they were handed over (``handoff_grad``): only the flag
        all-reduce remains.

        ``scan="reduced"`` tests the reduced gradients instead (additionally
        catches an fp16 overflow created by the sum itself); every
        reduce-scatter must then finish before the first update."""
        c = self.client
        if c.world_size == 1:
            return self.step()
        if scan not in ("local", "reduced", "done"):
            raise ValueError("scan must be 'local', 'reduced' or 'done'")
        lay = c.layout
        n_groups = lay.n_groups_comm
        item = CHUNK_DESC_DTYPE.itemsize
        with torch.cuda.device(self.device):
            st = self._stream()
            if scan in ("local", "done"):
                if self._dynamic:
                    if scan == "local":
                        check(lib.ps_overflow_scan_buffer(c.fp16.data_ptr(), c.fp16.numel(),
                                                          self._scaler.flag_ptr, st), "ps_overflow_scan_buffer")
                    c.all_reduce_flag(self._scaler.flag_tensor)
                self._begin(c.world_size, st)
            # reduce-scatters already fired from the backward hand-off are only waited for
            fired, self._rs_fired, self._handed = self._rs_fired, {}, {}
            rs = [fired[g] if g in fired else c.reduce_scatter_group(g, async_op=True) for g in range(n_groups)]
            if scan == "reduced":
                for g in range(n_groups):
                    rs[g].wait()  # stream-level wait, not a host block
                    if self._dynamic:
                        check(lib.ps_overflow_scan(self._desc_dev.data_ptr() + g * item, 1, self._max_numel,
                                                   self._scaler.flag_ptr, st), "ps_overflow_scan")
                if self._dynamic:
                    c.all_reduce_flag(self._scaler.flag_tensor)
                self._begin(c.world_size, st)
            ag = []
            n_res = c.n_resident   # local chunk k belongs to communication group k
            for g in range(min(n_res, n_groups)):
                if scan != "reduced":
                    rs[g].wait()
                self._update_resident(st, first=g, count=1)
                ag.append(c.all_gather_group(g, async_op=True))
            if self._offload is not None:
                # hybrid placement: the groups whose local chunk keeps its fp32 state in
                # pinned host memory go through the offload pipeline once their reduced
                # gradients are in, and are gathered when it has drained (PCIe, at 14 ms
                # per chunk, dwarfs the 1-2 ms of their all-gathers)
                if scan != "reduced":
                    for g in range(n_res, n_groups):
                        rs[g].wait()
                self._offload.run()
                for g in range(n_res, n_groups):
                    ag.append(c.all_gather_group(g, async_op=True))
            self._update_torch_params(st)
            for w in ag:
                w.wait()
        return None

    @torch.no_grad()
    def step_fused_collectives(self, transport="multimem", scan="local"):
        """The multi-GPU chunk step as ONE kernel over NVSwitch multicast memory
        (needs ``ChunkClient(symmetric=True)``): the gradient of every owned
        element is loaded as the in-switch sum over all ranks' fp16 buffers — the
        reduce-scatter of patrickstar/core/client.py:818-856 — and the updated
        fp16 param is stored to all ranks' buffers — the all-gather of
        client.py:428-497.  Nothing crosses NVLink twice and no collective kernel
        runs beside the step.

        Order on every rank: overflow scan of the rank's own gradients (the
        reference's pre-reduction check, patrickstar/core/hook.py:212), MAX
        all-reduce of the flag (which is also the barrier "all gradients are
        written"), step-begin, the fused kernel over the owned chunks, a 4-byte
        all-reduce as the barrier "all params have arrived".

        ``transport="multimem"``: in-switch reduction and multicast stores;
        ``transport="p2p"``: peer loads summed in fp32 in rank order and peer
        stores (exact single rounding, no multicast object needed, cheaper on
        the links for 2-3 ranks, dearer for 8);
        ``transport="staged"``: the multimem form as a two-kernel pipeline — a light
        puller brings chunk k+1's reduced gradients into a local staging buffer
        while the step kernel updates chunk k (same results bit for bit);
        ``transport="copy"``: the copy engines pull the peers' gradients of chunk
        k+1 and push the params of chunk k-1 while a purely local kernel updates
        chunk k (same bits as "p2p"; the links run at the copy engines' rate);
        ``transport="copy_pull"``: the copy engines only pull; the kernel stores the
        params into every rank's buffer itself (posted peer stores).

        ``scan="done"``: the gradients were tested when they were handed over
        (``handoff_grad``), so the scan of the whole fp16 buffer is left out."""
        c = self.client
        if c.world_size == 1:
            return self.step()
        if c.symm_handle is None:
            raise RuntimeError("step_fused_collectives needs ChunkClient(symmetric=True)")
        if self._offload is not None:
            raise NotImplementedError("fused collectives with offloaded chunks")
        if scan not in ("local", "done"):
            raise ValueError("scan must be 'local' or 'done'")
        self._handed = {}
        mark = self.phase_marker or (lambda name: None)
        with torch.cuda.device(self.device):
            st = self._stream()
            if self._dynamic and scan == "local":
                check(lib.ps_overflow_scan_buffer(c.fp16.data_ptr(), c.fp16.numel(), self._scaler.flag_ptr, st),
                      "ps_overflow_scan_buffer")
            mark("scan")
            c.all_reduce_flag(self._scaler.flag_tensor)
            self._begin(c.world_size, st)
            mark("flag")
            if transport == "multimem":
                check(lib.ps_chunk_step_fused(self._desc_dev.data_ptr(), c.n_resident, self._max_numel_resident,
                                              self._segs_dev.data_ptr(), self._ctrl.data_ptr(), c.fp16.data_ptr(),
                                              c.fp16_multicast_ptr, c.peer_bases.data_ptr(), c.world_size, st),
                      "ps_chunk_step_fused")
            elif transport == "p2p":
                check(lib.ps_chunk_step_p2p(self._desc_dev.data_ptr(), c.n_resident, self._max_numel_resident,
                                            self._segs_dev.data_ptr(), self._ctrl.data_ptr(), c.fp16.data_ptr(),
                                            c.peer_bases.data_ptr(), c.world_size, st), "ps_chunk_step_p2p")
            elif transport == "staged":
                if getattr(self, "_fused_pipe", None) is None:
                    self._fused_pipe = C.c_void_p()
                    check(lib.ps_fused_pipe_create(C.byref(self._fused_pipe)), "ps_fused_pipe_create")
                    slot = (self._max_numel_resident + 7) // 8 * 8
                    self._fused_staging = torch.empty(2 * slot, dtype=torch.float16, device=self.device)
                check(lib.ps_chunk_step_fused_staged(self._fused_pipe, self._desc_dev.data_ptr(), c.n_resident,
                                                     self._max_numel_resident, self._segs_dev.data_ptr(),
                                                     self._ctrl.data_ptr(), c.fp16.data_ptr(),
                                                     c.fp16_multicast_ptr, c.peer_bases.data_ptr(),
                                                     c.world_size, self._fused_staging.data_ptr(), st),
                      "ps_chunk_step_fused_staged")
            elif transport in ("copy", "copy_pull"):
                if getattr(self, "_copy_pipe", None) is None:
                    self._copy_pipe = C.c_void_p()
                    n_slots = int(getattr(self, "copy_slots", 4))
                    check(lib.ps_copy_pipe_create(C.byref(self._copy_pipe), n_slots), "ps_copy_pipe_create")
                    slot = (self._max_numel_resident + 7) // 8 * 8
                    self._copy_staging = torch.empty(n_slots * (c.world_size - 1) * slot, dtype=torch.float16,
                                                     device=self.device)
                    self._copy_table = torch.empty(max(c.n_resident, 1) * c.world_size, dtype=torch.int64,
                                                   device=self.device)
                    self._peer_bases_host = (C.c_uint64 * c.world_size)(*[int(p) for p in c.symm_handle.buffer_ptrs])
                check(lib.ps_chunk_step_copy(self._copy_pipe, self._desc_dev.data_ptr(), self._desc_host.ctypes.data,
                                             c.n_resident, self._max_numel_resident, self._segs_dev.data_ptr(),
                                             self._ctrl.data_ptr(), c.fp16.data_ptr(), self._peer_bases_host,
                                             c.peer_bases.data_ptr() if transport == "copy_pull" else None,
                                             c.rank, c.world_size, self._copy_staging.data_ptr(),
                                             self._copy_table.data_ptr(), st), "ps_chunk_step_copy")
            else:
                raise ValueError("transport must be 'multimem', 'p2p', 'staged', 'copy' or 'copy_pull'")
            self._update_torch_params(st)
            mark("kernel")
            if getattr(self, "_barrier_buf", None) is None:
                self._barrier_buf = torch.zeros(1, dtype=torch.int32, device=self.device)
            c.all_reduce_flag(self._barrier_buf)
            mark("barrier")
        return None

    def reduced_gradients(self, transport="multimem", only=None):
        """What the fused kernel loads as gradients: per owned chunk the sum of all
        ranks' fp16 slots, in-switch ("multimem") or fp32-accumulated over peer
        loads ("p2p") (for tests; call between two barriers).  ``only``: local
        chunk indices to probe (default all)."""
        c = self.client
        cs = c.layout.chunk_size
        out = []
        with torch.cuda.device(self.device):
            for k, cid in enumerate(c.local_ids):
                if only is not None and k not in only:
                    continue
                dst = torch.empty(cs, dtype=torch.float16, device=self.device)
                if transport == "p2p":
                    check(lib.ps_p2p_reduce_probe(c.fp16.data_ptr() + 2 * cid * cs, c.fp16.data_ptr(),
                                                  c.peer_bases.data_ptr(), c.world_size, dst.data_ptr(), cs,
                                                  self._stream()), "ps_p2p_reduce_probe")
                else:
                    check(lib.ps_multimem_reduce_probe(c.fp16_multicast_ptr + 2 * cid * cs, dst.data_ptr(), cs,
                                                       self._stream()), "ps_multimem_reduce_probe")
                out.append(dst)
        return out

    def __del__(self):
        pipe = getattr(self, "_fused_pipe", None)
        if pipe is not None and pipe.value:
            lib.ps_fused_pipe_destroy(pipe)
            self._fused_pipe = None
        pipe = getattr(self, "_copy_pipe", None)
        if pipe is not None and pipe.value:
            lib.ps_copy_pipe_destroy(pipe)
            self._copy_pipe = None

    # --------------------------------------------------------------- inspection
    def read_ctrl(self) -> StepCtrl:
        out = StepCtrl()
        with torch.cuda.device(self.device):
            check(lib.ps_ctrl_read(self._ctrl.data_ptr(), C.byref(out), self._stream()), "ps_ctrl_read")
        if out.error:
            raise RuntimeError("device-side error word set: %d" % out.error)
        return out

    @property
    def step_count(self):
        """state["step"] of the reference: number of non-skipped steps (syncs)."""
        return int(self.read_ctrl().step)

    @property
    def skipped_steps(self):
        return int(self.read_ctrl().n_skipped)

    @property
    def params_per_step(self):
        """Number of parameters this rank updates per step."""
        return self._n_updated

    # --------------------------------------------------------------- checkpoint
    def state_dict(self):
        """fp16_cpu_adam.py:630-658 — per parameter: CPU clones of exp_avg /
        exp_avg_sq (local pieces), step, betas, lr, weight_decay, eps.  In addition
        (the reference forgets both) the loss-scaler state and the native
        beta^t history, so that a resumed run continues bit-exactly."""
        ctrl = self.read_ctrl()
        packed = {}
        idx = 0
        groups = []
        for group in self.param_groups:
            ids = []
            for p in group["params"]:
                st = self.state[p]
                entry = {k: st[k] for k in ("betas", "lr", "weight_decay", "eps")}
                entry["step"] = int(ctrl.step)
                for kind in ("exp_avg", "exp_avg_sq"):
                    if kind in st:   # torch-managed parameter: plain tensors
                        entry[kind] = st[kind].detach().cpu().clone()
                        continue
                    pieces = self.client.access_data(st["name"], kind)
                    numel = self.client.layout.tensor(st["name"]).numel
                    if pieces and sum(t.numel() for t, _ in pieces) == numel:
                        flat = torch.empty(numel, dtype=torch.float32)
                        for t, off in pieces:
                            flat[off:off + t.numel()] = t.detach().cpu()
                        entry[kind] = flat.view(p.shape)
                packed[idx] = entry
                ids.append(idx)
                idx += 1
            g = {k: v for k, v in group.items() if k != "params"}
            g["params"] = ids
            groups.append(g)
        return {
            "state": packed,
            "param_groups": groups,
            "loss_scaler": self._scaler.state_dict(),
            "native_clock": {"step": int(ctrl.step), "native_step": int(ctrl.native_step),
                             "betta1": ctrl.betta1, "betta2": ctrl.betta2,
                             "betta1_t": ctrl.betta1_t, "betta2_t": ctrl.betta2_t},
        }

    def load_state_dict(self, state_dict):
        """fp16_cpu_adam.py:660-694 — by parameter order."""
        state_dict = deepcopy(state_dict)
        saved_groups = state_dict["param_groups"]
        saved_state = state_dict["state"]
        assert len(saved_groups) == len(self.param_groups)
        step = None
        for sg, group in zip(saved_groups, self.param_groups):
            assert len(sg["params"]) == len(group["params"])
            for old_id, p in zip(sg["params"], group["params"]):
                saved = saved_state[old_id]
                st = self.state[p]
                for k in ("betas", "lr", "weight_decay", "eps"):
                    st[k] = saved[k]
                step = saved["step"] if step is None else step
                for kind in ("exp_avg", "exp_avg_sq"):
                    if kind in saved and kind in st:
                        st[kind].copy_(saved[kind])
                    elif kind in saved:
                        flat = saved[kind].reshape(-1)
                        for t, off in self.client.access_data(st["name"], kind):
                            t.copy_(flat[off:off + t.numel()])
        with torch.cuda.device(self.device):
            clk = state_dict.get("native_clock")
            b1, b2 = self.param_groups[0]["betas"]
            check(lib.ps_ctrl_init(self._ctrl.data_ptr(), int(step or 0), b1, b2, self._stream()),
                  "ps_ctrl_init")
            if clk is not None:
                host = self.read_ctrl()
                host.native_step = clk["native_step"]
                host.betta1, host.betta2 = clk["betta1"], clk["betta2"]
                host.betta1_t, host.betta2_t = clk["betta1_t"], clk["betta2_t"]
                buf = torch.frombuffer(bytearray(bytes(host)), dtype=torch.uint8)
                self._ctrl.copy_(buf)
        if "loss_scaler" in state_dict and self.loss_scaler is not None:
            self._scaler.load_state_dict(state_dict["loss_scaler"])
        self._calls = max(self._calls, int(step or 0))
        self._pow_len = 0
        self._ensure_pow_table(self._calls + 1)
