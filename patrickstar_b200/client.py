"""Chunk manager for the optimizer step.

The slice of ``PatrickStarClient`` (patrickstar/core/client.py) the optimizer
step touches: it owns the chunk payloads, hands out tensor views into them
(``access_data``), says which chunks are local, and runs the two chunk
collectives of a communication group (reduce-scatter of fp16 grads
client.py:818-856, all-gather of fp16 params client.py:428-497).

Memory layout on one GPU
  * ``fp16`` — ONE contiguous fp16 buffer of ``n_chunks * chunk_size`` elements
    holding every chunk of the list, local and remote, in chunk order.  Chunk k
    of communication group g is slice ``k % world`` of the group's contiguous
    ``world * chunk_size`` run, so reduce-scatter and all-gather run in place
    on it with no flatten copy.  Parameters are views into this buffer; their
    storage receives the gradients after backward
    (patrickstar/core/hook.py:214-216) and the updated fp16 params after the
    step.
  * ``p32`` / ``exp_avg`` / ``exp_avg_sq`` — fp32 master, momentum, variance of
    the LOCAL chunks only (patrickstar/ops/fp16_cpu_adam.py:132-170), laid out
    like the fp16 chunk.  The first ``n_resident`` local chunks live in HBM;
    the rest ("hybrid" placement, fp16_cpu_adam.py:523-528) live in pinned host
    memory and are streamed through staging slots by the offload pipeline.
"""
import torch

from . import comm
from .chunk_list import ChunkLayout, DEFAULT_CHUNK_SIZE


class ChunkClient:
    def __init__(self, rank=0, default_chunk_size=DEFAULT_CHUNK_SIZE, config=None, world_size=None,
                 device=None, pack="no_split", process_group=None, symmetric=False, rs_max_ctas=None):
        if not torch.cuda.is_available():
            raise RuntimeError("patrickstar_b200 needs a CUDA device (sm_100a); none found")
        self.local_rank = rank
        # symmetric=True: the fp16 chunk buffer is allocated as NVSwitch multicast
        # ("symmetric") memory, which the fused reduce-scatter + step + all-gather
        # kernel needs; plain device memory otherwise
        self.symmetric = bool(symmetric)
        self.symm_handle = None
        if world_size is None:
            world_size = (torch.distributed.get_world_size(process_group)
                          if torch.distributed.is_available() and torch.distributed.is_initialized() else 1)
        self.world_size = world_size
        self.rank = (torch.distributed.get_rank(process_group)
                     if world_size > 1 and torch.distributed.is_initialized() else 0)
        self.process_group = process_group
        # Separate communicators for the two chunk collectives, so that the
        # reduce-scatter of one communication group and the all-gather of another
        # can be in flight together (collectives of one communicator serialise).
        self.pg_reduce_scatter = self.pg_all_gather = process_group
        if world_size > 1 and torch.distributed.is_initialized():
            ranks = torch.distributed.get_process_group_ranks(
                process_group if process_group is not None else torch.distributed.group.WORLD)
            rs_options = None
            if rs_max_ctas:
                # a reduce-scatter fired from the backward hand-off runs beside backward's
                # compute kernels: capping its CTAs leaves them the SMs
                rs_options = torch.distributed.ProcessGroupNCCL.Options()
                rs_options.config.max_ctas = int(rs_max_ctas)
            self.pg_reduce_scatter = torch.distributed.new_group(ranks, pg_options=rs_options)
            self.pg_all_gather = torch.distributed.new_group(ranks)
        self.device = torch.device("cuda", rank) if device is None else torch.device(device)
        self.config = config or {}
        self.layout = ChunkLayout(default_chunk_size, world_size, pack)
        self.default_chunk_size = default_chunk_size
        self.params = {}      # name -> fp16 nn.Parameter view
        self.fp16 = None
        self.p32 = self.exp_avg = self.exp_avg_sq = None          # device-resident local chunks
        # offloaded local chunks: one pinned host tensor per chunk and kind (None when there are none)
        self.p32_host = self.exp_avg_host = self.exp_avg_sq_host = None
        self.n_resident = 0
        self._budget = None   # what allocate() was given: None, bytes, or "auto"
        self.local_ids = []
        self._pending = []    # (name, nn.Parameter) registered from a module, placed at allocate()
        # parameters managed by torch instead of the chunk list (the reference's TORCH_BASED
        # kind, patrickstar/core/preprocess.py:351-369): name -> (fp32 nn.Parameter, number of
        # chunk tensors registered before it, i.e. its place in the optimizer's visiting order)
        self.torch_params = {}

    # ------------------------------------------------------------- registration
    def append_tensor_list(self, specs, shapes=None):
        return self.layout.append_tensor_list(specs, shapes)

    def append_tensor(self, name, numel, group=0, shape=None):
        return self.layout.append_tensor(name, numel, group, shape)

    def append_torch_param(self, name, param):
        """Register a parameter that stays outside the chunk list: fp32, updated in
        place from its fp32 ``.grad``, no fp16 slot (the reference keeps the
        CPU-embedding weights this way, patrickstar/core/preprocess.py:351-369,
        patrickstar/ops/fp16_cpu_adam.py:345-353).  Its place in the optimizer's
        visiting order is after the chunk tensors registered so far."""
        if name in self.torch_params or name in self.layout._by_name:
            raise ValueError("duplicate tensor name %r" % name)
        if self.layout._frozen:
            raise RuntimeError("layout is frozen")
        self.torch_params[name] = (param, len(self.layout.tensors))
        return param

    def register_module(self, module, group_of=None, torch_based=None):
        """Register every parameter of an nn.Module, one atomic list per
        sub-module as the reference's pre-process context does
        (patrickstar/core/preprocess.py:341-435).  ``group_of(name, param)``
        gives the hyper-parameter group index (default 0); parameters for which
        ``torch_based(name, param)`` is true stay outside the chunk list as fp32
        torch parameters (``append_torch_param``)."""
        for mod_name, mod in module.named_modules():
            specs, shapes, plist = [], [], []
            for pname, p in mod.named_parameters(recurse=False):
                full = (mod_name + "." if mod_name else "") + pname
                if torch_based is not None and torch_based(full, p):
                    if specs:   # keep the visiting order: flush the chunk tensors seen so far
                        self.layout.append_tensor_list(specs, shapes)
                        self._pending.extend(plist)
                        specs, shapes, plist = [], [], []
                    self.append_torch_param(full, p)
                    continue
                g = group_of(full, p) if group_of else 0
                specs.append((full, p.numel(), g))
                shapes.append(tuple(p.shape))
                plist.append((full, p))
            if specs:
                self.layout.append_tensor_list(specs, shapes)
                self._pending.extend(plist)
        return self

    # ---------------------------------------------------------------- allocation
    def allocate(self, state_budget_bytes=None, init_master_from_fp16=True):
        """Freeze the layout and allocate the payloads.  ``state_budget_bytes``
        caps the HBM spent on fp32 master/momentum/variance chunks; local chunks
        beyond it are placed in pinned host memory (hybrid placement)."""
        lay = self.layout.freeze()
        cs = lay.chunk_size
        self.local_ids = lay.local_chunk_ids(self.rank)
        n_local = len(self.local_ids)
        self._budget = state_budget_bytes
        # the fp16 chunk list is allocated below: it comes out of what is free now
        self.n_resident = self._derive_n_resident(state_budget_bytes, reserve=2 * lay.n_chunks * cs)
        n_off = n_local - self.n_resident
        dev = self.device
        if self.symmetric and self.world_size > 1:
            import torch.distributed._symmetric_memory as symm_mem
            group = self.process_group if self.process_group is not None else torch.distributed.group.WORLD
            self.fp16 = symm_mem.empty(lay.n_chunks * cs, dtype=torch.float16, device=dev)
            self.fp16.zero_()
            self.symm_handle = symm_mem.rendezvous(self.fp16, group)
            self.fp16_multicast_ptr = int(self.symm_handle.multicast_ptr)
            if self.fp16_multicast_ptr == 0:
                raise RuntimeError("NVSwitch multicast is not available for this group of GPUs")
            self.peer_bases = torch.tensor([int(p) for p in self.symm_handle.buffer_ptrs],
                                           dtype=torch.int64, device=dev)
        else:
            self.fp16 = torch.zeros(lay.n_chunks * cs, dtype=torch.float16, device=dev)

        def dev_buf():
            return torch.zeros(max(self.n_resident, 0) * cs, dtype=torch.float32, device=dev)

        def host_buf():
            return self._pinned_chunks(n_off, zero=True)

        self.p32, self.exp_avg, self.exp_avg_sq = dev_buf(), dev_buf(), dev_buf()
        self.p32_host, self.exp_avg_host, self.exp_avg_sq_host = host_buf(), host_buf(), host_buf()
        # parameters registered from a module: move their values into the chunks
        for full, p in self._pending:
            info = lay.tensor(full)
            view = self.fp16_view(info)
            view.copy_(p.detach().to(device=dev, dtype=torch.float16).reshape(-1))
            p.data = view.view(p.shape)
            self.params[full] = p
        if not self._pending:
            # tensors registered by shape only: parameters are views of the fp16 buffer
            for info in lay.tensors:
                view = self.fp16_view(info).view(info.shape)
                self.params[info.name] = torch.nn.Parameter(view, requires_grad=False)
        if init_master_from_fp16 and self._pending:
            for k, c in enumerate(self.local_ids):
                self.chunk_state(k)[0].copy_(self.fp16_chunk(c).float())
        self._pending = []
        for name, (p, _) in self.torch_params.items():
            p.data = p.data.to(device=dev, dtype=torch.float32)
        return self

    def _pinned_chunks(self, n, zero=False):
        """``n`` chunk-sized fp32 buffers in pinned host memory, or None for n = 0.
        One allocation per chunk, made pinned at once: torch's pinned-memory
        allocator rounds every request up to a power of two, which for one buffer
        of tens of GiB per rank would waste up to as much again."""
        if n <= 0:
            return None
        make = torch.zeros if zero else torch.empty
        return [make(self.layout.chunk_size, dtype=torch.float32, pin_memory=True) for _ in range(n)]

    def _derive_n_resident(self, budget, reserve=0, held=0):
        """How many local chunks keep their fp32 state in HBM.  ``None``: all;
        a number: that many bytes; ``"auto"``: what the reference derives from its
        memory tracer every step — the chunks that fit into the GPU memory left
        over, scaled by margin_use_ratio
        (patrickstar/core/memtracer/memtracer.py:190-227, default ratio 0.8).
        ``reserve`` bytes are about to be allocated by the caller, ``held`` bytes of
        state are already in HBM and count as available."""
        n_local = len(self.local_ids)
        per_chunk = 3 * 4 * self.layout.chunk_size
        if budget is None:
            return n_local
        if budget == "auto":
            ratio = (self.config.get("mem_tracer", {}) or {}).get("margin_use_ratio", 0.8)
            free, _ = self.mem_get_info(self.device)
            return max(0, min(n_local, int((free - reserve + held) * ratio) // per_chunk))
        return max(0, min(n_local, int(budget) // per_chunk))

    @staticmethod
    def mem_get_info(device):
        """(bytes this process can still place on the device, total bytes): what the
        driver reports free plus what torch's caching allocator holds but is not
        using (it hands that out again before asking the driver).  Replaced by
        tests to play a device that is short of memory."""
        free, total = torch.cuda.mem_get_info(device)
        cached = torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
        return free + max(0, cached), total

    def rebalance(self, state_budget_bytes=None):
        """Re-derive the hybrid placement from the memory that is free NOW and move
        chunk states between HBM and pinned host memory accordingly — what the
        reference does before every step (``margin_chunk_num_for_gpu_adam``,
        patrickstar/ops/fp16_cpu_adam.py:523-528; the chunk moves themselves happen
        in patrickstar/core/chunk_data.py:275-366).  ``state_budget_bytes``
        defaults to what ``allocate`` was given.  Returns True when the split
        changed; the optimizer then has to rebuild its tables
        (``FP16Adam.rebalance`` does both)."""
        budget = self._budget if state_budget_bytes is None else state_budget_bytes
        if budget is None:
            return False
        cs = self.layout.chunk_size
        old = self.n_resident
        new = self._derive_n_resident(budget, held=3 * 4 * cs * old)
        self._budget = budget
        if new == old:
            return False
        dev = self.device
        torch.cuda.current_stream(dev).synchronize()   # no step may be in flight on the states
        names = ("p32", "exp_avg", "exp_avg_sq")
        for name in names:   # one kind at a time: the transient extra HBM is one third of the state
            d_old, h_old = getattr(self, name), getattr(self, name + "_host") or []
            d_new = torch.empty(new * cs, dtype=torch.float32, device=dev)
            keep = min(old, new)
            d_new[:keep * cs].copy_(d_old[:keep * cs])
            if new > old:    # chunks old..new-1 come up from the host
                for i in range(new - old):
                    d_new[(old + i) * cs:(old + i + 1) * cs].copy_(h_old[i])
                h_new = h_old[new - old:]
            else:            # chunks new..old-1 go down to the host
                h_new = self._pinned_chunks(old - new)
                for i in range(old - new):
                    h_new[i].copy_(d_old[(new + i) * cs:(new + i + 1) * cs])
                h_new = h_new + list(h_old)
            torch.cuda.current_stream(dev).synchronize()
            setattr(self, name, d_new)
            setattr(self, name + "_host", h_new or None)
            del d_old, h_old
        self.n_resident = new
        return True

    # -------------------------------------------------------------------- views
    def fp16_chunk(self, chunk_id):
        cs = self.layout.chunk_size
        return self.fp16[chunk_id * cs:(chunk_id + 1) * cs]

    def fp16_group(self, group_id):
        n = self.layout.chunk_size * self.world_size
        return self.fp16[group_id * n:(group_id + 1) * n]

    def fp16_view(self, info):
        s = info.flat_start(self.layout.chunk_size)
        return self.fp16[s:s + info.numel]

    def chunk_state(self, local_index):
        """(p32, exp_avg, exp_avg_sq) chunk views of the local_index-th local chunk;
        device tensors for resident chunks, pinned host tensors for offloaded ones."""
        cs = self.layout.chunk_size
        if local_index < self.n_resident:
            sl = slice(local_index * cs, (local_index + 1) * cs)
            return self.p32[sl], self.exp_avg[sl], self.exp_avg_sq[sl]
        k = local_index - self.n_resident
        return self.p32_host[k], self.exp_avg_host[k], self.exp_avg_sq_host[k]

    def is_local(self, name):
        """True when every element of the tensor lies in chunks this rank owns."""
        info = self.layout.tensor(name)
        cs = self.layout.chunk_size
        first = info.chunk_id
        last = (info.flat_start(cs) + max(info.numel, 1) - 1) // cs
        return all(self.layout.is_local(c, self.rank) for c in range(first, last + 1))

    def access_data(self, name, kind="p32"):
        """Views of one tensor's optimizer state, one per chunk piece:
        list of (tensor_view, flat_offset_in_tensor).  ``kind`` is ``p32``,
        ``exp_avg`` or ``exp_avg_sq``.  Only the pieces in local chunks are
        returned (client.py access_data on a CHUNK_BASED fp32 param)."""
        idx = {"p32": 0, "exp_avg": 1, "exp_avg_sq": 2}[kind]
        info = self.layout.tensor(name)
        cs = self.layout.chunk_size
        out = []
        c, off, rest, done = info.chunk_id, info.start_offset, info.numel, 0
        while rest > 0:
            take = min(rest, cs - off)
            if self.layout.is_local(c, self.rank):
                k = self.local_ids.index(c)
                out.append((self.chunk_state(k)[idx][off:off + take], done))
            rest -= take
            done += take
            c += 1
            off = 0
        return out

    # -------------------------------------------------------------- collectives
    def reduce_scatter_group(self, group_id, async_op=False):
        """SUM reduce-scatter of one communication group's fp16 chunks, in place
        (see ``comm.reduce_scatter_group``)."""
        if self.world_size == 1:
            return None
        return comm.reduce_scatter_group(self.fp16_group(group_id), self.rank, self.world_size,
                                         self.layout.chunk_size, self.pg_reduce_scatter, async_op)

    def all_gather_group(self, group_id, async_op=False):
        """All-gather of one communication group's fp16 param chunks, in place."""
        if self.world_size == 1:
            return None
        return comm.all_gather_group(self.fp16_group(group_id), self.rank, self.world_size,
                                     self.layout.chunk_size, self.pg_all_gather, async_op)

    def all_reduce_flag(self, flag):
        """MAX all-reduce of the overflow flag; stays on the device (the reference
        follows it with `.item()`, fp16_cpu_adam.py:297)."""
        if self.world_size == 1:
            return
        comm.all_reduce_flag(flag, self.process_group)
