"""Host side of the offload tier: which local chunks are streamed, their staging
slots and descriptors.  The pipeline itself (streams, events, copies, kernel
launches) is native: ``ps_offload_step`` in ``csrc/ps_offload.cu``.

The reference decides per step how many chunks fit on the GPU for Adam
(``margin_chunk_num_for_gpu_adam``, patrickstar/ops/fp16_cpu_adam.py:523-528)
and updates the others with its CPU Adam.  Here the split is decided at
allocation (``ChunkClient.allocate(state_budget_bytes=...)``) and re-decided on
request between steps (``FP16Adam.rebalance``): the first ``n_resident`` local
chunks stay in HBM, the others live in pinned host memory and are updated by
the same GPU kernel through ``n_slots`` staging slots.
"""
import ctypes as C

import numpy as np
import torch

from ._lib import CHUNK_DESC_DTYPE, OFFLOAD_CHUNK_DTYPE, check, lib


class OffloadPipeline:
    def __init__(self, client, optimizer, n_slots=2, piece_elems=16 * 1024 * 1024):
        """n_slots staging slots (2 = double buffering), each 3 fp32 buffers of
        `piece_elems` elements: a chunk is streamed in pieces of that size, which
        keeps the pipeline's fill and drain (one copy in, one copy out) short."""
        self.client = client
        self.opt = optimizer
        self.n_slots = n_slots
        cs = client.layout.chunk_size
        dev = client.device
        n_off = len(client.local_ids) - client.n_resident
        self.n_off = n_off
        piece = min(cs, max(2048, (piece_elems // 2048) * 2048))
        self.piece_elems = piece
        self.staging = [[torch.empty(piece, dtype=torch.float32, device=dev) for _ in range(3)]
                        for _ in range(n_slots)]
        self._staging_ptrs = (C.c_void_p * (3 * n_slots))(
            *[t.data_ptr() for slot in self.staging for t in slot])
        base = optimizer._desc_host
        n_local = len(base)
        rows, jobs = [], []
        i = 0
        for k in range(client.n_resident, n_local):
            numel = int(base["numel"][k])
            p, m, v = client.chunk_state(k)
            for first in range(0, numel, piece):
                count = min(piece, numel - first)
                s = i % n_slots
                d = base[k].copy()
                d["p32"], d["exp_avg"], d["exp_avg_sq"] = (t.data_ptr() - 4 * first for t in self.staging[s])
                d["numel"] = first + count
                d["reserved"] = first
                rows.append(d)
                jobs.append((p.data_ptr() + 4 * first, m.data_ptr() + 4 * first, v.data_ptr() + 4 * first,
                             count, n_local + i))
                i += 1
        self._jobs = np.array(jobs, dtype=OFFLOAD_CHUNK_DTYPE) if jobs else np.zeros(0, dtype=OFFLOAD_CHUNK_DTYPE)
        self.n_pieces = len(jobs)
        # the resident chunks' descriptors are validated as a table; the piece descriptors
        # share their chunk's (validated) segment range and only narrow [first, numel)
        if client.n_resident:
            check(lib.ps_table_check(base.ctypes.data, client.n_resident, optimizer._segs_host.ctypes.data,
                                     len(optimizer._segs_host), len(optimizer.param_groups) + 1, cs),
                  "ps_table_check")
        if rows:
            # the piece rows too: biased state pointers, first element (`reserved`) and length
            piece_rows = np.array(rows, dtype=CHUNK_DESC_DTYPE)
            check(lib.ps_piece_table_check(piece_rows.ctypes.data, len(piece_rows), len(optimizer._segs_host), cs),
                  "ps_piece_table_check")
        desc = np.concatenate([base, np.array(rows, dtype=CHUNK_DESC_DTYPE)]) if rows else base
        optimizer._desc_host = desc
        optimizer._desc_dev = torch.from_numpy(desc.view(np.uint8).copy()).to(dev)
        self._handle = C.c_void_p()
        with torch.cuda.device(dev):
            check(lib.ps_offload_create(C.byref(self._handle), n_slots), "ps_offload_create")

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h is not None and h.value:
            lib.ps_offload_destroy(h)
            self._handle = C.c_void_p()

    def run(self):
        """Enqueue the streamed update of every offloaded chunk (after ps_step_begin)."""
        if self.n_off == 0:
            return
        opt = self.opt
        with torch.cuda.device(self.client.device):
            check(lib.ps_offload_step(self._handle, self._jobs.ctypes.data, self.n_pieces, self._staging_ptrs,
                                      opt._desc_dev.data_ptr(), opt._segs_dev.data_ptr(),
                                      opt._ctrl.data_ptr(), opt._stream()), "ps_offload_step")
