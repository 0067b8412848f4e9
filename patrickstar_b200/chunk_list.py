"""Chunk-tensor index and chunk list: where every parameter lives.

A minimal restatement of the two host indices the optimizer step reads in the
reference — ``ChunkTensorIndex`` (patrickstar/core/chunk_tensor_index.py) and
``ChunkList`` (patrickstar/core/chunk_list.py) — reduced to what the step needs:
the tensor -> (chunk, offset, numel) map, chunk ownership, and from them the
device tables the kernels take (``ps_chunk_desc`` / ``ps_segment``).  The
dynamic move/evict state machine of the reference serves forward/backward and
is not rebuilt here.

Packing rules
  * ``no_split`` — the reference's rule: a tensor never straddles a chunk; a
    list of tensors (one module's parameters) goes into the current chunk as a
    whole or opens a new one (chunk_tensor_index.py:239-264,
    patrickstar/core/client.py:246-309).  A tensor larger than a chunk raises,
    as in the reference (client.py:272-279).
  * ``flat`` — tensors are concatenated in order and cut at chunk boundaries, so
    tensors (and param-group segments) may straddle chunks.  Needed for models
    whose single tensors exceed the chunk size.

Ownership (chunk_list.py:377-392, chunk_tensor_index.py:115-125): the k-th
chunk belongs to rank ``k % world`` and to communication group ``k // world``;
the list is padded with dummy chunks to a multiple of ``world``
(patrickstar/core/preprocess.py:335-339).
"""
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np

DEFAULT_CHUNK_SIZE = 32 * 1024 * 1024  # patrickstar/runtime/__init__.py:37


@dataclass
class TensorInfo:
    """chunk_tensor_index.py TensorInfo: one parameter's place in the chunk list."""
    name: str
    numel: int
    group: int          # hyper-parameter group index
    chunk_id: int       # chunk holding the first element
    start_offset: int   # offset of the first element inside that chunk
    shape: Tuple[int, ...] = ()

    def flat_start(self, chunk_size):
        return self.chunk_id * chunk_size + self.start_offset


@dataclass
class CommInfo:
    """chunk_list.py:383-387."""
    group_id: int
    offset: int


@dataclass
class Piece:
    """A maximal run of elements of one chunk with one hyper-parameter group."""
    chunk_id: int
    start: int
    end: int
    group: int
    tensor_index: int = -1   # position of the piece's tensor in registration order


class ChunkLayout:
    """Host-only index: packing, ownership and the segment lists."""

    def __init__(self, chunk_size=DEFAULT_CHUNK_SIZE, world_size=1, pack="no_split"):
        if chunk_size <= 0 or chunk_size >= 0x7fffff00:
            raise ValueError("chunk_size out of range: %r" % (chunk_size,))
        if pack not in ("no_split", "flat"):
            raise ValueError("pack must be 'no_split' or 'flat'")
        if world_size < 1:
            raise ValueError("world_size must be >= 1")
        self.chunk_size = int(chunk_size)
        self.world_size = int(world_size)
        self.pack = pack
        self.tensors: List[TensorInfo] = []
        self._by_name = {}
        self._n_chunks = 0          # chunks holding tensors
        self._fill = 0              # used elements of the last chunk
        self._frozen = False
        self._piece_cache = None    # filled once the layout is frozen
        self._by_chunk = None

    # ------------------------------------------------------------------ packing
    def append_tensor_list(self, specs: Sequence[Tuple[str, int, int]], shapes=None):
        """Append (name, numel, group) tuples atomically (no_split) or in order
        (flat).  Returns the TensorInfo list."""
        if self._frozen:
            raise RuntimeError("layout is frozen")
        for name, numel, _ in specs:
            if name in self._by_name:
                raise ValueError("duplicate tensor name %r" % name)
            if numel < 0:
                raise ValueError("negative numel for %r" % name)
        out = []
        if self.pack == "no_split":
            total = sum(n for _, n, _ in specs)
            for name, numel, _ in specs:
                if numel > self.chunk_size:
                    raise RuntimeError(
                        "tensor %s (%d elements) is larger than the chunk size %d; raise "
                        "default_chunk_size or use pack='flat'" % (name, numel, self.chunk_size))
            if self._n_chunks == 0 or (self.chunk_size - self._fill < total and total <= self.chunk_size):
                self._n_chunks += 1
                self._fill = 0
            for i, (name, numel, group) in enumerate(specs):
                if self.chunk_size - self._fill < numel:
                    # a list that cannot fit one chunk as a whole spills tensor by tensor
                    self._n_chunks += 1
                    self._fill = 0
                info = TensorInfo(name, int(numel), int(group), self._n_chunks - 1, self._fill,
                                  tuple(shapes[i]) if shapes else (int(numel),))
                self._fill += int(numel)
                out.append(info)
        else:
            for i, (name, numel, group) in enumerate(specs):
                if self._n_chunks == 0 or self._fill == self.chunk_size:
                    self._n_chunks += 1
                    self._fill = 0
                info = TensorInfo(name, int(numel), int(group), self._n_chunks - 1, self._fill,
                                  tuple(shapes[i]) if shapes else (int(numel),))
                rest = int(numel)
                while rest > 0:
                    if self._fill == self.chunk_size:
                        self._n_chunks += 1
                        self._fill = 0
                    take = min(rest, self.chunk_size - self._fill)
                    self._fill += take
                    rest -= take
                out.append(info)
        for info in out:
            self.tensors.append(info)
            self._by_name[info.name] = info
        return out

    def append_tensor(self, name, numel, group=0, shape=None):
        return self.append_tensor_list([(name, numel, group)], [shape] if shape else None)[0]

    def freeze(self):
        self._frozen = True
        return self

    def set_group(self, name, group):
        """Re-assign a tensor's hyper-parameter group (the optimizer's param groups
        decide it) and drop the cached segment lists."""
        self._by_name[name].group = int(group)
        self._piece_cache = None
        self._by_chunk = None

    # ---------------------------------------------------------------- geometry
    @property
    def n_data_chunks(self):
        return self._n_chunks

    @property
    def n_chunks(self):
        """Chunk count including the dummy chunks that pad to a multiple of world."""
        w = self.world_size
        return ((self._n_chunks + w - 1) // w) * w

    @property
    def n_groups_comm(self):
        return self.n_chunks // self.world_size

    def comm_info(self, chunk_id) -> CommInfo:
        return CommInfo(group_id=chunk_id // self.world_size, offset=chunk_id % self.world_size)

    def is_local(self, chunk_id, rank):
        return chunk_id % self.world_size == rank

    def is_dummy(self, chunk_id):
        return chunk_id >= self._n_chunks

    def local_chunk_ids(self, rank) -> List[int]:
        return [c for c in range(self.n_chunks) if self.is_local(c, rank)]

    def chunk_numel(self, chunk_id) -> int:
        """Elements in use in a chunk (end of its last tensor)."""
        if chunk_id >= self._n_chunks:
            return 0
        if chunk_id < self._n_chunks - 1 and self.pack == "flat":
            return self.chunk_size
        end = 0
        for p in self.pieces_of_chunk(chunk_id):
            end = max(end, p.end)
        return end

    def tensor(self, name) -> TensorInfo:
        return self._by_name[name]

    def add_to_comm_groups(self, info: TensorInfo, acc: dict):
        """Add a tensor's elements to ``acc[communication group]``, cut at chunk
        boundaries (a tensor may straddle chunks and groups).  Summed over all
        tensors this is the number of gradient elements a group must have received
        before its reduce-scatter may start (patrickstar/core/client.py:793-817
        waits for every tensor of the group's chunks to be HOLD_AFTER_BWD)."""
        cs, w = self.chunk_size, self.world_size
        pos, rest = info.flat_start(cs), info.numel
        while rest > 0:
            take = min(rest, cs - pos % cs)
            g = (pos // cs) // w
            acc[g] = acc.get(g, 0) + take
            pos += take
            rest -= take
        return acc

    def total_numel(self):
        return sum(t.numel for t in self.tensors)

    # ---------------------------------------------------------------- segments
    def _pieces(self) -> List[Piece]:
        """Every tensor cut at chunk boundaries, in storage order."""
        if getattr(self, "_piece_cache", None) is not None and self._frozen:
            return self._piece_cache
        out = []
        cs = self.chunk_size
        for ti, t in enumerate(self.tensors):
            c, off, rest = t.chunk_id, t.start_offset, t.numel
            while rest > 0:
                take = min(rest, cs - off)
                out.append(Piece(c, off, off + take, t.group, ti))
                rest -= take
                c += 1
                off = 0
        if self._frozen:
            self._piece_cache = out
        return out

    def pieces_of_chunk(self, chunk_id) -> List[Piece]:
        if getattr(self, "_by_chunk", None) is None or not self._frozen:
            by = {}
            for p in self._pieces():
                by.setdefault(p.chunk_id, []).append(p)
            for v in by.values():
                v.sort(key=lambda p: p.start)
            if not self._frozen:
                return by.get(chunk_id, [])
            self._by_chunk = by
        return self._by_chunk.get(chunk_id, [])

    def calls_of_rank(self, rank) -> List[Piece]:
        """The per-tensor pieces a rank visits in one step, in the reference's
        order (storage order of its local chunks; fp16_cpu_adam.py:569-606).  One
        entry per adam_update call the reference would make."""
        out = []
        for c in self.local_chunk_ids(rank):
            out.extend(self.pieces_of_chunk(c))
        return out

    def segments_of_chunk(self, chunk_id) -> List[Piece]:
        """Pieces of a chunk with adjacent pieces of the same group merged."""
        out: List[Piece] = []
        for p in self.pieces_of_chunk(chunk_id):
            if out and out[-1].end == p.start and out[-1].group == p.group:
                out[-1] = Piece(chunk_id, out[-1].start, p.end, p.group)
            else:
                out.append(Piece(chunk_id, p.start, p.end, p.group))
        return out

    def build_tables(self, rank, first_call_slot=True):
        """Segment table and per-chunk segment ranges for a rank's local chunks.

        Returns (local_chunk_ids, numels, seg_ranges, segments) where segments is
        a numpy array of SEGMENT_DTYPE-compatible rows (start, end, slot) and
        slot = 1 + group, except that the very first piece the rank visits gets
        slot 0: the reference's first adam_update call of a step sees a
        different beta^t than the later ones
        (patrickstar/ops/csrc/includes/cpu_adam.h:143-162)."""
        local = self.local_chunk_ids(rank)
        calls = self.calls_of_rank(rank)
        first = calls[0] if calls else None
        rows = []
        ranges = []
        numels = []
        for c in local:
            begin = len(rows)
            segs = self.segments_of_chunk(c)
            if first_call_slot and first is not None and c == first.chunk_id and len(calls) >= 2:
                # split the first piece off so that it can carry slot 0
                split = []
                for s in segs:
                    if s.start == first.start and s.end > first.end:
                        split.append(Piece(c, first.start, first.end, -1))
                        split.append(Piece(c, first.end, s.end, s.group))
                    elif s.start == first.start:
                        split.append(Piece(c, s.start, s.end, -1))
                    else:
                        split.append(s)
                segs = split
            elif first_call_slot and first is not None and c == first.chunk_id:
                segs = [Piece(c, s.start, s.end, -1) if s.start == first.start else s for s in segs]
            for s in segs:
                rows.append((s.start, s.end, 0 if s.group < 0 else 1 + s.group, 0))
            ranges.append((begin, len(rows)))
            numels.append(self.chunk_numel(c))
        seg_arr = np.array(rows, dtype=np.uint32).reshape(-1, 4)
        return local, numels, ranges, seg_arr

    def plan_groups(self, rank):
        """(first_group, last_group, n_calls) of a rank's call sequence."""
        calls = self.calls_of_rank(rank)
        if not calls:
            return 0, 0, 0
        return calls[0].group, calls[-1].group, len(calls)
