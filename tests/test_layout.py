"""Chunk layout: packing rules, ownership, segment tables (host logic only).
Modelled on the reference's unitest/test_chunk_tensor_index.py and
unitest/test_chunk_data.py."""
import numpy as np
import pytest

from patrickstar_b200.chunk_list import ChunkLayout


def test_no_split_packing_like_the_reference():
    # unitest/test_chunk_tensor_index.py:82-170: tensors never straddle; a module's list is atomic
    lay = ChunkLayout(chunk_size=20, pack="no_split")
    a = lay.append_tensor_list([("m1.w", 10, 0), ("m1.b", 2, 0)])
    assert [(t.chunk_id, t.start_offset) for t in a] == [(0, 0), (0, 10)]
    b = lay.append_tensor_list([("m2.w", 7, 0), ("m2.b", 2, 0)])   # 9 > 8 free -> new chunk as a whole
    assert [(t.chunk_id, t.start_offset) for t in b] == [(1, 0), (1, 7)]
    c = lay.append_tensor("m3.w", 11)
    assert (c.chunk_id, c.start_offset) == (1, 9)
    with pytest.raises(RuntimeError, match="larger than the chunk size"):
        lay.append_tensor("huge", 21)
    with pytest.raises(ValueError, match="duplicate"):
        lay.append_tensor("m3.w", 1)
    lay.freeze()
    assert lay.n_data_chunks == 2 and lay.chunk_numel(0) == 12 and lay.chunk_numel(1) == 20


def test_flat_packing_splits_tensors_at_chunk_boundaries():
    lay = ChunkLayout(chunk_size=100, pack="flat")
    lay.append_tensor_list([("a", 30, 0), ("b", 90, 1), ("c", 50, 0), ("big", 260, 1), ("d", 10, 0)])
    lay.freeze()
    assert lay.total_numel() == 440 and lay.n_data_chunks == 5
    assert [lay.chunk_numel(c) for c in range(5)] == [100, 100, 100, 100, 40]
    segs = {c: [(p.start, p.end, p.group) for p in lay.segments_of_chunk(c)] for c in range(5)}
    assert segs[0] == [(0, 30, 0), (30, 100, 1)]
    assert segs[1] == [(0, 20, 1), (20, 70, 0), (70, 100, 1)]
    assert segs[2] == [(0, 100, 1)] and segs[3] == [(0, 100, 1)]
    assert segs[4] == [(0, 30, 1), (30, 40, 0)]
    # every element is covered exactly once
    cover = np.zeros(500, dtype=int)
    for c in range(5):
        for s, e, _ in segs[c]:
            cover[c * 100 + s:c * 100 + e] += 1
    assert (cover[:440] == 1).all() and (cover[440:] == 0).all()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ownership_and_padding(world):
    # chunk_list.py:383-387: k-th chunk -> rank k % world, group k // world;
    # preprocess.py:335-339: padded with dummy chunks to a multiple of world
    lay = ChunkLayout(chunk_size=10, world_size=world, pack="flat")
    lay.append_tensor("t", 10 * 11)
    lay.freeze()
    assert lay.n_data_chunks == 11
    assert lay.n_chunks % world == 0 and lay.n_chunks - 11 < world
    owned = [lay.local_chunk_ids(r) for r in range(world)]
    assert sorted(sum(owned, [])) == list(range(lay.n_chunks))
    assert len(set(len(o) for o in owned)) == 1 == (len(owned[0]) == lay.n_groups_comm)
    for r in range(world):
        for k, c in enumerate(owned[r]):
            ci = lay.comm_info(c)
            assert (ci.group_id, ci.offset) == (k, r)
    for c in range(11, lay.n_chunks):
        assert lay.is_dummy(c) and lay.chunk_numel(c) == 0 and lay.segments_of_chunk(c) == []


def test_tables_first_call_slot_and_plan():
    lay = ChunkLayout(chunk_size=100, world_size=2, pack="flat")
    lay.append_tensor_list([("a", 30, 0), ("b", 90, 1), ("c", 50, 0), ("d", 10, 1)])
    lay.freeze()
    local, numels, ranges, segs = lay.build_tables(0)
    assert local == [0] and numels == [100] and ranges == [(0, 2)]
    assert segs.tolist() == [[0, 30, 0, 0], [30, 100, 2, 0]]      # first piece -> slot 0, group 1 -> slot 2
    assert lay.plan_groups(0) == (0, 1, 2)
    local, numels, ranges, segs = lay.build_tables(1)
    assert local == [1] and numels == [80]
    assert segs.tolist() == [[0, 20, 0, 0], [20, 70, 1, 0], [70, 80, 2, 0]]
    assert lay.plan_groups(1) == (1, 1, 3)
    # one single piece: it is the first call, slot 0
    one = ChunkLayout(chunk_size=64, pack="flat")
    one.append_tensor("w", 64)
    one.freeze()
    assert one.build_tables(0)[3].tolist() == [[0, 64, 0, 0]] and one.plan_groups(0) == (0, 0, 1)
    # first piece merged with a same-group neighbour is split off again
    two = ChunkLayout(chunk_size=64, pack="flat")
    two.append_tensor_list([("w1", 10, 0), ("w2", 20, 0), ("b", 4, 1)])
    two.freeze()
    assert two.build_tables(0)[3].tolist() == [[0, 10, 0, 0], [10, 30, 1, 0], [30, 34, 2, 0]]


def test_gpt2_xl_layout_counts():
    """GPT-2 1.5B (48 layers, hidden 1600, vocab 50257, 1024 positions) packed flat
    into 64 Mi-element chunks: 1,557,611,200 parameters -> 24 chunks."""
    from patrickstar_b200.model_layouts import gpt_tensor_specs
    specs = gpt_tensor_specs(n_layer=48, hidden=1600, vocab=50257, n_pos=1024)
    lay = ChunkLayout(chunk_size=64 * 1024 * 1024, pack="flat")
    lay.append_tensor_list([(n, int(np.prod(s)), g) for n, s, g in specs])
    lay.freeze()
    assert lay.total_numel() == 1557611200
    assert lay.n_data_chunks == 24
    groups = {g for _, _, g in specs}
    assert groups == {0, 1}
    n_decay = sum(int(np.prod(s)) for _, s, g in specs if g == 0)
    assert n_decay == 48 * (1600 * 4800 + 1600 * 1600 + 1600 * 6400 + 6400 * 1600) + 50257 * 1600 + 1024 * 1600


def test_random_layouts_cover_every_element_once():
    """Property test over random tensor lists, chunk sizes, packings and world
    sizes: segments tile exactly the elements of the tensors (no overlap, no
    hole inside a tensor), every chunk has one owner, the per-rank tables list
    exactly the rank's segments, and slot 0 marks exactly the first piece."""
    rng = np.random.RandomState(1234)
    for trial in range(60):
        cs = int(rng.choice([64, 100, 257, 1024]))
        world = int(rng.choice([1, 2, 3, 4, 8]))
        pack = str(rng.choice(["flat", "no_split"]))
        lay = ChunkLayout(cs, world, pack)
        n_t = int(rng.randint(1, 25))
        total = 0
        for i in range(n_t):
            hi = cs if pack == "no_split" else 3 * cs
            numel = int(rng.randint(1, hi + 1))
            lay.append_tensor("t%d" % i, numel, int(rng.randint(0, 3)))
            total += numel
        lay.freeze()
        assert lay.total_numel() == total
        assert lay.n_chunks % world == 0 and lay.n_chunks >= lay.n_data_chunks
        cover = np.zeros(lay.n_chunks * cs, dtype=np.int32)
        group_at = np.full(lay.n_chunks * cs, -1, dtype=np.int32)
        for t in lay.tensors:
            s = t.flat_start(cs)
            if pack == "no_split":
                assert t.start_offset + t.numel <= cs          # never straddles
            group_at[s:s + t.numel] = t.group
        seen_chunks = []
        for r in range(world):
            local, numels, ranges, segs = lay.build_tables(r)
            seen_chunks += local
            first_slots = 0
            for k, c in enumerate(local):
                assert numels[k] == lay.chunk_numel(c) <= cs
                prev = 0
                for row in segs[ranges[k][0]:ranges[k][1]]:
                    a, b, slot = int(row[0]), int(row[1]), int(row[2])
                    assert prev <= a < b <= numels[k]
                    prev = b
                    cover[c * cs + a:c * cs + b] += 1
                    g = group_at[c * cs + a:c * cs + b]
                    assert (g == g[0]).all() and g[0] >= 0
                    if slot == 0:
                        first_slots += 1
                    else:
                        assert slot == 1 + g[0]
            calls = lay.calls_of_rank(r)
            assert first_slots == (1 if calls else 0)
            assert lay.plan_groups(r)[2] == len(calls)
        assert sorted(seen_chunks) == list(range(lay.n_chunks))
        assert (cover[group_at >= 0] == 1).all() and (cover[group_at < 0] == 0).all()


@pytest.mark.parametrize("name,chunks,per_rank_at_8", [("gpt_12b", 192, 24), ("gpt_40b", 583, 73)])
def test_large_gpt_layouts_and_ownership(name, chunks, per_rank_at_8):
    """The 12B (40 layers, hidden 5120) and 40B (48 layers, hidden 8192) GPT
    configurations cut into 64 Mi-element chunks: single tensors exceed a chunk
    (flat packing is required), chunk counts and the per-rank share on 8 ranks."""
    from patrickstar_b200.model_layouts import model_specs
    specs = model_specs(name)
    cs = 64 * 1024 * 1024
    assert max(int(np.prod(s)) for _, s, _ in specs) > cs
    with pytest.raises(RuntimeError, match="larger than the chunk size"):
        ChunkLayout(cs, 8, "no_split").append_tensor_list([(n, int(np.prod(s)), g) for n, s, g in specs])
    lay = ChunkLayout(cs, 8, "flat")
    lay.append_tensor_list([(n, int(np.prod(s)), g) for n, s, g in specs])
    lay.freeze()
    assert lay.n_data_chunks == chunks
    assert lay.n_chunks == per_rank_at_8 * 8 and len(lay.local_chunk_ids(3)) == per_rank_at_8
    # 12 B of fp32 state per parameter on the owner: the 40B model needs the offload tier under a 40 GB budget
    state_gib = per_rank_at_8 * 12 * cs / 2 ** 30
    assert (state_gib > 40) == (name == "gpt_40b")


def test_handoff_counts_per_communication_group():
    """Elements a tensor adds to each communication group's hand-off count (the trigger of the
    group's reduce-scatter): tensors straddling chunks and groups are split at the boundaries,
    and the per-group totals equal the elements in use in the group's chunks."""
    cs, w = 100, 2
    lay = ChunkLayout(cs, w, "flat")
    lay.append_tensor_list([("a", 150, 0), ("b", 120, 1), ("c", 260, 0), ("d", 30, 1)])
    lay.freeze()
    assert lay.n_data_chunks == 6 and lay.n_groups_comm == 3
    total = {}
    per_tensor = {t.name: lay.add_to_comm_groups(t, {}) for t in lay.tensors}
    for t in lay.tensors:
        lay.add_to_comm_groups(t, total)
    assert per_tensor["a"] == {0: 150}
    assert per_tensor["b"] == {0: 50, 1: 70}
    assert per_tensor["c"] == {1: 130, 2: 130}
    assert per_tensor["d"] == {2: 30}
    used = {g: sum(lay.chunk_numel(c) for c in range(g * w, (g + 1) * w)) for g in range(3)}
    assert total == used == {0: 200, 1: 200, 2: 160}
