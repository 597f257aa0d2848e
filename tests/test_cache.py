"""The cache's host side: no slot or block lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

import xeno_rt_b200  # noqa: F401
from xeno_rt_b200.cache import BlockAllocator, Cache, KVNeed, SlotAllocator, StateNeed
from xeno_rt_b200.core import CacheError, DType


def test_block_allocator_books_balance():
    a = BlockAllocator(8)
    first = a.take(3)
    assert first == [0, 1, 2] and a.free == 5 and a.held == 3
    second = a.take(5)
    assert sorted(first + second) == list(range(8))
    with pytest.raises(CacheError, match="full"):
        a.take(1)
    a.give_back([1])
    with pytest.raises(CacheError, match="twice"):
        a.give_back([1])
    with pytest.raises(CacheError, match="does not exist"):
        a.give_back([8])
    assert a.take(1) == [1]  # what was given back is used again first
    a.check()


def test_slot_allocator():
    s = SlotAllocator(2)
    a, b = s.open(), s.open()
    assert {a, b} == {0, 1}
    with pytest.raises(CacheError, match="no free slot"):
        s.open()
    s.close(a)
    with pytest.raises(CacheError, match="not open"):
        s.close(a)
    assert s.open() == a
    s.check()


def _cache(max_tokens=64 * 6, max_positions=256, needs=None, max_slots=None):
    needs = needs if needs is not None else [KVNeed(2, 16), KVNeed(2, 16)]
    return Cache(needs, max_tokens, max_positions, DType.F32, "cpu", max_slots)


def test_reserve_advance_close():
    c = _cache()
    assert c.n_blocks == 6 and c.blocks_per_seq == 4 and len(c.kv_groups) == 1
    s = c.open_slot()
    assert c.reserve(s, 70) == 0  # two blocks
    assert c.blocks_free() == 4 and c.length(s) == 0
    c.advance(s, 70)
    assert c.reserve(s, 1) == 70 and c.blocks_free() == 4  # position 70 is inside the second block
    c.advance(s, 1)
    c.advance(s, 57)  # up to 128, still the two blocks
    with pytest.raises(CacheError, match="passes what was reserved"):
        c.advance(s, 1)
    assert c.reserve(s, 1) == 128 and c.blocks_free() == 3
    c.check()
    c.close_slot(s)
    assert c.blocks_free() == 6
    with pytest.raises(CacheError, match="not open"):
        c.close_slot(s)
    with pytest.raises(CacheError, match="not open"):
        c.length(s)
    c.check()


def test_limits():
    c = _cache(max_tokens=64 * 3, max_positions=100)
    a, b = c.open_slot(), c.open_slot()
    with pytest.raises(CacheError, match="positions"):
        c.reserve(a, 101)
    c.reserve(a, 100)
    c.reserve(b, 64)
    with pytest.raises(CacheError, match="full"):
        c.reserve(b, 65)
    with pytest.raises(CacheError, match="at least one token"):
        c.reserve(b, 0)
    c.check()


def test_blocks_are_used_again_and_tables_follow():
    c = _cache()
    a = c.open_slot()
    c.reserve(a, 128)
    c.advance(a, 128)
    blocks_a = list(c.kv_groups[0].table_host[a, :2])
    c.flush_tables()
    assert c.kv_groups[0].table[a, :2].tolist() == blocks_a
    c.close_slot(a)
    b = c.open_slot()
    assert b == a
    c.reserve(b, 10)
    assert c.kv_groups[0].table_host[b, 0] == min(blocks_a)
    c.flush_tables()
    assert c.kv_groups[0].table[b].tolist()[1:] == [-1] * (c.blocks_per_seq - 1)
    c.check()


def test_groups_have_storage_of_their_own_and_state_is_zeroed():
    needs = [KVNeed(2, 16), KVNeed(2, 16, window=32), None, StateNeed((3, 5)), KVNeed(2, 16)]
    c = _cache(needs=needs)
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    full, windowed = c.store(0), c.store(1)
    assert full.k.data_ptr() != windowed.k.data_ptr() and full.block_table is not windowed.block_table
    assert c.store(4).k.shape == full.k.shape and c.store(4).k.data_ptr() != full.k.data_ptr()
    assert c.store(2) is None
    state = c.store(3).state
    assert tuple(state.shape) == (c.max_slots, 3, 5)
    extra = c.register_sequence_state("t.x", (2,), state.dtype)
    s = c.open_slot()
    state[s] += 1
    extra[s] += 1
    c.close_slot(s)
    assert c.open_slot() == s and float(state[s].abs().sum()) == 0.0 and float(extra[s].abs().sum()) == 0.0


def test_a_windowed_group_gives_blocks_back_as_the_sequence_moves_on():
    """Window of 70 keys: a token at position p sees p-69 .. p.  Block b (positions 64 b .. 64 b + 63) may
    go once the sequence's length L has 64 b + 63 <= L - 70; the group that keeps every key holds on."""
    c = _cache(max_tokens=64 * 8, max_positions=512, needs=[KVNeed(2, 16), KVNeed(2, 16, window=70)], max_slots=3)
    full, windowed = c.kv_groups
    assert full.need.window is None and windowed.need.window == 70
    s = c.open_slot()
    c.reserve(s, 133)
    assert windowed.allocator.held == 3  # the prompt's own step needs every block: its first tokens see the first keys
    c.advance(s, 133)  # the next token, at 133, sees 64 .. 133: block 0 (0 .. 63) is done
    assert windowed.allocator.held == 2 and full.allocator.held == 3
    assert windowed.table_host[s, 0] == -1 and windowed.table_host[s, 1] >= 0
    c.check()
    c.reserve(s, 1)
    c.advance(s, 1)  # length 134: the next token sees 65 .. 134; block 1 still holds visible keys
    assert windowed.allocator.held == 2
    for _ in range(62):
        c.reserve(s, 1)
        c.advance(s, 1)
    assert c.length(s) == 196 and windowed.allocator.held == 3  # block 3 was taken for 192 ..; block 1 still needed
    released = int(windowed.table_host[s, 1])
    c.reserve(s, 1)
    c.advance(s, 1)  # length 197: the next token sees 128 .. 197, so block 1 (64 .. 127) is done
    assert windowed.allocator.held == 2 and windowed.table_host[s, 1] == -1
    c.check()
    # what was given back is used by another sequence while the first one lives on
    t = c.open_slot()
    c.reserve(t, 10)
    assert int(windowed.table_host[t, 0]) == released and int(full.table_host[t, 0]) == 4  # used again; the other group has no old block
    c.advance(t, 10)
    c.check()
    c.close_slot(s)
    c.close_slot(t)
    assert windowed.allocator.free == 8 and full.allocator.free == 8
    c.check()
    with pytest.raises(CacheError, match="not open"):
        c.close_slot(s)


@pytest.mark.parametrize("window", [None, 100])
def test_random_traffic_never_loses_or_doubles_a_block(window):
    rng = random.Random(3)
    c = _cache(max_tokens=64 * 20, max_positions=640, max_slots=6, needs=[KVNeed(2, 16), KVNeed(2, 16, window=window)])
    live = {}
    for _ in range(400):
        op = rng.random()
        if op < 0.3 and c.slots.free:
            live[c.open_slot()] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = rng.randint(1, 90)
            try:
                c.reserve(s, n)
                c.advance(s, n)
                live[s] += n
            except CacheError:
                pass
        elif live:
            s = rng.choice(list(live))
            c.close_slot(s)
            del live[s]
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
    for s in list(live):
        c.close_slot(s)
    assert all(g.allocator.free == 20 for g in c.kv_groups) and c.slots.free == 6


def test_a_place_may_ask_for_several_storages_by_list_and_by_part_name():
    """A mixer that wants keys AND a fixed-size state asks with a list; a layer with two parts that
    keep something asks with a dict by part name; ``store`` answers in the same shape, and equal
    needs still share one group of storage."""
    from xeno_rt_b200.cache import KVStore, StateStore
    needs = [[KVNeed(2, 16), StateNeed((4,))],
             {"mixer": KVNeed(2, 16), "memory": [StateNeed((4,)), StateNeed((2, 2), "int32")]},
             None, {}]
    c = _cache(needs=needs)
    assert len(c.kv_groups) == 1 and c.kv_groups[0].k.shape[0] == 2
    assert len(c.state_groups) == 2
    first = c.store(0)
    assert isinstance(first, list) and isinstance(first[0], KVStore) and isinstance(first[1], StateStore)
    second = c.store(1)
    assert set(second) == {"mixer", "memory"} and isinstance(second["mixer"], KVStore)
    assert [tuple(s.state.shape[1:]) for s in second["memory"]] == [(4,), (2, 2)]
    assert second["mixer"].k.data_ptr() != first[0].k.data_ptr()
    assert second["memory"][0].state.data_ptr() != first[1].state.data_ptr()
    assert c.store(2) is None and c.store(3) == {}
    with pytest.raises(CacheError, match="unknown cache need"):
        _cache(needs=[{"mixer": 3}])


def test_a_step_that_cannot_be_served_takes_nothing():
    """reserve_all serves every sequence of a step or none: when a later sequence finds the pool
    empty, the earlier ones give back what they just took."""
    c = _cache(max_tokens=64 * 4, needs=[KVNeed(2, 16), KVNeed(2, 16, window=70)])
    a, b, d = c.open_slot(), c.open_slot(), c.open_slot()
    assert c.reserve_all([a], [70]) == [0]
    c.advance(a, 70)                       # a holds 2 of 4 blocks
    free = c.blocks_free()
    with pytest.raises(CacheError, match="full"):
        c.reserve_all([b, a, d], [64, 1, 130])  # b takes one, a none, d needs three: one is left
    assert c.blocks_free() == free
    c.check()
    assert c.length(b) == 0 and c.length(a) == 70
    assert c.reserve_all([b, a], [64, 1]) == [0, 70]
    c.advance(b, 64)
    c.advance(a, 1)
    c.check()
    with pytest.raises(CacheError):       # a limit of the model's positions, after an entry that was served
        c.reserve_all([d, a], [10, 10_000])
    assert c.blocks_free() == 1
    c.check()
    for s in (a, b, d):
        c.close_slot(s)
    c.check()
    assert c.blocks_free() == 4


def test_block_tables_reach_the_device_tensor_row_by_row():
    """flush_tables brings the changed rows of the host's block tables into the device tensor (here a
    CPU tensor) and nothing else; sequences of unequal lengths change some row at nearly every step."""
    c = _cache(max_tokens=64 * 8, needs=[KVNeed(2, 16)])
    a, b = c.open_slot(), c.open_slot()
    c.reserve_all([a, b], [70, 5])
    c.flush_tables()
    table = c.store(0).block_table
    assert (table[a, :2] >= 0).all() and table[a, 2] == -1 and table[b, 0] >= 0 and table[b, 1] == -1
    c.advance(a, 70)
    c.advance(b, 5)
    before = table.clone()
    c.reserve_all([a, b], [1, 60])   # b crosses into its second block, a stays in its second
    c.flush_tables()
    assert (table[a] == before[a]).all() and table[b, 1] >= 0 and (table[b, 0] == before[b, 0])
    c.check()


def test_pinned_buffers_are_used_in_turn_and_grow():
    """The ring of host buffers behind every small copy to the device: a buffer comes back only after
    the others, and a larger request gets a larger buffer (on the CPU nothing is pinned or waited for)."""
    from xeno_rt_b200.core.staging import PinnedRing
    ring = PinnedRing("cpu", count=3)
    turns = []
    for n in (10, 20, 5000, 7):
        turn, buf = ring.take(n)
        assert buf.numel() == n and buf.dtype == torch.int32
        buf.fill_(n)
        ring.copied(turn)
        turns.append(turn)
    assert turns == [0, 1, 2, 0]
    assert ring.buffers[2].numel() >= 5000 and ring.buffers[0].numel() >= 1024
