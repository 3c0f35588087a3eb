"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from scriptling_llm_lib_b200.cache import PAGE, CacheFull, CacheNeed, FreeList, SequenceCache, StateNeed, pages_for


def test_free_list_never_hands_out_twice_and_refuses_double_free():
    fl = FreeList(5, "thing")
    got = [fl.alloc() for _ in range(5)]
    assert sorted(got) == [0, 1, 2, 3, 4] and fl.n_free == 0 and fl.n_held == 5
    with pytest.raises(CacheFull):
        fl.alloc()
    fl.free(3)
    with pytest.raises(ValueError):
        fl.free(3)
    with pytest.raises(ValueError):
        fl.free(7)
    assert fl.alloc() == 3 and fl.n_free == 0


def test_free_list_random_walk_conserves_ids():
    rng = random.Random(0)
    fl = FreeList(17, "thing")
    held = set()
    for _ in range(2000):
        if held and (rng.random() < 0.5 or fl.n_free == 0):
            i = rng.choice(sorted(held))
            fl.free(i)
            held.remove(i)
        else:
            i = fl.alloc()
            assert i not in held
            held.add(i)
        assert fl.n_held == len(held) and fl.n_free + fl.n_held == 17


def make_cache(n_slots=4, n_pages=8, window=None):
    needs = {0: CacheNeed("full", 2, 16), 1: CacheNeed("full", 2, 16), 2: CacheNeed("window", 1, 32, window or 70)}
    return SequenceCache(needs, {0: None, 1: StateNeed((3,), torch.float32), 2: None}, n_slots, n_pages, torch.float32, "cpu")


def test_groups_have_storage_of_their_own():
    c = make_cache()
    assert len(c.groups) == 2
    full, win = c.groups[c.group_of_unit[0]], c.groups[c.group_of_unit[2]]
    assert c.group_of_unit[0] == c.group_of_unit[1] != c.group_of_unit[2]
    assert full.k.shape == (2, 8 + 1, 2, PAGE, 16) and win.k.shape == (1, 8 + 1, 1, PAGE, 32)   # + the spare page
    k0, _ = full.unit_storage(0)
    k1, _ = full.unit_storage(1)
    assert k0.data_ptr() != k1.data_ptr() and k0.shape == (9, 2, PAGE, 16)
    assert c.state[1].shape == (4 + 1, 3) and 0 not in c.state


def test_pages_follow_each_sequences_own_length():
    c = make_cache()
    a, b = c.open(), c.open()
    c.reserve([(a, 5), (b, 130)])
    c.advance([(a, 5), (b, 130)])
    assert c.length[a] == 5 and c.length[b] == 130
    full = c.groups[c.group_of_unit[0]]
    assert len(full.pages[a]) == 1 and len(full.pages[b]) == 3
    assert len(set(full.pages[a]) | set(full.pages[b])) == 4            # no page held twice
    bt = c.block_table(c.group_of_unit[0], [a, b])
    assert bt.shape == (2, 3) and bt[0, 1] == -1 and list(bt[1]) == full.pages[b]
    c.reserve([(a, 59)])                                               # 5 + 59 = 64 tokens: still one page
    assert len(full.pages[a]) == 1
    c.advance([(a, 59)])
    c.reserve([(a, 1)])
    assert len(full.pages[a]) == 2


def test_reserve_is_all_or_nothing():
    c = make_cache(n_pages=4)
    a, b = c.open(), c.open()
    c.reserve([(a, 100)])
    c.advance([(a, 100)])
    before = [g.pool.n_free for g in c.groups]
    with pytest.raises(CacheFull):
        c.reserve([(a, 60), (b, 100)])                                 # 1 + 2 more pages, 2 free
    assert [g.pool.n_free for g in c.groups] == before and c.length[a] == 100 and c.length[b] == 0
    c.reserve([(b, 100)])


def test_slots_and_pages_come_back_and_are_used_again():
    c = make_cache(n_slots=2, n_pages=6)
    a, b = c.open(), c.open()
    with pytest.raises(CacheFull):
        c.open()
    c.reserve([(a, 128), (b, 200)])
    c.advance([(a, 128), (b, 200)])
    c.state[1][a] = 5.0
    c.close(a)
    with pytest.raises(ValueError):
        c.close(a)                                                     # not freed twice
    assert all(g.pool.n_held == 4 for g in c.groups if g.need.kind == "full")
    a2 = c.open()
    assert a2 == a and c.length[a2] == 0 and float(c.state[1][a2].abs().sum()) == 0.0   # state starts at zero
    c.reserve([(a2, 128)])
    c.close(a2)
    c.close(b)
    for g in c.groups:
        assert g.pool.n_free == g.pool.n and not g.pages                # nothing lost
    assert c.slots.n_free == 2


def test_window_group_gives_back_pages_no_later_query_can_see():
    c = make_cache(n_pages=8, window=70)
    a = c.open()
    win = c.groups[c.group_of_unit[2]]
    full = c.groups[c.group_of_unit[0]]
    c.reserve([(a, 200)])
    assert win.pool.n_held == pages_for(200) == 4                      # the prompt's own step needs all its keys
    c.advance([(a, 200)])
    # next query is at position 200 and sees keys 131..200: pages 0 and 1 (keys 0..127) are unseen
    assert win.pages[a][:2] == [-1, -1] and win.pages[a][2] >= 0 and win.pool.n_held == 2
    assert full.pool.n_held == 4
    for _ in range(120):
        c.reserve([(a, 1)])
        c.advance([(a, 1)])
    assert c.length[a] == 320 and win.pool.n_held == 2                 # keys 251..320 live in pages 3 and 4
    assert [p >= 0 for p in win.pages[a]] == [False, False, False, True, True]
    bt = c.block_table(c.group_of_unit[2], [a])
    assert list(bt[0][:3]) == [-1, -1, -1]
    c.close(a)
    assert win.pool.n_free == 8 and full.pool.n_free == 8


def test_state_record_is_zeroed_at_open_and_seeded_per_sequence():
    """Beside keys and values every slot has a record of eight words (tokens held, tokens generated,
    last token, flags, sampling key x2, draw counter x2): zero when the slot is opened, whoever
    held it before; `seed` sets the key of freshly opened sequences and nothing else."""
    from scriptling_llm_lib_b200.cache.store import SEQ_COUNTER, SEQ_KEY, SEQ_STATE_WORDS
    c = make_cache()
    assert c.seq_state.shape == (4 + 1, SEQ_STATE_WORDS) and c.seq_state.dtype == torch.int32
    a, b = c.open(), c.open()
    c.seed([a, b], [7, (5 << 32) | 0xFFFFFFFE])
    rec = c.seq_state.numpy().astype("int64") & 0xFFFFFFFF
    assert list(rec[a]) == [0, 0, 0, 0, 7, 0, 0, 0]
    assert list(rec[b]) == [0, 0, 0, 0, 0xFFFFFFFE, 5, 0, 0]
    c.seq_state[a, SEQ_COUNTER] = 12                                      # as the sampling kernel would leave it
    c.close(a)
    again = c.open()
    assert again == a and int(c.seq_state[a].abs().sum()) == 0 and int(c.seq_state[b, SEQ_KEY + 1]) == 5


def test_cache_kinds_are_a_registry():
    from scriptling_llm_lib_b200.cache import register_cache_kind
    with pytest.raises(ValueError, match="known"):
        CacheNeed("no_such_kind", 1, 16)
    with pytest.raises(ValueError, match="already registered"):
        register_cache_kind("full", lambda need, length: 0)
    # a kind that keeps only the last two pages' worth of positions, whatever the need's window says
    register_cache_kind("last_128", lambda need, length: length - 128, replace=True)
    c = SequenceCache({0: CacheNeed("last_128", 1, 16)}, {0: None}, 2, 8, torch.float32, "cpu")
    s = c.open()
    c.reserve([(s, 300)])
    c.advance([(s, 300)])
    assert c.groups[0].pages[s][:2] == [-1, -1] and all(p >= 0 for p in c.groups[0].pages[s][2:])   # positions < 172: pages 0, 1 gone
    c.close(s)
    assert c.groups[0].pool.n_held == 0
