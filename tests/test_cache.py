"""The cache's bookkeeping (no GPU): no slot or page lost, held twice or freed twice."""
import pytest
import torch

from questwend_b200.cache import CacheError, CacheFull, CacheManager, FreeList, pages_for
from questwend_b200.kernels.ops import PAGE_SIZE
from questwend_b200.parts.base import KVSpec, StateSpec


def test_free_list():
    fl = FreeList(4, "slot")
    a = fl.take(3)
    assert a == [0, 1, 2] and fl.n_free == 1
    with pytest.raises(CacheFull):
        fl.take(2)
    assert fl.n_free == 1                      # a refused take changes nothing
    fl.give_back([1])
    assert fl.take(1) == [1]                   # the lowest free id comes first: ids are used again
    with pytest.raises(CacheError, match="not held"):
        fl.give_back([3])
    fl.give_back([0])
    with pytest.raises(CacheError, match="not held"):
        fl.give_back([0])                      # freed twice
    with pytest.raises(CacheError, match="does not exist"):
        fl.give_back([9])
    fl.give_back([1, 2])
    assert sorted(fl.take(4)) == [0, 1, 2, 3]  # nothing lost


def _manager(units=None, **kw):
    units = units or [(KVSpec(2, 16), None, None), (KVSpec(2, 16), None, None)]
    args = dict(max_tokens=8 * PAGE_SIZE, max_slots=4, max_seq_len=4 * PAGE_SIZE, dtype=torch.float32, device="cpu")
    args.update(kw)
    return CacheManager(units, **args)


def test_slots_and_pages_are_conserved():
    m = _manager()
    assert m.n_groups() == 1 and m.free_pages() == [8]
    slots = m.open(3)
    assert slots == [0, 1, 2] and [m.length(s) for s in slots] == [0, 0, 0]
    m.reserve({0: 1, 1: PAGE_SIZE, 2: PAGE_SIZE + 1})
    assert m.free_pages() == [8 - 4]
    m.reserve({0: 1, 1: PAGE_SIZE, 2: PAGE_SIZE + 1})            # asking again takes nothing more
    assert m.free_pages() == [4]
    pages = [p for s in slots for p in m._groups[0].pages[s]]
    assert len(set(pages)) == len(pages) == 4                    # no page held twice
    m.advance(2, PAGE_SIZE + 1)
    m.close([1])
    assert m.free_pages() == [5]
    with pytest.raises(CacheError, match="not open"):
        m.close([1])                                             # closed twice
    with pytest.raises(CacheError, match="not open"):
        m.length(1)
    with pytest.raises(CacheError, match="twice"):
        m.close([0, 0])
    assert m.open(1) == [1] and m.length(1) == 0                 # the slot comes back, empty
    m.close([0, 1, 2])
    assert m.free_pages() == [8] and m.slots.n_free == 4         # nothing lost


def test_full_cache_changes_nothing():
    m = _manager(max_tokens=7 * PAGE_SIZE)
    a, b = m.open(2)
    m.reserve({a: 3 * PAGE_SIZE})
    with pytest.raises(CacheFull, match="pages"):
        m.reserve({a: 4 * PAGE_SIZE, b: 4 * PAGE_SIZE})          # 1 + 4 more pages, 4 are left
    assert m.free_pages() == [4] and len(m._groups[0].pages[b]) == 0 and len(m._groups[0].pages[a]) == 3
    with pytest.raises(CacheFull, match="longest"):
        m.reserve({b: 4 * PAGE_SIZE + 1})                        # beyond max_seq_len
    m.open(2)
    with pytest.raises(CacheFull, match="slot"):
        m.open(1)


def test_page_table_and_truncate():
    m = _manager()
    a, b = m.open(2)
    m.reserve({a: 2 * PAGE_SIZE + 5, b: 3})
    m.advance(a, 2 * PAGE_SIZE + 5)
    table = m.page_table_host(0, [b, a])
    assert table.shape == (2, 4) and table.dtype.name == "int32"
    assert list(table[1, :3]) == m._groups[0].pages[a] and list(table[0, :1]) == m._groups[0].pages[b]
    m.truncate(a, PAGE_SIZE)                                     # the reference's rewind: core/runtime.cpp:2804-2811
    assert m.length(a) == PAGE_SIZE and len(m._groups[0].pages[a]) == 1 and m.free_pages() == [8 - 2]
    with pytest.raises(CacheError):
        m.truncate(a, PAGE_SIZE + 1)


def test_groups_have_storage_of_their_own():
    full, windowed = KVSpec(2, 16), KVSpec(2, 16, window=32)
    other = KVSpec(1, 32)
    m = _manager([(full, None, None), (windowed, None, None), (full, None, None), (other, None, None),
                  (None, StateSpec((3, 2)), None), (None, None, 0)])
    assert m.n_groups() == 3
    u0, u1, u2, u3, u4, u5 = (m.unit_cache(i) for i in range(6))
    assert u0.group_id == u2.group_id != u1.group_id and u3.group_id not in (u0.group_id, u1.group_id)
    assert u0.k_pool.shape == (8, 2, PAGE_SIZE, 16) and u3.k_pool.shape == (8, 1, PAGE_SIZE, 32)
    assert u0.k_pool.data_ptr() != u2.k_pool.data_ptr()
    assert u4.k_pool is None and u4.state.shape == (4, 3, 2)
    # a run that reads another run's cache sees that run's tensors and may not write
    assert u5.k_pool.data_ptr() == u0.k_pool.data_ptr() and not u5.writable and u0.writable
    (s,) = m.open(1)
    m.reserve({s: 70})
    assert m.free_pages() == [6, 6, 6]                           # every group gives the sequence its pages


def test_state_is_zeroed_when_a_slot_is_handed_out_again():
    m = _manager([(None, StateSpec((5,)), None)])
    (s,) = m.open(1)
    m.unit_cache(0).state[s] = 7.0
    m.close([s])
    (t,) = m.open(1)
    assert t == s and float(m.unit_cache(0).state[t].abs().sum()) == 0.0
    with pytest.raises(CacheError, match="fixed-size state"):
        m.truncate(t, 0)


def test_sizes():
    assert pages_for(0) == 0 and pages_for(1) == 1 and pages_for(PAGE_SIZE) == 1 and pages_for(PAGE_SIZE + 1) == 2
    with pytest.raises(CacheError):
        _manager(max_tokens=0)


def test_random_histories_lose_and_duplicate_nothing():
    """Random sequences of open / reserve+advance / truncate / close, two groups (one with a window): after every
    operation no page is held twice, held and free pages add up to the pool, and lengths fit the pages held."""
    from hypothesis import given, settings, strategies as st

    ops_strategy = st.lists(st.tuples(st.sampled_from(["open", "grow", "cut", "close"]), st.integers(0, 5),
                                      st.integers(1, 3 * PAGE_SIZE)), min_size=1, max_size=60)

    @settings(max_examples=60, deadline=None)
    @given(ops_strategy, st.booleans())
    def run(history, with_state):
        units = [(KVSpec(2, 16), None, None), (KVSpec(1, 32, window=40), None, None)]
        if with_state:                                 # a sequence with fixed-size state cannot be cut back: "cut" is refused
            units.append((None, StateSpec((3,)), None))
        m = _manager(units=units, max_tokens=10 * PAGE_SIZE, max_slots=5)
        held = set()
        for what, which, amount in history:
            try:
                if what == "open":
                    held.update(m.open(1))
                elif not held:
                    continue
                else:
                    slot = sorted(held)[which % len(held)]
                    if what == "grow":
                        want = m.length(slot) + amount
                        m.reserve({slot: want})
                        m.advance(slot, amount)
                    elif what == "cut":
                        m.truncate(slot, min(m.length(slot), amount))
                    else:
                        m.close([slot])
                        held.discard(slot)
            except CacheError:
                pass                                   # a refusal (full, too long, fixed-size state): nothing may change
            assert m.slots.n_free == 5 - len(held)
            for g in m._groups:
                pages = [p for s in held for p in g.pages[s]]
                assert len(pages) == len(set(pages))
                assert len(pages) + g.pool.n_free == g.pool.n
                for s in held:
                    assert len(g.pages[s]) * PAGE_SIZE >= m.length(s)
        m.close(sorted(held))
        assert m.slots.n_free == 5 and all(g.pool.n_free == g.pool.n for g in m._groups)

    run()
