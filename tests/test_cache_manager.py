"""Cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; window groups give pages back; state slots."""
import random

import pytest
import torch

from photon_infer_b200.cache import NO_PAGE, CacheManager, PagePool, StateSlotPool
from photon_infer_b200.errors import ErrorCode, PhotonError
from photon_infer_b200.parts.base import PagedCacheSpec, StateSpec

FULL = PagedCacheSpec(2, 16, None)
WIN = PagedCacheSpec(2, 16, 24)


def _manager(num_pages=16, page_size=8, max_sequences=4, window=True, state=False):
    needs = [(WIN if window else FULL, StateSpec((3,)) if state else None), (FULL, None),
             (WIN if window else FULL, None), (FULL, None)]
    return CacheManager(needs, [None] * 4, page_size, num_pages, max_sequences, torch.float32, None)


def test_page_pool_order_and_errors():
    pool = PagePool(4)
    assert [pool.allocate() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(PhotonError) as e:
        pool.allocate()
    assert e.value.code == ErrorCode.OUT_OF_MEMORY
    pool.free(2)
    pool.free(0)
    with pytest.raises(PhotonError) as e:
        pool.free(0)
    assert e.value.code == ErrorCode.DOUBLE_FREE
    with pytest.raises(PhotonError):
        pool.free(9)
    assert pool.allocate() == 0 and pool.allocate() == 2        # freed last, used first
    assert pool.high_water == 4 and pool.num_free == 0
    with pytest.raises(PhotonError):
        pool.allocate_many(1)


def test_groups_are_formed_by_need():
    m = _manager()
    assert len(m.groups) == 2
    assert m.groups[0].spec == WIN and m.groups[0].entries == [0, 2]
    assert m.groups[1].spec == FULL and m.groups[1].entries == [1, 3]
    assert m.entry_location == [(0, 0), (1, 0), (0, 1), (1, 1)]


def test_shared_cache_entries():
    needs = [(FULL, None), (None, None), (FULL, None)]
    m = CacheManager(needs, [None, 0, None], 8, 4, 2, torch.float32, None)
    assert m.groups[0].entries == [0, 2]
    assert m.entry_location[1] == m.entry_location[0] and m.entry_shared == [False, True, False]
    with pytest.raises(PhotonError):
        CacheManager([(None, None), (FULL, None)], [None, 0], 8, 4, 2, torch.float32, None)


def test_extend_commit_and_free():
    m = _manager(window=False)
    m.add_request("a")
    assert m.pages_needed("a", 20) == [3]
    m.extend("a", 20)
    m.extend("a", 20)                                   # asking again takes nothing more
    assert m.groups[0].pages_held("a") == 3
    m.commit("a", 20)
    assert m.length("a") == 20
    assert m.pages_needed("a", 4) == [0] and m.pages_needed("a", 5) == [1]
    m.check_consistency()
    m.free_request("a")
    assert m.free_pages() == [16]
    with pytest.raises(PhotonError) as e:
        m.free_request("a")
    assert e.value.code == ErrorCode.DOUBLE_FREE


def test_extend_is_all_or_nothing_across_groups():
    m = _manager(num_pages=4)
    m.add_request("a")
    m.extend("a", 30)                                   # 4 pages in both groups
    m.commit("a", 30)
    m.add_request("b")
    before = m.free_pages()
    with pytest.raises(PhotonError) as e:
        m.extend("b", 8)
    assert e.value.code == ErrorCode.OUT_OF_MEMORY and m.free_pages() == before
    assert not m.can_extend("b", 8)
    m.check_consistency()


def test_window_group_returns_pages():
    m = _manager(num_pages=32, page_size=8)
    m.add_request("a")
    total = 0
    for n in (5, 30, 1, 1, 40, 2, 64, 1):
        m.extend("a", n)
        m.commit("a", n)
        total += n
        win, full = m.groups
        assert full.pages_held("a") == (total + 7) // 8
        first_visible = max(0, total - 24 + 1)
        assert win.tables["a"][: first_visible // 8] == [NO_PAGE] * (first_visible // 8)
        assert all(p != NO_PAGE for p in win.tables["a"][first_visible // 8:])
        assert win.pages_held("a") <= 24 // 8 + 2
        m.check_consistency()
    # a long portion needs all of its own pages during the step, and the window's before it
    assert m.pages_needed("a", 40)[0] == (total + 40 - 1) // 8 - (total - 1) // 8


def test_slot_mapping_and_block_table():
    import numpy as np
    m = _manager(window=False, page_size=8)
    m.add_request("a"); m.add_request("b")
    m.extend("b", 3); m.commit("b", 3)                  # page 0
    m.extend("a", 20); m.commit("a", 20)                # pages 1, 2, 3
    m.extend("a", 6)
    out = np.empty(6, dtype=np.int32)
    m.fill_slot_mapping(0, "a", 20, 6, out)
    assert out.tolist() == [3 * 8 + 4, 3 * 8 + 5, 3 * 8 + 6, 3 * 8 + 7, 4 * 8 + 0, 4 * 8 + 1]
    w = m.table_width(["a", "b"])
    assert w == [8]
    table = np.empty((2, 8), dtype=np.int32)
    m.fill_block_table(0, ["a", "b"], table)
    assert table[0].tolist() == [1, 2, 3, 4, -1, -1, -1, -1] and table[1].tolist() == [0] + [-1] * 7


def test_state_slots():
    m = _manager(state=True, max_sequences=2)
    assert m.states.bytes_per_slot() == 12
    s0, s1 = m.add_request("a"), m.add_request("b")
    assert {s0, s1} == {0, 1}
    with pytest.raises(PhotonError) as e:
        m.add_request("c")
    assert e.value.code == ErrorCode.OUT_OF_MEMORY
    m.free_request("a")
    assert m.add_request("c") == s0
    with pytest.raises(PhotonError):
        m.add_request("c")
    pool = StateSlotPool(2, {0: StateSpec((2, 2))}, torch.device("cpu"))
    pool.tensors[0].fill_(7.0)
    slot = pool.allocate("x")
    assert float(pool.tensors[0][slot].abs().max()) == 0.0          # cleared when handed out
    pool.free("x")
    with pytest.raises(PhotonError):
        pool.free("x")


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    m = _manager(num_pages=24, page_size=8, max_sequences=5)
    live, lengths, next_id = [], {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            rid = f"r{next_id}"; next_id += 1
            m.add_request(rid); live.append(rid); lengths[rid] = 0
        elif op < 0.85 and live:
            rid = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 7, 19, 40])
            if m.can_extend(rid, n):
                m.extend(rid, n); m.commit(rid, n); lengths[rid] += n
            else:
                before = m.free_pages()
                with pytest.raises(PhotonError):
                    m.extend(rid, n)
                assert m.free_pages() == before
        elif live:
            rid = live.pop(rng.randrange(len(live)))
            m.free_request(rid); del lengths[rid]
        m.check_consistency()
        for rid in live:
            assert m.length(rid) == lengths[rid]
    for rid in live:
        m.free_request(rid)
    assert m.free_pages() == [24, 24] and m.states.num_free == 5
    assert all(g.pool.high_water <= 24 for g in m.groups)
