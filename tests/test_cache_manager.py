"""Cache manager bookkeeping: no page lost, held twice or freed twice, under random
orders of requests; window groups give pages back while a request lives; growth is
all or nothing; state slots are zeroed when handed out."""
import random

import numpy as np
import pytest
import torch

from arle_b200.cache import CacheManager, NoFreeSlot, OutOfPages, PagePool
from arle_b200.parts import CacheNeed, StateNeed


def manager(needs=None, states=(), page_size=4, pages=16, slots=4, max_tokens=256):
    needs = needs if needs is not None else [CacheNeed(2, 8)] * 2
    return CacheManager(needs, list(states), page_size, pages, slots, max_tokens, torch.float32, "cpu")


def test_pool_lifo_and_double_free():
    p = PagePool(4)
    assert p.alloc(2) == [0, 1]
    p.free([0])
    assert p.alloc(1) == [0]               # the page given back last is used again first
    with pytest.raises(RuntimeError, match="twice"):
        p.free([3])
    with pytest.raises(OutOfPages):
        p.alloc(3)
    assert p.num_free == 2
    p.check()


def test_tail_page_is_filled_before_a_new_one():
    m = manager()
    m.add_request("a")
    m.append([("a", 3)])
    assert m.free_pages() == [15] and m.pages_needed("a", 1) == [0] and m.pages_needed("a", 2) == [1]
    m.append([("a", 1)])
    assert m.free_pages() == [15]
    m.append([("a", 1)])
    assert m.free_pages() == [14] and m.num_tokens("a") == 5
    assert m.slot_mapping(0, "a", 0, 5).tolist() == [0, 1, 2, 3, 4]
    m.check()


def test_append_is_all_or_nothing():
    m = manager(pages=5)
    for r in "abc":
        m.add_request(r)
    m.append([("a", 8)])
    before = (m.free_pages(), m.num_tokens("a"), m.num_tokens("b"))
    with pytest.raises(OutOfPages):
        m.append([("b", 8), ("c", 8)])
    assert (m.free_pages(), m.num_tokens("a"), m.num_tokens("b")) == before
    with pytest.raises(ValueError, match="twice"):
        m.append([("b", 1), ("b", 1)])
    assert m.can_append([("b", 8), ("c", 4)]) and not m.can_append([("b", 8), ("c", 5)])
    m.check()


def test_groups_by_need_have_their_own_pages_and_windows_release():
    needs = [CacheNeed(2, 8), CacheNeed(2, 8, window=6), CacheNeed(1, 16), CacheNeed(2, 8, window=6)]
    m = manager(needs, page_size=4, pages=10)
    assert len(m.groups) == 3 and [g.layers for g in m.groups] == [[0], [1, 3], [2]]
    m.add_request("a")
    m.append([("a", 17)])
    assert m.free_pages() == [5, 5, 5]
    assert m.release_passed("a") == 3      # keys < 17 - 6 + 1 = 12 are out of sight: pages 0, 1, 2
    assert m.free_pages() == [5, 8, 5]
    assert m.block_rows(1, ["a"]).tolist() == [[-1, -1, -1, 3, 4]]
    m.append([("a", 1)])
    assert m.release_passed("a") == 0      # 18 - 6 + 1 = 13: page 3 (tokens 12..15) still seen
    m.check()
    m.free_request("a")
    assert m.free_pages() == [10, 10, 10]
    m.check()


def test_slots_and_state_arrays():
    m = manager(states=[StateNeed((3,)), StateNeed((2, 2), torch.int32)], slots=2)
    s = m.add_request("a")
    m.states[0][s] += 5
    m.add_request("b")
    with pytest.raises(NoFreeSlot):
        m.add_request("c")
    with pytest.raises(ValueError):
        m.add_request("a")
    m.free_request("a")
    s2 = m.add_request("c")
    assert s2 == s and m.states[0][s2].abs().sum() == 0 and m.states[1].dtype == torch.int32
    m.check()


def test_truncate_gives_back_whole_pages_beyond():
    m = manager()
    m.add_request("a")
    m.append([("a", 9)])
    m.truncate("a", 4)
    assert m.free_pages() == [15] and m.num_tokens("a") == 4
    m.append([("a", 1)])
    assert m.slot_mapping(0, "a", 4, 1).tolist()[0] % 4 == 0
    m.check()


def test_per_request_limit():
    m = manager(max_tokens=10)
    m.add_request("a")
    with pytest.raises(ValueError, match="more than the 10"):
        m.append([("a", 11)])


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    needs = [CacheNeed(2, 8), CacheNeed(2, 8, window=rng.choice([3, 7, 10]))]
    m = manager(needs, page_size=rng.choice([2, 4, 8]), pages=24, slots=4, max_tokens=80)
    live, n = {}, 0
    used_pages = set()
    for _ in range(400):
        op = rng.random()
        if op < 0.2 and len(live) < 4:
            rid = f"r{n}"
            n += 1
            m.add_request(rid)
            live[rid] = 0
        elif op < 0.85 and live:
            k = rng.randint(1, min(3, len(live)))
            items = [(r, rng.choice([1, 1, 2, 5, 9])) for r in rng.sample(sorted(live), k)]
            items = [(r, c) for r, c in items if live[r] + c <= 80]
            if not items:
                continue
            ok = m.can_append(items)
            try:
                m.append(items)
                assert ok
                for r, c in items:
                    sm = m.slot_mapping(0, r, live[r], c)
                    used_pages.update((sm // m.page_size).tolist())
                    live[r] += c
                    m.release_passed(r)
            except OutOfPages:
                assert not ok
        elif live:
            rid = rng.choice(sorted(live))
            m.free_request(rid)
            del live[rid]
        m.check()
        for r, c in live.items():
            assert m.num_tokens(r) == c
        # no two live requests share a physical page in any group
        for gi, g in enumerate(m.groups):
            rows = m.block_rows(gi, sorted(live)) if live else np.zeros((0, 1), dtype=np.int32)
            held = rows[rows >= 0]
            assert len(set(held.tolist())) == held.size
    for rid in sorted(live):
        m.free_request(rid)
    m.check()
    assert all(f == 24 for f in m.free_pages())


def test_a_need_names_its_own_per_token_arrays():
    """Attention keeps keys and values of one shape; a mixer may name other arrays (one compressed
    vector per token; keys wider than values).  Each stream gets pages of its own shape per layer,
    all under the group's one block table, and the bytes per token follow."""
    needs = [CacheNeed(2, 8), CacheNeed(streams=((1, 24),)), CacheNeed(streams=((2, 16), (2, 8))), CacheNeed(streams=((1, 24),))]
    cm = CacheManager(needs, [], 4, 10, 2, 40, torch.float32, "cpu")
    assert [len(g.arrays) for g in cm.groups] == [2, 1, 2] and [g.layers for g in cm.groups] == [[0], [1, 3], [2]]
    assert [tuple(a.shape) for a in cm.groups[1].arrays] == [(2, 10, 1, 4, 24)]
    assert [tuple(a.shape) for a in cm.groups[2].arrays] == [(1, 10, 2, 4, 16), (1, 10, 2, 4, 8)]
    assert cm.bytes_per_token() == (2 * 2 * 8 + 2 * 24 + 2 * 16 + 2 * 8) * 4
    cm.add_request("a")
    cm.append([("a", 9)])
    bt = torch.zeros(1, 3, dtype=torch.int32)
    view = cm.layer_view(3, bt, torch.zeros(9, dtype=torch.int32), True)
    assert len(view.streams) == 1 and tuple(view.streams[0].shape) == (10, 1, 4, 24)
    view = cm.layer_view(2, bt, torch.zeros(9, dtype=torch.int32), True)
    assert tuple(view.k.shape) == (10, 2, 4, 16) and tuple(view.v.shape) == (10, 2, 4, 8)
    cm.free_request("a")
    cm.check()
