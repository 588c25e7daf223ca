"""The cache manager's bookkeeping (no GPU): no page is lost, held twice or freed twice, under
random orders of requests; groups with a window give pages back; a step's pages are all-or-nothing."""
import random

import pytest

from nanoinfer_b200.cache import CacheError, CacheManager, PagePool, PoolExhausted
from nanoinfer_b200.parts.base import KVCacheSpec, StateSpec

FULL = KVCacheSpec(n_kv_head=2, head_dim=16, window=0)
WIN = KVCacheSpec(n_kv_head=1, head_dim=32, window=40)


def manager(max_tokens=256, max_requests=4, needs=None, **kw):
    needs = needs if needs is not None else [(0, FULL), (1, FULL)]
    return CacheManager(needs, kw.pop("state_needs", []), max_tokens=max_tokens, max_requests=max_requests,
                        page_size=16, device=None, **kw)


def test_pool_order_and_errors():
    p = PagePool(3)
    assert [p.take(), p.take(), p.take()] == [0, 1, 2]      # page 0 is handed out first
    with pytest.raises(PoolExhausted):
        p.take()
    p.give_back(1)
    with pytest.raises(CacheError):
        p.give_back(1)                                        # freed twice
    with pytest.raises(CacheError):
        p.give_back(7)
    assert p.take() == 1                                      # given back, used again at once
    p.check()


def test_layers_with_the_same_need_share_a_group():
    m = manager(needs=[(0, FULL), (1, WIN), (2, FULL), (3, WIN)])
    assert len(m.groups) == 2
    assert m.groups[0].owners == [0, 2] and m.groups[1].owners == [1, 3]
    assert m.group_index(3) == 1 and m.groups[1].layer_of(3) == 1


def test_pages_follow_the_length_and_come_back():
    m = manager(max_tokens=64)                                # 4 pages
    a = m.open_request()
    assert m.pages_needed(a, 17) == [2]
    m.append([(a, 17)]); m.commit(a, 17)
    assert a.blocks == [[0, 1]] and a.n_tokens == 17
    assert m.pages_needed(a, 15) == [0] and m.pages_needed(a, 16) == [1]
    b = m.open_request()
    m.append([(b, 30)]); m.commit(b, 30)
    assert b.blocks == [[2, 3]] and m.pages_free() == [0]
    m.close_request(a)
    assert m.pages_free() == [2]
    c = m.open_request()
    m.append([(c, 20)]); m.commit(c, 20)
    assert sorted(c.blocks[0]) == [0, 1]                      # a's pages are used again
    m.check()
    with pytest.raises(CacheError):
        m.close_request(a)                                    # not live any more


def test_a_step_takes_all_its_pages_or_none():
    m = manager(max_tokens=64)
    a, b = m.open_request(), m.open_request()
    m.append([(a, 33)]); m.commit(a, 33)                      # 3 of 4 pages
    before = (list(a.blocks[0]), list(b.blocks[0]), m.pages_free())
    assert not m.can_append([(a, 1), (b, 17)])
    with pytest.raises(PoolExhausted):
        m.append([(a, 1), (b, 17)])                           # needs 0 + 2 pages, one is free
    assert (list(a.blocks[0]), list(b.blocks[0]), m.pages_free()) == before
    m.append([(a, 1), (b, 16)])
    m.check()


def test_context_limit_and_slots():
    m = manager(max_tokens=512, max_requests=2, max_positions=64)
    a = m.open_request()
    with pytest.raises(CacheError, match="context full"):
        m.append([(a, 65)])
    m.append([(a, 64)])
    m.open_request()
    with pytest.raises(PoolExhausted, match="slot"):
        m.open_request()
    assert m.max_blocks == [4]


def test_window_group_gives_pages_back_as_the_window_passes():
    m = manager(max_tokens=1024, needs=[(0, FULL), (1, WIN)])
    full, win = (0, 1) if m.groups[0].spec is FULL or m.groups[0].spec == FULL else (1, 0)
    a = m.open_request()
    held = []
    for n in [50, 1, 1, 30, 7, 64, 1]:
        m.append([(a, n)]); m.commit(a, n)
        m.check()
        blocks = a.blocks[win]
        first_needed = max(0, a.n_tokens - WIN.window + 1) // 16
        assert all(p == -1 for p in blocks[:first_needed])              # passed pages went back
        assert all(p >= 0 for p in blocks[first_needed:])               # the window's pages are held
        assert all(p >= 0 for p in a.blocks[full])                      # the other group keeps everything
        held.append(sum(1 for p in blocks if p >= 0))
    assert max(held[1:]) <= (WIN.window + 16) // 16 + 1
    assert m.pages_used()[full] == -(-a.n_tokens // 16)
    m.close_request(a)
    assert m.pages_used() == [0, 0]


def test_truncate_gives_back_whole_pages_past_the_length():
    m = manager()
    a = m.open_request()
    m.append([(a, 50)]); m.commit(a, 50)
    m.truncate(a, 33)
    assert a.n_tokens == 33 and len(a.blocks[0]) == 3 and m.pages_used() == [3]
    m.truncate(a, 32)
    assert len(a.blocks[0]) == 2
    with pytest.raises(CacheError):
        m.truncate(a, 40)
    m.check()


def test_state_slots_are_per_request():
    m = manager(state_needs=[(1, StateSpec((4, 8)))], max_requests=3)
    a, b = m.open_request(), m.open_request()
    assert a.slot != b.slot
    m.close_request(a)
    c = m.open_request()
    assert c.slot == a.slot                                   # the slot is used again
    m.check()
    with pytest.raises(CacheError):
        m.append([(b, 5)]); m.commit(b, 5); m.truncate(b, 2)  # state cannot be rolled back


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    needs = [(0, FULL), (1, WIN), (2, FULL)] if seed % 2 else [(0, FULL)]
    m = manager(max_tokens=rng.choice([96, 160, 320]), max_requests=4, needs=needs, max_positions=200)
    live = []
    total = m.groups[0].pool.n_pages
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            live.append(m.open_request())
        elif op < 0.40 and live:
            m.close_request(live.pop(rng.randrange(len(live))))
        elif live:
            k = rng.randint(1, len(live))
            work = [(r, rng.choice([1, 1, 1, 2, 5, 16, 17, 40])) for r in rng.sample(live, k)]
            work = [(r, n) for r, n in work if r.n_tokens + n <= 200]
            if not work:
                continue
            if m.can_append(work):
                m.append(work)
                for r, n in work:
                    m.commit(r, n)
            else:
                before = m.pages_free()
                with pytest.raises(PoolExhausted):
                    m.append(work)
                assert m.pages_free() == before
        m.check()
        for gi, g in enumerate(m.groups):
            held = sum(1 for r in live for p in r.blocks[gi] if p >= 0)
            assert held + g.pool.n_free == g.pool.n_pages
            for r in live:                                    # every position a query may read has a page
                lo = max(0, r.n_tokens - g.spec.window + 1) if g.spec.window else 0
                assert all(r.blocks[gi][j // 16] >= 0 for j in range(lo, r.n_tokens))
    for r in live:
        m.close_request(r)
    assert all(g.pool.n_free == g.pool.n_pages for g in m.groups) and m.slots.n_free == 4
    assert total == m.groups[0].pool.n_pages


def test_padding_page_and_slot_lie_outside_the_pools():
    """With ``padding`` the cache has one page per group and one state slot that no request can get."""
    import torch
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.parts.base import KVCacheSpec
    needs = [(0, KVCacheSpec(2, 16, 0)), (1, KVCacheSpec(2, 16, 8))]
    c = CacheManager(needs, [], max_tokens=64, max_requests=3, page_size=16, dtype=torch.float32,
                     device=torch.device("cpu"), padding=True)
    assert c.pad_slot == 3 and c.pad_page == [4, 4]
    assert [g.tensor.shape[1] for g in c.groups] == [5, 5]
    reqs = [c.open_request() for _ in range(3)]
    assert sorted(r.slot for r in reqs) == [0, 1, 2]
    c.append([(reqs[0], 33), (reqs[1], 16)])
    for r in reqs[:2]:
        c.commit(r, 33 if r is reqs[0] else 16)
    held = {p for r in reqs for blocks in r.blocks for p in blocks}
    assert 4 not in held and c.pages_free()[0] == 0
    c.check()
    plain = CacheManager(needs, [], max_tokens=64, max_requests=3, page_size=16, dtype=torch.float32,
                         device=torch.device("cpu"))
    assert plain.pad_slot is None and plain.pad_page is None and plain.groups[0].tensor.shape[1] == 4
