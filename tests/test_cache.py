"""The cache manager's accounting, without a GPU: no page lost, held twice or freed twice, under
random orders of requests; groups; windows; reuse; state slots."""
import random

import pytest
import torch

from fellm_b200.cache import CacheManager, PageAllocator
from fellm_b200.config import CacheError
from fellm_b200.parts.base import FixedState, PagedKV

FULL = PagedKV(2, 16, None)
WIN = PagedKV(1, 32, 24)
CONV = FixedState((2, 8))


def make(needs=(CONV, FULL, CONV, FULL), page_tokens=8, max_tokens=64, max_requests=4, n_ctx=128):
    return CacheManager(list(needs), page_tokens=page_tokens, max_tokens=max_tokens, max_requests=max_requests,
                        n_ctx=n_ctx, dtype=torch.float32, device="cpu")


def test_allocator_discipline():
    a = PageAllocator(3)
    p = [a.alloc(), a.alloc(), a.alloc()]
    assert sorted(p) == [0, 1, 2] and a.free_count == 0
    with pytest.raises(CacheError, match="out of cache pages"):
        a.alloc()
    a.free(p[1])
    with pytest.raises(CacheError, match="freed but not held"):
        a.free(p[1])
    with pytest.raises(CacheError):
        a.free(7)
    assert a.alloc() == p[1]                       # the page freed last is used next


def test_groups_by_need():
    c = make((CONV, FULL, CONV, FULL, WIN, None))
    assert len(c.paged) == 2 and len(c.fixed) == 1
    # 8 pages and 4 slots to hand out, and one page and one slot more that nobody gets: the padding rows' own
    assert c.paged[0].pool.shape == (9, 2, 2, 2, 8, 16)          # pages, layers, k/v, G, tokens, hd
    assert c.paged[1].pool.shape == (9, 1, 2, 1, 8, 32)
    assert c.fixed[0].states.shape == (5, 2, 2, 8)
    assert c.n_pages == 8 and c.free_pages() == 8 and c.pad_slot == 4
    for g in c.paged:
        assert int(g.table_host[c.pad_slot, 0]) == 8 and int(g.table_host[c.pad_slot, 1]) == -1
    v = c.views(None)
    assert v[1].layer == 0 and v[3].layer == 1 and v[4].window == 24 and v[5] is None
    assert v[0].states.shape == (5, 2, 8) and v[2].states.data_ptr() != v[0].states.data_ptr()


def test_reserve_advance_release_and_reuse():
    c = make()
    c.add_request("a")
    c.reserve("a", 20)
    c.advance("a", 20)
    assert c.length("a") == 20 and c.free_pages() == 8 - 3
    held = c.paged[0].held_pages(c.slot("a"))
    assert len(held) == 3
    c.reserve("a", 4)                               # 24 tokens: still 3 pages
    c.advance("a", 4)
    assert c.free_pages() == 5
    c.reserve("a", 1)
    c.advance("a", 1)
    assert c.free_pages() == 4
    c.audit()
    held = c.paged[0].held_pages(c.slot("a"))
    c.release("a")
    assert c.free_pages() == 8
    c.add_request("b")
    c.reserve("b", 8)
    assert c.paged[0].held_pages(c.slot("b"))[0] in held
    c.audit()
    with pytest.raises(CacheError, match="released but not live"):
        c.release("a")
    with pytest.raises(CacheError, match="already live"):
        c.add_request("b")


def test_freed_pages_are_used_next():
    c = make(max_tokens=32)
    c.add_request("a"); c.reserve("a", 16); c.advance("a", 16)
    pages_a = c.paged[0].held_pages(c.slot("a"))
    c.release("a")
    c.add_request("b"); c.reserve("b", 16)
    assert set(c.paged[0].held_pages(c.slot("b"))) == set(pages_a)


def test_all_or_nothing_and_context_limit():
    c = make(max_tokens=32, n_ctx=40)
    c.add_request("a"); c.add_request("b")
    c.reserve("a", 24); c.advance("a", 24)
    assert not c.can_reserve([("b", 16)])
    with pytest.raises(CacheError, match="out of cache pages"):
        c.reserve("b", 16)
    assert c.free_pages() == 1 and c.length("b") == 0
    c.audit()
    assert c.can_reserve([("b", 8)]) and not c.can_reserve([("a", 1), ("b", 8)])
    with pytest.raises(CacheError, match="context holds 40"):
        c.reserve("a", 17)
    c2 = make(max_requests=2)
    c2.add_request(1); c2.add_request(2)
    assert not c2.can_admit()
    with pytest.raises(CacheError, match="out of request slots"):
        c2.add_request(3)


def test_state_slot_zeroed_on_admission():
    c = make()
    s = c.add_request("a")
    c.fixed[0].states[s].fill_(3.0)
    c.release("a")
    s2 = c.add_request("b")
    assert s2 == s and float(c.fixed[0].states[s2].abs().sum()) == 0.0


def test_window_gives_pages_back():
    c = make((WIN,), page_tokens=8, max_tokens=48, n_ctx=512)
    c.add_request("a")
    total = 0
    for n in (8, 8, 8, 5, 3, 8, 16, 1, 1, 16, 2, 7):
        c.reserve("a", n); c.advance("a", n)
        total += n
        g = c.paged[0]
        slot = c.slot("a")
        first_needed = max(0, total - 24 + 1) // 8          # page of the oldest key the next query reads
        assert g.first_page[slot] == first_needed
        assert len(g.held_pages(slot)) == -(-total // 8) - first_needed
        assert all(int(g.table_host[slot, i]) == -1 for i in range(first_needed))
        c.audit()
    assert total > 48                                       # more tokens went through than the pool holds


def test_block_table_mirror_and_flush():
    c = make()
    c.add_request("a"); c.reserve("a", 17)
    g = c.paged[0]
    assert g.dirty[c.slot("a")] == [0, 3]
    c.flush()
    assert torch.equal(g.table_dev, g.table_host) and not g.dirty
    c.advance("a", 17); c.release("a"); c.flush()
    assert int(g.table_dev[:c.pad_slot].max()) == -1        # (the row behind the slots is the padding rows' own)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_share_a_page(seed):
    rng = random.Random(seed)
    c = make((CONV, FULL, WIN, FULL), page_tokens=8, max_tokens=96, max_requests=4, n_ctx=200)
    live, next_id = [], 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and c.can_admit():
            c.add_request(next_id); live.append(next_id); next_id += 1
        elif op < 0.85 and live:
            r = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 3, 5, 8, 13, 21])
            if c.length(r) + n <= c.n_ctx and c.can_reserve([(r, n)]):
                c.reserve(r, n); c.advance(r, n)
            else:
                with pytest.raises(CacheError):
                    c.reserve(r, n)
        elif live:
            r = live.pop(rng.randrange(len(live)))
            c.release(r)
        c.audit()
    for r in live:
        c.release(r)
    c.audit()
    assert all(g.alloc.free_count == g.alloc.n_pages for g in c.paged) and c.slots.free_count == 4
