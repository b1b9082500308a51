"""The cache's host-side ledger: no slot or page is lost, held twice or freed twice."""
import random

import pytest

from catena_models_b200.cache.allocators import CacheError, CacheFull, IndexAllocator
from catena_models_b200.cache.cache import CacheBook
from catena_models_b200.cache.spec import FixedStateSpec, KVStateSpec


def test_index_allocator_lowest_first_and_guards():
    a = IndexAllocator(4, "slot")
    assert a.take(2) == [0, 1]
    a.give_back([0])
    assert a.take(1) == [0]                      # the lowest free index is used again
    with pytest.raises(CacheError):
        a.give_back([3])                         # never taken
    a.give_back([1])
    with pytest.raises(CacheError):
        a.give_back([1])                         # freed twice
    with pytest.raises(CacheError):
        a.give_back([0, 0])
    with pytest.raises(CacheFull):
        a.take(4)
    assert a.free_count == 3 and a.held == {0}


def test_spec_geometry():
    full, ring = KVStateSpec(2, 16), KVStateSpec(2, 16, window=70)
    assert full.ring == 0 and ring.ring == 128
    assert [full.pages(n) for n in (0, 1, 64, 65)] == [0, 1, 1, 2]
    assert [ring.pages(n) for n in (1, 64, 65, 128, 500)] == [1, 1, 2, 2, 2]
    assert ring.entries(500) == 128 and full.entries(500) == 500
    assert FixedStateSpec((2, 64)) == FixedStateSpec((2, 64), "float32")


def test_sizing_from_max_tokens():
    book = CacheBook([KVStateSpec(2, 16), KVStateSpec(2, 16, window=16)], max_tokens=1000, max_len=512)
    assert book.page_budget == 16 and book.max_seqs == 16
    assert book.group_pages == [16, 16] and book.pages_per_seq == [8, 1]


def test_reserve_is_all_or_nothing_and_release_returns_everything():
    book = CacheBook([KVStateSpec(1, 8), KVStateSpec(1, 8, window=64)], max_tokens=256)
    a, b = book.admit(), book.admit()
    ups = book.reserve(a, 130)
    assert [(g, j) for g, j, _ in ups] == [(0, 0), (0, 1), (0, 2), (1, 0)]
    book.advance(a, 130)
    assert book.reserve(a, 131) == []            # same pages
    with pytest.raises(CacheFull):
        book.reserve(b, 129)                     # three more pages wanted, one free in the growing group
    assert book.page_alloc[0].free_count == 1 and book.page_alloc[1].free_count == 3
    assert book.reserve(b, 64) and book.page_alloc[0].free_count == 0
    book.release(a)
    assert book.page_alloc[0].free_count == 3
    with pytest.raises(CacheError):
        book.release(a)                          # a slot is not released twice
    with pytest.raises(CacheError):
        book.reserve(a, 1)                       # nor used after its release
    book.release(b)
    assert book.page_alloc[0].free_count == 4 and book.slots.free_count == book.max_seqs


def test_random_traffic_conserves_slots_and_pages():
    rng = random.Random(0)
    specs = [KVStateSpec(2, 16), KVStateSpec(2, 16, window=100)]
    book = CacheBook(specs, max_tokens=64 * 40, max_seqs=12, max_len=64 * 40)
    live = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.25 and book.slots.free_count:
            s = book.admit()
            assert s not in live
            live[s] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = live[s] + rng.choice([1, 1, 1, 17, 64, 200])
            try:
                book.reserve(s, n)
                book.advance(s, n)
                live[s] = n
            except CacheFull:
                pass
        elif live:
            s = rng.choice(list(live))
            book.release(s)
            del live[s]
        # invariants: every page is either free or held by exactly one sequence
        for g, spec in enumerate(specs):
            held = [p for s in live for p in book.pages[s][g]]
            assert len(held) == len(set(held)) == book.group_pages[g] - book.page_alloc[g].free_count
            for s, n in live.items():
                assert len(book.pages[s][g]) >= spec.pages(n)
        assert set(book.live) == set(live) and book.slots.free_count == 12 - len(live)
    for s in list(live):
        book.release(s)
    assert all(a.free_count == n for a, n in zip(book.page_alloc, book.group_pages))
