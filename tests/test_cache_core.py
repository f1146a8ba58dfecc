"""The cache manager's host side (C++ core through its bindings): allocator, hash, prefix cache,
paged and contiguous policies, layer groups with windows, state slots.  No GPU.

Invariants after the reference's tests (tests/test_block_allocator.cpp, tests/test_managers.cpp,
tests/test_prefix_cache.cpp): no page lost, none held twice, none freed twice, under random
orders of requests."""
import random

import pytest

from kvcm.cache import core


def make_seq(sid, tokens):
    s = core.Sequence()
    s.id = sid
    s.tokens = list(tokens)
    s.prompt_len = len(tokens)
    return s


# ------------------------------------------------------------------------------- hash

def test_xxh64_known_vectors():
    # Published XXH64 test values (seed 0), the ones the reference checks too.
    assert core.xxh64(b"", 0) == 0xEF46DB3751D8E999
    assert core.xxh64(b"a", 0) == 0xD24EC4F1A98C6E5B
    assert core.xxh64(b"abc", 0) == 0x44BC2CF5AD770999
    assert core.xxh64(b"Nobody inspects the spammish repetition", 0) == 0xFBCEA83C8A378BF1


def test_page_hash_chains_on_the_parent():
    a = core.page_hash(0, [1, 2, 3, 4])
    assert core.page_hash(0, [1, 2, 3, 4]) == a
    assert core.page_hash(a, [1, 2, 3, 4]) != a
    assert core.page_hash(0, [1, 2, 3, 5]) != a


# -------------------------------------------------------------------------- allocator

def test_allocator_hands_out_all_then_none():
    a = core.BlockAllocator(5)
    got = [a.allocate() for _ in range(5)]
    assert got == [0, 1, 2, 3, 4] and a.allocate() == -1 and a.num_free() == 0
    for g in got:
        a.free(g)
    assert a.num_free() == 5
    assert a.allocate() == 4                       # LIFO reuse


def test_allocator_refcounts_and_misuse():
    a = core.BlockAllocator(2)
    b = a.allocate()
    a.incref(b)
    a.free(b)
    assert a.refcount(b) == 1 and not a.is_free(b)
    a.free(b)
    assert a.is_free(b)
    with pytest.raises(Exception):
        a.free(b)                                  # freed twice
    with pytest.raises(Exception):
        a.incref(b)                                # incref on a free page
    with pytest.raises(Exception):
        a.push_free(1)                             # already free
    with pytest.raises(Exception):
        a.free(7)                                  # outside the pool


def test_allocator_random_ops_against_a_shadow():
    rng = random.Random(0)
    n = 64
    a = core.BlockAllocator(n)
    shadow = [0] * n
    for _ in range(50000):
        op = rng.random()
        held = [i for i in range(n) if shadow[i] > 0]
        if op < 0.4:
            b = a.allocate()
            if b < 0:
                assert len(held) == n
            else:
                assert shadow[b] == 0
                shadow[b] = 1
        elif op < 0.6 and held:
            b = rng.choice(held)
            a.incref(b)
            shadow[b] += 1
        elif held:
            b = rng.choice(held)
            a.free(b)
            shadow[b] -= 1
        assert a.num_free() == sum(1 for c in shadow if c == 0)
    for i in range(n):
        assert a.refcount(i) == shadow[i]


# ----------------------------------------------------------------------- prefix cache

def test_prefix_hit_partial_and_miss():
    B = 4
    m = core.PagedManager(16, B, 64, True, 0)
    t1 = list(range(100, 113))                    # 13 tokens: 3 full pages + 1
    s1 = make_seq(1, t1)
    assert m.can_admit(s1)
    m.admit(s1)
    assert s1.num_computed == 0 and m.ensure(s1, 13) and len(s1.table(0)) == 4
    s1.num_computed = 13
    m.commit(s1)
    assert m.num_hashed() == 3
    # same first two pages, then diverges
    s2 = make_seq(2, t1[:8] + [7, 7, 7, 7, 7])
    m.admit(s2)
    assert s2.cached_tokens == 8 and s2.num_computed == 8 and s2.table(0) == s1.table(0)[:2]
    assert m.refcount(s1.table(0)[0]) == 2
    # first page differs: nothing shared
    s3 = make_seq(3, [9] + t1[1:])
    m.admit(s3)
    assert s3.cached_tokens == 0
    for s in (s3, s2, s1):
        m.release(s)
    assert m.blocks_in_use() == 0


def test_full_prompt_hit_still_computes_the_last_token():
    B = 4
    m = core.PagedManager(8, B, 64, True, 0)
    t = list(range(8))
    s1 = make_seq(1, t)
    m.admit(s1); m.ensure(s1, 8); s1.num_computed = 8; m.commit(s1); m.release(s1)
    s2 = make_seq(2, t)
    m.admit(s2)
    assert s2.cached_tokens == 4                  # the page that holds the last token is not shared


def test_released_pages_stay_findable_and_are_recycled_oldest_first():
    B = 4
    m = core.PagedManager(4, B, 64, True, 0)
    s1 = make_seq(1, list(range(12)) + [0])
    m.admit(s1); m.ensure(s1, 13); s1.num_computed = 13; m.commit(s1)
    pages = s1.table(0)
    m.release(s1)
    assert m.blocks_in_use() == 0 and m.blocks_cached_free() == 3
    assert m.lru_order() == [pages[2], pages[1], pages[0]]      # tail parked first, head last
    s2 = make_seq(2, list(range(12)) + [0])
    assert m.can_admit(s2)
    m.admit(s2)
    assert s2.cached_tokens == 12 and m.blocks_cached_free() == 0
    m.release(s2)
    # a different request needs all 4 pages: the parked ones are recycled, tail of the prefix first
    s3 = make_seq(3, [50 + i for i in range(16)])
    m.admit(s3)
    assert m.ensure(s3, 16)
    assert m.prefix_stats().evictions == 3 and m.num_hashed() == 0


def test_can_admit_counts_parked_hits_against_what_is_available():
    B = 4
    m = core.PagedManager(4, B, 64, True, 0)
    s1 = make_seq(1, list(range(9)))
    m.admit(s1); m.ensure(s1, 9); s1.num_computed = 9; m.commit(s1); m.release(s1)
    assert m.blocks_cached_free() == 2
    # 5 pages, 2 of them hits that sit parked: 3 more from (2 free + 2 parked - 2 parked hits) = 2
    s2 = make_seq(2, list(range(8)) + [3] * 12)
    assert not m.can_admit(s2)
    s3 = make_seq(3, list(range(8)) + [3] * 8)
    assert m.can_admit(s3)


def test_disabled_cache_never_shares():
    m = core.PagedManager(8, 4, 64, False, 0)
    s1 = make_seq(1, list(range(9)))
    m.admit(s1); m.ensure(s1, 9); s1.num_computed = 9; m.commit(s1)
    s2 = make_seq(2, list(range(9)))
    m.admit(s2)
    assert s2.cached_tokens == 0 and m.name() == "paged"


def test_prefix_caching_refuses_windows_and_many_groups():
    with pytest.raises(Exception):
        core.PagedManager(8, 4, 64, True, 0, [core.LayerGroupSpec(0), core.LayerGroupSpec(0)])
    with pytest.raises(Exception):
        core.PagedManager(8, 4, 64, True, 0, [core.LayerGroupSpec(16)])


# ---------------------------------------------------------------------------- managers

def test_paged_takes_pages_on_demand():
    B = 16
    m = core.PagedManager(8, B, 128, False, 0)
    s = make_seq(1, [1] * 20)
    m.admit(s)
    assert m.ensure(s, 20) and len(s.table(0)) == 2
    for n in range(21, 33):
        s.append_token(1)
        assert m.ensure(s, n) and len(s.table(0)) == 2
    s.append_token(1)
    assert m.ensure(s, 33) and len(s.table(0)) == 3      # the third page appears at token 33
    m.release(s)
    assert m.blocks_in_use() == 0


def test_paged_ensure_fails_when_the_pool_is_empty():
    m = core.PagedManager(2, 4, 64, False, 0)
    s = make_seq(1, [1] * 8)
    m.admit(s)
    assert m.ensure(s, 8)
    s.append_token(1)
    assert not m.ensure(s, 9)
    m.release(s)
    assert m.num_free() == 2


def test_watermark_keeps_pages_spare_at_admission():
    m = core.PagedManager(10, 4, 64, False, 2)
    assert m.can_admit(make_seq(1, [1] * 32))            # 8 pages <= 10 - 2
    assert not m.can_admit(make_seq(2, [1] * 33))        # 9 pages
    assert not m.can_admit(make_seq(3, [1] * 65))        # longer than max_seq_len


def test_contiguous_reserves_consecutive_pages_and_coalesces():
    m = core.ContiguousManager(64, 16, 256)
    assert m.reserve_blocks() == 16
    seqs = [make_seq(i, [1] * 10) for i in range(4)]
    for s in seqs:
        assert m.can_admit(s)
        m.admit(s)
        t = s.table(0)
        assert t == list(range(t[0], t[0] + 16))
    assert not m.can_admit(make_seq(9, [1]))
    m.release(seqs[1])
    m.release(seqs[2])
    assert m.num_free_extents() == 1                     # neighbours merged
    m.release(seqs[0]); m.release(seqs[3])
    assert m.num_free_extents() == 1 and m.blocks_in_use() == 0
    s = make_seq(5, [1] * 10)
    m.admit(s)
    assert m.ensure(s, 256) and not m.ensure(s, 257)


def test_factory_and_unknown_policy():
    c = core.KVManagerConfig()
    c.num_blocks, c.watermark_blocks = 200, -1
    m = core.make_kv_manager(c)
    assert m.name() == "paged" and m.can_admit(make_seq(1, [1] * 16 * 198)) is False   # 1 % spare = 2
    c.policy = "contiguous"
    assert core.make_kv_manager(c).name() == "contiguous"
    c.policy = "nope"
    with pytest.raises(Exception):
        core.make_kv_manager(c)


@pytest.mark.parametrize("policy", ["paged", "paged+prefix", "contiguous", "two-groups"])
def test_random_churn_no_page_lost_held_twice_or_freed_twice(policy):
    rng = random.Random(1)
    B, N = 4, 48
    groups = [core.LayerGroupSpec(0)]
    if policy == "two-groups":
        groups = [core.LayerGroupSpec(0), core.LayerGroupSpec(8)]
    if policy == "contiguous":
        m = core.ContiguousManager(N, B, 32)
    else:
        m = core.PagedManager(N, B, 64, policy == "paged+prefix", 0, groups)
    live = []
    next_id = 0
    for _ in range(6000):
        r = rng.random()
        if r < 0.3:
            n = rng.randint(1, 24)
            # few distinct prefixes so that the prefix cache sees hits
            toks = [rng.randint(0, 1)] * min(n, 8) + [rng.randint(0, 50) for _ in range(max(0, n - 8))]
            s = make_seq(next_id, toks)
            next_id += 1
            if m.can_admit(s):
                m.admit(s)
                assert m.ensure(s, s.length())
                s.num_computed = s.length()
                m.commit(s)
                live.append(s)
        elif r < 0.7 and live:
            s = rng.choice(live)
            s.append_token(rng.randint(0, 50))
            if m.ensure(s, s.length()):
                s.num_computed = s.length()
                m.commit(s)
            else:
                live.remove(s)
                m.release(s)
        elif live:
            s = live.pop(rng.randrange(len(live)))
            m.release(s)
            assert all(len(s.table(g)) == 0 for g in range(m.num_groups()))
        # invariants
        for g in range(m.num_groups()):
            holders = {}
            for s in live:
                for p in s.table(g):
                    if p >= 0:
                        holders[p] = holders.get(p, 0) + 1
            if policy == "paged+prefix":
                for p, c in holders.items():
                    assert m.refcount(p) == c            # shared pages are counted once per holder
            elif policy != "contiguous":
                assert all(c == 1 for c in holders.values()), "a page is held twice"
                assert m.blocks_in_use(g) == len(holders)
                assert m.num_free(g) == N - len(holders)
            else:
                assert all(c == 1 for c in holders.values())
                assert m.blocks_in_use() == len(holders)
    for s in live:
        m.release(s)
    for g in range(m.num_groups()):
        assert m.blocks_in_use(g) == 0, "pages lost"


def test_window_group_gives_back_passed_pages():
    B, W = 4, 6
    m = core.PagedManager(16, B, 256, False, 0, [core.LayerGroupSpec(0), core.LayerGroupSpec(W)])
    s = make_seq(1, [1] * 30)
    m.admit(s)
    assert m.ensure(s, 30)
    assert len(s.table(0)) == 8 and len(s.table(1)) == 8     # the portion itself needs all pages
    s.num_computed = 30
    m.commit(s)
    # next query at position 30 reads keys 25..30: pages 0..5 (positions < 24) are dead
    assert s.table(1)[:6] == [-1] * 6 and all(p >= 0 for p in s.table(1)[6:])
    assert all(p >= 0 for p in s.table(0))
    assert m.blocks_in_use(1) == 2 and m.blocks_in_use(0) == 8
    for _ in range(30):                                       # decoding: the window group stays small
        s.append_token(1)
        assert m.ensure(s, s.length())
        s.num_computed = s.length()
        m.commit(s)
        assert m.blocks_in_use(1) <= (W + B - 1) // B + 1
    m.release(s)
    assert m.blocks_in_use(0) == 0 and m.blocks_in_use(1) == 0


def test_kv_stats_accounting():
    m = core.PagedManager(8, 4, 64, False, 0)
    s = make_seq(1, [1] * 6)
    m.admit(s); m.ensure(s, 6); s.num_computed = 6
    st = m.stats([s])
    assert (st.blocks_in_use, st.allocated_slots, st.used_slots, st.tail_waste_slots) == (2, 8, 6, 2)
    assert abs(st.fragmentation() - 0.25) < 1e-9
    c = core.ContiguousManager(8, 4, 16)
    q = make_seq(2, [1] * 6)
    c.admit(q); q.num_computed = 6
    st = c.stats([q])
    assert st.reserved_unused_slots == 8 and st.tail_waste_slots == 2 and st.used_slots == 6


# -------------------------------------------------------------------------- state slots

def test_state_slots():
    s = core.StateSlots(3)
    got = [s.take() for _ in range(3)]
    assert sorted(got) == [0, 1, 2] and s.take() == -1 and s.num_taken() == 3
    s.give_back(1)
    assert not s.is_taken(1) and s.take() == 1
    with pytest.raises(Exception):
        s.give_back(7)
    s.give_back(0)
    with pytest.raises(Exception):
        s.give_back(0)
