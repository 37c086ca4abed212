"""The cache manager on the host: no page is lost, held twice or freed twice, under
random orders of requests; windows give pages back; tables point at the sink where
nothing is held (reference: pagemap_fuzz and check(), src/cuda/qwen2/pages.rs:322-438)."""

import random

import numpy as np
import pytest

from axon_b200.kernels import lib


@pytest.fixture(scope="module")
def host():
    return lib.host()


def test_allocator_basics(host):
    a = host.PageAllocator(4)
    pages = [a.alloc() for _ in range(4)]
    assert pages == [0, 1, 2, 3] and a.alloc() == -1
    a.release(2)
    assert a.n_free == 0 and a.n_retired == 1      # two-phase: not free before the flush
    assert a.alloc() == -1
    a.flush()
    assert a.alloc() == 2
    a.check()
    with pytest.raises(host.CacheError, match="freed twice"):
        a.release(1), a.release(1)
    a.retain(0)
    a.release(0)
    assert a.refs(0) == 1
    a.check()


def test_shuffled_hand_out_is_a_permutation(host):
    a = host.PageAllocator(50, shuffle_seed=7)
    pages = [a.alloc() for _ in range(50)]
    assert sorted(pages) == list(range(50)) and pages != list(range(50))
    b = host.PageAllocator(50, shuffle_seed=7)
    assert [b.alloc() for _ in range(50)] == pages


def test_reserve_is_all_or_nothing_and_tables_follow(host):
    m = host.CacheManager([host.GroupConfig(4, 6)], max_slots=3, max_positions=40)
    s = m.open_slot()
    assert m.reserve(s, 9)                         # 3 pages
    t = m.table(0)
    assert t.shape == (3, 10)
    assert list(t[s, :3]) == [0, 1, 2] and all(t[s, 3:] == m.sink_page(0))
    s2 = m.open_slot()
    assert not m.reserve(s2, 13)                   # needs 4, only 3 free: nothing taken
    assert m.free_pages(0) == 3 and m.slot_pages(0, s2) == 0
    assert m.pages_short(s2, 13) == 1
    assert m.reserve(s2, 12)
    assert m.free_pages(0) == 0
    m.commit(s, 9)
    with pytest.raises(host.CacheError, match="without pages"):
        m.commit(s2, 13)
    m.close_slot(s)
    assert m.free_pages(0) == 0 and m.retired_pages(0) == 3
    m.flush()
    assert m.free_pages(0) == 3
    assert all(m.table(0)[s] == m.sink_page(0))
    with pytest.raises(host.CacheError, match="closed twice"):
        m.close_slot(s)
    m.check()


def test_window_group_gives_pages_back(host):
    # group 0 keeps everything, group 1 a window of 6 positions; pages of 4
    m = host.CacheManager([host.GroupConfig(4, 20), host.GroupConfig(4, 20, 6)], max_slots=2, max_positions=64)
    s = m.open_slot()
    length = 0
    for step in range(30):
        n = 1 + step % 3
        assert m.reserve(s, length + n)
        length += n
        m.commit(s, length)
        m.flush()
        m.check()
        # the next query (position `length`) sees keys from length - 5: pages before that are gone
        first_key = max(0, length - 6 + 1)
        assert m.slot_pages(1, s) == -(-length // 4) - first_key // 4
        assert m.slot_pages(0, s) == -(-length // 4)
        t = m.table(1)[s]
        assert all(t[: first_key // 4] == m.sink_page(1))
        assert all(t[first_key // 4: -(-length // 4)] != m.sink_page(1))
    assert m.held_pages(1) <= 3


@pytest.mark.parametrize("seed", range(6))
def test_fuzz_random_orders(host, seed):
    rng = random.Random(seed)
    groups = [host.GroupConfig(rng.choice([2, 4, 16]), rng.randint(8, 40), rng.choice([0, 0, 5, 17]))
              for _ in range(rng.randint(1, 3))]
    # one page size per manager, as the engine builds it
    ps = groups[0].page_size
    for g in groups:
        g.page_size = ps
    m = host.CacheManager(groups, max_slots=5, max_positions=200, shuffle_seed=seed)
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and m.n_open < 5:
            s = m.open_slot()
            assert s >= 0 and s not in live
            live[s] = 0
        elif op < 0.75 and live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 30])
            if live[s] + n > 200:
                continue
            before = [m.free_pages(g) for g in range(m.n_groups)]
            if m.reserve(s, live[s] + n):
                live[s] += n
                m.commit(s, live[s])
            else:
                assert [m.free_pages(g) for g in range(m.n_groups)] == before
        elif op < 0.9 and live:
            s = rng.choice(list(live))
            m.close_slot(s)
            del live[s]
        else:
            m.flush()
        m.check()
        for s, n in live.items():
            assert m.length(s) == n
    for s in list(live):
        m.close_slot(s)
    m.flush()
    m.check()
    for g in range(m.n_groups):
        assert m.free_pages(g) == m.group(g).n_pages and m.held_pages(g) == 0
        assert np.all(m.table(g) == m.sink_page(g))


def test_slots_are_reused_and_limited(host):
    m = host.CacheManager([host.GroupConfig(4, 4)], max_slots=2, max_positions=16)
    a, b = m.open_slot(), m.open_slot()
    assert {a, b} == {0, 1} and m.open_slot() == -1
    m.close_slot(a)
    assert m.open_slot() == a
    with pytest.raises(host.CacheError, match="exceeds"):
        m.reserve(b, 17)
    assert m.could_ever_hold(16) and not m.could_ever_hold(17)


def test_staged_decode_step_matches_the_calls_it_replaces(host):
    """stage_decode checks, reserves and lays out a step of single tokens in one call; the layout and
    the manager's state are what reserve/commit entry by entry give, and irregular input takes nothing."""
    def fresh():
        m = host.CacheManager([host.GroupConfig(4, 12)], max_slots=4, max_positions=64)
        slots = [m.open_slot() for _ in range(3)]
        for s, n in zip(slots, (3, 4, 8)):
            assert m.reserve(s, n)
            m.commit(s, n)
        return m, slots
    m, slots = fresh()
    out = np.full(64, -7, dtype=np.int32)
    rc, bad = m.stage_decode(slots, [5, 6, 7], [1, 0, 1], 100, out)
    assert (rc, bad) == (0, -1)
    n = 3
    assert out[0:n].tolist() == [5, 6, 7] and out[n:2 * n].tolist() == [3, 4, 8] and out[2 * n:3 * n].tolist() == slots
    assert out[3 * n:7 * n].reshape(4, n).tolist() == [slots, [0, 1, 2], [1, 1, 1], [4, 5, 9]]
    assert out[7 * n:7 * n + 2].tolist() == [0, 2]                      # wanted rows
    assert out[7 * n + 2:7 * n + 2 + 2 * n].tolist() == [0, 0, 1, 0, 2, 0]  # work items
    assert [m.reserved_length(s) for s in slots] == [4, 5, 9]
    m.commit_decode(slots)
    assert [m.length(s) for s in slots] == [4, 5, 9]
    m.check()
    # the same through the single calls
    m2, slots2 = fresh()
    for s in slots2:
        assert m2.reserve(s, m2.length(s) + 1)
    for s in slots2:
        m2.commit(s, m2.length(s) + 1)
    assert [m2.length(s) for s in slots2] == [4, 5, 9] and m2.free_pages(0) == m.free_pages(0)
    # irregular input: nothing is taken
    for bad_slots, toks in (([slots[0], slots[0]], [1, 1]), ([slots[0], 3], [1, 1]), ([slots[0]], [100]), ([slots[0]], [-1])):
        free = m.free_pages(0)
        rc, _ = m.stage_decode(bad_slots, toks, [1] * len(toks), 100, out)
        assert rc == 1 and m.free_pages(0) == free
    # no pages: says which request
    m3 = host.CacheManager([host.GroupConfig(4, 3)], max_slots=4, max_positions=64)
    a, b = m3.open_slot(), m3.open_slot()
    assert m3.reserve(a, 4) and m3.reserve(b, 8)
    m3.commit(a, 4); m3.commit(b, 8)
    rc, bad = m3.stage_decode([a, b], [1, 1], [1, 1], 100, out)
    assert (rc, bad) == (2, 0)


def test_pool_sized_from_free_memory():
    """The arithmetic of the automatic pool size (the reference's rule, src/serve.rs:2411-2449):
    free memory less workspace and reserve, in whole pages, one page kept for the sink, and never
    more than every slot at full context needs."""
    from axon_b200.cache.manager import POOL_RESERVE_BYTES, plan_pool_tokens
    per_token, page = 57344, 16              # the 7B shape in bfloat16
    # plenty of memory: capped by slots x context (rounded up to pages)
    assert plan_pool_tokens(160 << 30, per_token, page, 64, 4096) == 64 * 4096
    assert plan_pool_tokens(160 << 30, per_token, page, 3, 100) == 3 * 112
    # little memory: what fits, less the sink page
    free = POOL_RESERVE_BYTES + 10 * page * per_token + 5
    assert plan_pool_tokens(free, per_token, page, 64, 4096) == 9 * page
    assert plan_pool_tokens(free, per_token, page, 64, 4096, workspace_bytes=4 * page * per_token) == 5 * page
    # nothing fits: zero, which the builder turns into an error
    assert plan_pool_tokens(POOL_RESERVE_BYTES, per_token, page, 64, 4096) == 0
    assert plan_pool_tokens(0, per_token, page, 64, 4096) == 0
    # a model that keeps no keys and values needs no memory per position
    assert plan_pool_tokens(0, 0, page, 4, 64) == 4 * 64


def test_needs_by_part_name_make_groups_and_views():
    """A schedule entry may hold several cache-keeping parts (by name), parts of equal geometry
    share a group, and a part with one plane or another value width gets a group of its own."""
    import torch
    from axon_b200.cache.manager import PagedCache, bytes_per_token
    from axon_b200.parts.spec import KvNeed, StateNeed
    a, b = KvNeed(2, 16), KvNeed(2, 16, window=8)
    latent = KvNeed(1, 24, planes=1)
    wide_v = KvNeed(2, 16, v_dim=40)
    needs = [{"mixer": a}, {"attn": a, "memory": StateNeed((4,), "float32")}, {}, None, {"mixer": b},
             {"mixer": latent}, wide_v, {"x": wide_v, "y": a}]
    c = PagedCache(needs, torch.bfloat16, "cpu", page_size=16, max_tokens=64, max_slots=2, allocate=False)
    assert [len(g.members) for g in c.groups] == [3, 1, 1, 2]
    assert c.groups[0].members == [(0, "mixer"), (1, "attn"), (7, "y")]
    assert c.parts(1) == ["attn", "memory"] and c.parts(2) == [] and c.parts(6) == ["mixer"]
    assert latent.elements_per_token == 24 and wide_v.elements_per_token == 2 * (16 + 40)
    assert bytes_per_token(needs, torch.bfloat16) == 2 * (4 * 64 + 24 + 2 * 112)


def test_staged_step_of_any_shape(host):
    """stage_step lays out portions of prompts beside single tokens in one call: the layout is what
    the step function needs (tokens, positions, slots, segments, wanted rows), pages are taken
    for every entry, and irregular input takes nothing."""
    m = host.CacheManager([host.GroupConfig(4, 16)], max_slots=4, max_positions=40)
    a, b, c = (m.open_slot() for _ in range(3))
    assert m.reserve(a, 5) and m.reserve(c, 2)
    m.commit(a, 5); m.commit(c, 2)
    i32 = lambda x: np.asarray(x, dtype=np.int32)
    out = np.full(128, -7, dtype=np.int32)
    # a: one decoded token (wanted); b: a portion of 6 (places 0 and 5 wanted); c: a portion of 3 (nothing wanted)
    slots, tok_off, want_off = i32([a, b, c]), i32([0, 1, 7, 10]), i32([0, 1, 3, 3])
    tokens, wants = i32([9, 1, 2, 3, 4, 5, 6, 7, 7, 7]), i32([0, 0, 5])
    rc, bad, T, S, W, decode_only, total = m.stage_step(slots, tok_off, tokens, want_off, wants, 10, 64, out)
    assert (rc, bad, T, S, W, decode_only) == (0, -1, 10, 3, 3, 0) and total == 3 * 10 + 4 * 3 + 3
    assert out[0:T].tolist() == tokens.tolist()
    assert out[T:2 * T].tolist() == [5, 0, 1, 2, 3, 4, 5, 2, 3, 4]
    assert out[2 * T:3 * T].tolist() == [a] + [b] * 6 + [c] * 3
    assert out[3 * T:3 * T + 4 * S].reshape(4, S).tolist() == [[a, b, c], [0, 1, 7], [1, 6, 3], [6, 6, 5]]
    assert out[3 * T + 4 * S:total].tolist() == [0, 1, 6]
    assert out[total] == -7
    assert [m.reserved_length(s) for s in (a, b, c)] == [6, 6, 5] and [m.length(s) for s in (a, b, c)] == [5, 0, 2]
    m.commit_step(out[3 * T:3 * T + 4 * S], S)
    assert [m.length(s) for s in (a, b, c)] == [6, 6, 5]
    m.check()
    # single tokens only: the work items follow the wanted rows
    rc, bad, T, S, W, decode_only, total = m.stage_step(i32([c, a]), i32([0, 1, 2]), i32([3, 4]), i32([0, 0, 1]), i32([0]), 10, 64, out)
    assert (rc, T, S, W, decode_only, total) == (0, 2, 2, 1, 1, 6 + 8 + 1 + 4)
    assert out[6 + 8:6 + 8 + 1].tolist() == [1] and out[6 + 8 + 1:total].tolist() == [0, 0, 1, 0]
    m.commit_step(out[3 * T:3 * T + 4 * S], S)
    # irregular input: refused with nothing taken
    free = m.free_pages(0)
    bad_steps = [
        (i32([a, a]), i32([0, 1, 2]), i32([1, 1]), i32([0, 0, 0]), i32([])),      # a slot twice
        (i32([3]), i32([0, 1]), i32([1]), i32([0, 0]), i32([])),                   # a slot that is not open
        (i32([a]), i32([0, 1]), i32([10]), i32([0, 0]), i32([])),                  # a token outside the vocabulary
        (i32([a]), i32([0, 2]), i32([1, 1]), i32([0, 1]), i32([2])),               # a wanted place outside the entry
        (i32([a]), i32([0, 0]), i32([]), i32([0, 0]), i32([])),                    # an entry without tokens
        (i32([b]), i32([0, 35]), i32([1] * 35), i32([0, 0]), i32([])),             # past the context of 40
    ]
    for args in bad_steps:
        assert m.stage_step(*args, 10, 64, out)[0] == 1 and m.free_pages(0) == free
    assert m.stage_step(i32([b]), i32([0, 9]), i32([1] * 9), i32([0, 0]), i32([]), 10, 8, out)[0] == 1   # over the step limit
    # no pages: says which entry
    small = host.CacheManager([host.GroupConfig(4, 2)], max_slots=2, max_positions=40)
    x, y = small.open_slot(), small.open_slot()
    rc, bad, *_ = small.stage_step(i32([x, y]), i32([0, 4, 9]), i32([1] * 9), i32([0, 0, 0]), i32([]), 10, 64, out)
    assert (rc, bad) == (2, 1)
