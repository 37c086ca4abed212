"""The scheduler's decisions without a model: a toy "model" whose next token is a hash
of the request's whole history stands in for the step function (the reference tests
its generation loop the same way with ``Toy: Lm``, src/generate.rs:341-445, and its
scheduler by pure-function tests, src/serve/engine.rs:2569-3790)."""

import random

import pytest

from axon_b200.kernels import lib


@pytest.fixture(scope="module")
def host():
    return lib.host()


def toy_next(history):
    h = 17
    for t in history:
        h = (h * 31 + t + 1) % 1000003
    return h % 97


class ToyRunner:
    """Executes plans against a toy model that checks what the cache must hold."""

    def __init__(self, host, cache, sched, flat=False):
        self.host, self.cache, self.sched = host, cache, sched
        #: report the picks as an array in the plan's order (the serving loop's way) instead of a dict
        self.flat = flat
        self.fed = {}       # slot -> tokens the "cache" holds
        self.steps = 0
        self.max_tokens_seen = 0

    def run_step(self):
        plan = self.sched.plan()
        picked = {}
        slots = set()
        for e in plan.entries:
            assert e.slot not in slots, "a slot appears twice in a step"
            slots.add(e.slot)
            held = self.fed.setdefault(e.slot, [])
            if e.start == 0:
                held.clear()
            assert e.start == len(held), "a portion must continue exactly where the cache ends"
            assert self.cache.reserved_length(e.slot) >= e.start + len(e.tokens), "no pages under the tokens"
            held.extend(e.tokens)
            if e.want_logits:
                picked[e.id] = toy_next(held)
        self.max_tokens_seen = max(self.max_tokens_seen, plan.n_tokens)
        assert plan.n_tokens == sum(len(e.tokens) for e in plan.entries)
        if self.flat:
            import numpy as np
            ids, slots_a, tok_off, tokens, want_off, wants = plan.flat()
            assert ids.tolist() == [e.id for e in plan.entries] and slots_a.tolist() == [e.slot for e in plan.entries]
            assert tokens.tolist() == [t for e in plan.entries for t in e.tokens]
            assert np.diff(tok_off).tolist() == [len(e.tokens) for e in plan.entries]
            assert np.diff(want_off).tolist() == [int(e.want_logits) for e in plan.entries]
            assert wants.tolist() == [len(e.tokens) - 1 for e in plan.entries if e.want_logits]
            done = self.sched.commit_in_order(plan, np.asarray([picked[e.id] for e in plan.entries if e.want_logits], dtype=np.int32))
        else:
            done = self.sched.commit(plan, picked)
        self.cache.check()
        self.steps += 1
        return plan, done


def expected_output(prompt, max_new, stop=()):
    hist, out = list(prompt), []
    while len(out) < max_new:
        t = toy_next(hist)
        if t in stop:
            break
        out.append(t)
        hist.append(t)
    return out


def make(host, n_pages=64, page=4, slots=4, budget=32, running=4, chunk=0, positions=256):
    cache = host.CacheManager([host.GroupConfig(page, n_pages)], slots, positions)
    sched = host.Scheduler(cache, host.SchedulerConfig(budget, running, chunk))
    return cache, sched


def test_single_request_prefill_in_portions_then_decode(host):
    cache, sched = make(host, budget=8)
    prompt = list(range(1, 21))
    sched.add(1, prompt, 5)
    r = ToyRunner(host, cache, sched)
    sizes = []
    outs = {}
    while not sched.idle():
        plan, done = r.run_step()
        sizes.append([len(e.tokens) for e in plan.entries])
        for d in done:
            assert d.finish == host.Finish.Length
            outs[d.id] = sched.take_output(d.id)
    assert sizes[:3] == [[8], [8], [4]]           # the budget cuts the prompt
    assert all(s == [1] for s in sizes[3:])
    assert outs[1] == expected_output(prompt, 5)
    assert cache.n_open == 0
    cache.flush()
    assert cache.free_pages(0) == 64              # everything given back


def test_decode_rows_come_first_and_share_the_budget(host):
    cache, sched = make(host, budget=10)
    sched.add(1, [1, 2, 3], 20)
    r = ToyRunner(host, cache, sched)
    r.run_step()                                  # prompt of 1 done, it decodes now
    sched.add(2, list(range(30)), 4)
    plan, _ = r.run_step()
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(1, 1), (2, 9)]   # 1 decode + 9 of the budget
    assert plan.entries[0].want_logits and not plan.entries[1].want_logits
    assert r.max_tokens_seen <= 10


def test_stop_token_ends_without_being_emitted(host):
    cache, sched = make(host)
    prompt = [5, 6, 7]
    full = expected_output(prompt, 8)
    stop = [full[3]]
    sched.add(9, prompt, 8, stop)
    r = ToyRunner(host, cache, sched)
    fin = None
    while not sched.idle():
        _, done = r.run_step()
        for d in done:
            fin = d.finish
    assert fin == host.Finish.Stop
    assert sched.take_output(9) == expected_output(prompt, 8, stop) == full[:3]


def test_requests_that_can_never_run_are_refused(host):
    cache, sched = make(host, n_pages=4, page=4, positions=64)
    with pytest.raises(host.SchedulerError, match="pool"):
        sched.add(1, list(range(15)), 4)          # 19 positions > 16 in the pool
    with pytest.raises(host.SchedulerError, match="context"):
        sched.add(2, list(range(60)), 10)
    with pytest.raises(host.SchedulerError, match="prompt token"):
        sched.add(3, [], 4)
    sched.add(4, [1], 4)
    with pytest.raises(host.SchedulerError, match="exists"):
        sched.add(4, [1], 4)


def test_out_of_pages_preempts_the_youngest_never_the_oldest(host):
    # 10 pages of 4 = 40 positions; three requests that each grow to 24 cannot all stay
    cache, sched = make(host, n_pages=10, page=4, slots=3, budget=16, running=3, positions=64)
    prompts = {1: [1] * 6, 2: [2] * 6, 3: [3] * 6}
    for i, p in prompts.items():
        sched.add(i, p, 18)
    r = ToyRunner(host, cache, sched)
    preempted = []
    outs = {}
    guard = 0
    while not sched.idle():
        plan, done = r.run_step()
        preempted += plan.preempted
        for d in done:
            outs[d.id] = sched.take_output(d.id)
        guard += 1
        assert guard < 500, "the scheduler does not make progress"
    assert preempted, "this pool is too small for three requests: someone must have yielded"
    assert 1 not in preempted, "the oldest request never yields"
    for i, p in prompts.items():
        assert outs[i] == expected_output(p, 18), f"request {i} changed by being preempted and fed again"
    cache.flush()
    assert cache.free_pages(0) == 10


@pytest.mark.parametrize("seed", range(5))
def test_fuzz_many_requests_small_pool(host, seed):
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    cache, sched = make(host, n_pages=rng.randint(14, 30), page=page, slots=4, budget=rng.choice([6, 12, 40]),
                        running=rng.randint(2, 4), chunk=rng.choice([0, 3, 8]), positions=128)
    r = ToyRunner(host, cache, sched, flat=seed % 2 == 1)      # every other seed the serving loop's way
    want, outs = {}, {}
    next_id = 0
    for step in range(400):
        if next_id < 14 and rng.random() < 0.3:
            p = [rng.randrange(97) for _ in range(rng.randint(1, 30))]
            n = rng.randint(1, 20)
            if cache.could_ever_hold(len(p) + n):
                sched.add(next_id, p, n)
                want[next_id] = expected_output(p, n)
                next_id += 1
        if sched.idle():
            continue
        plan, done = r.run_step()
        assert plan.n_tokens <= sched.config.max_batch_tokens
        assert sched.n_running <= sched.config.max_running
        for d in done:
            outs[d.id] = sched.take_output(d.id)
    guard = 0
    while not sched.idle():
        _, done = r.run_step()
        for d in done:
            outs[d.id] = sched.take_output(d.id)
        guard += 1
        assert guard < 2000
    assert outs == want
    cache.flush()
    cache.check()
    assert cache.free_pages(0) == cache.group(0).n_pages and cache.n_open == 0


def test_abort_frees_the_slot(host):
    cache, sched = make(host)
    sched.add(1, [1, 2, 3, 4, 5], 10)
    r = ToyRunner(host, cache, sched)
    r.run_step()
    assert cache.n_open == 1
    sched.abort(1)
    assert cache.n_open == 0 and sched.idle()
    assert sched.request(1).finish == host.Finish.Aborted
