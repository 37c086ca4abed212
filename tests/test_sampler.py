"""The sampler's host half against a plain restatement in Python: the generator
(xoshiro256** seeded by splitmix64, src/sample.rs:202-242), top-p and min-p
(src/sample.rs:465-500), the temperature draw (src/sample.rs:523-556), the penalty
window (src/sample.rs:309-314) and the command-line flags (src/sample.rs:129-191)."""

import math
import random

import numpy as np
import pytest

from axon_b200.kernels import lib
from axon_b200.sampling.sampler import SampleArgs, SampleCfg, _sorted_candidates

M64 = (1 << 64) - 1


def splitmix(s):
    s = (s + 0x9E3779B97F4A7C15) & M64
    z = s
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    return s, z ^ (z >> 31)


def rotl(x, k):
    return ((x << k) | (x >> (64 - k))) & M64


class PyRng:
    def __init__(self, seed):
        self.s = []
        for _ in range(4):
            seed, v = splitmix(seed)
            self.s.append(v)

    def next(self):
        s = self.s
        r = (rotl((s[1] * 5) & M64, 7) * 9) & M64
        t = (s[1] << 17) & M64
        s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]
        s[2] ^= t
        s[3] = rotl(s[3], 45)
        return r

    def uniform(self):
        return (self.next() >> 11) * (1.0 / (1 << 53))


@pytest.fixture(scope="module")
def host():
    return lib.host()


@pytest.mark.parametrize("seed", [0, 1, 42, 2**63 + 5])
def test_generator(host, seed):
    a, b = host.Rng(seed), PyRng(seed)
    assert list(a.state()) == b.s
    for _ in range(50):
        assert a.next_u64() == b.next()
    u = [a.uniform() for _ in range(1000)]
    assert all(0.0 <= x < 1.0 for x in u) and 0.4 < sum(u) / len(u) < 0.6


def py_kept(cfg, logits):
    n = 0
    while n < len(logits) and not math.isnan(logits[n]):
        n += 1
    l0 = float(logits[0])
    if n <= 1 or not math.isfinite(l0):
        return 1
    if cfg.top_p < 1.0:
        e = [math.exp(float(l) - l0) for l in logits[:n]]
        z = sum(e)
        cum, keep = 0.0, n
        for i, x in enumerate(e):
            cum += x / z
            if cum >= np.float64(np.float32(cfg.top_p)):
                keep = i + 1
                break
        n = keep
    if cfg.min_p > 0.0:
        lo = l0 + math.log(np.float64(np.float32(cfg.min_p)))
        k = 0
        while k < n and float(logits[k]) >= lo:
            k += 1
        n = max(k, 1)
    return n


def py_pick(cfg, logits, ids, u):
    n = py_kept(cfg, logits)
    if n == 1:
        return ids[0]
    l0, t = float(logits[0]), float(np.float32(cfg.temp))
    w = [math.exp((float(l) - l0) / t) for l in logits[:n]]
    z = sum(w)
    target = min(u * z, np.nextafter(z, 0.0))
    cum, last = 0.0, 0
    for i, x in enumerate(w):
        if x > 0:
            last = i
        cum += x
        if target < cum:
            return ids[i]
    return ids[last]


def test_kept_and_pick_against_python(host):
    rng = random.Random(3)
    for trial in range(300):
        k = rng.randint(1, 60)
        logits = np.sort(np.array([rng.gauss(0, 3) for _ in range(k)], dtype=np.float32))[::-1].copy()
        if trial % 17 == 0 and k > 2:
            logits[-1] = np.nan
        ids = np.array(rng.sample(range(1000), k), dtype=np.int32)
        cfg = SampleCfg(temp=rng.choice([0.3, 0.8, 1.5]), top_k=k, top_p=rng.choice([0.5, 0.9, 1.0]),
                        min_p=rng.choice([0.0, 0.05, 0.3]))
        hc = cfg.to_host()
        assert host.kept(hc, logits) == py_kept(cfg, logits)
        u = rng.random()
        assert host.pick_at(hc, logits, ids, u) == py_pick(cfg, logits, ids, u)
    # one candidate, or an infinite best logit: the first candidate
    hc = SampleCfg().to_host()
    assert host.pick_at(hc, np.array([np.inf, 1.0], dtype=np.float32), np.array([7, 8], dtype=np.int32), 0.99) == 7


def test_draw_follows_the_distribution(host):
    cfg = SampleCfg(temp=1.0, top_k=4, top_p=1.0, min_p=0.0, seed=9)
    s = host.Sampler(cfg.to_host())
    logits = np.log(np.array([0.5, 0.25, 0.15, 0.10], dtype=np.float32))
    ids = np.array([10, 11, 12, 13], dtype=np.int32)
    counts = {i: 0 for i in ids.tolist()}
    for _ in range(20000):
        counts[s.pick(logits, ids)] += 1
    for i, p in zip(ids.tolist(), [0.5, 0.25, 0.15, 0.10]):
        assert abs(counts[i] / 20000 - p) < 0.015


def test_penalty_window(host):
    assert host.penalty_ids([5, 1, 5, 9, 1, 3], 4) == [1, 3, 5, 9]
    assert host.penalty_ids([5, 1, 5, 9, 1, 3], 2) == [1, 3]
    assert host.penalty_ids([5, 1], 64) == [1, 5]
    assert host.penalty_ids([], 64) == []


def test_sorted_candidates_order():
    row = np.array([1.0, 3.0, np.nan, 3.0, -2.0], dtype=np.float32)
    assert _sorted_candidates(row).tolist() == [3, 1, 0, 4, 2]   # ties to the larger id, NaN last


def test_flags():
    a = SampleArgs()
    assert a.resolve(0.0) is None                      # gen: greedy without --temp
    c = a.resolve(0.8)
    assert (c.temp, c.top_k, c.top_p, c.min_p, c.repeat_penalty, c.repeat_last_n) == (0.8, 40, 0.9, 0.0, 1.1, 64)
    a.set("--temp", "0.5"); a.set("--top-k", "0"); a.set("--seed", "77"); a.set("--repeat-penalty", "1")
    c = a.resolve(0.0)
    assert (c.temp, c.top_k, c.seed, c.repeat_penalty) == (0.5, 0, 77, 1.0)
    assert a.any_besides_temp()
    for flag, bad, msg in [("--temp", "101", "from 0 to 100"), ("--top-p", "1.5", "from 0 to 1"),
                           ("--top-k", "-1", "whole number"), ("--repeat-penalty", "0", "above 0"),
                           ("--seed", "x", "whole number"), ("--min-p", None, "needs a value")]:
        with pytest.raises(ValueError, match=msg):
            SampleArgs().set(flag, bad)
    assert SampleArgs.is_flag("--min-p") and not SampleArgs.is_flag("--ctx")
