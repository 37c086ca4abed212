"""The plain implementation checked against itself: causality, a second statement of
attention with an explicit loop, and mutation checks: a wrong variant of each formula
must move the logits far beyond the tolerances the engine tests use
(the reference's guard rail: src/model.rs:4866-4924)."""

import math

import pytest
import torch

import plain_qwen2 as plain
from conftest import TINY


@pytest.fixture(scope="module")
def models(model_folders):
    return {k: plain.read_model(v) for k, v in model_folders.items()}


def _tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()


@pytest.mark.parametrize("name", ["A", "B"])
def test_causal_prefix_property(models, name):
    cfg, w = models[name]
    ids = _tokens(cfg, 23, 5)
    full = plain.forward(cfg, w, ids)
    part = plain.forward(cfg, w, ids[:9])
    assert torch.allclose(full[:9], part, rtol=0, atol=1e-12)


def test_attention_against_an_explicit_loop():
    torch.manual_seed(0)
    T, H, Hkv, hd = 7, 6, 2, 8
    q, k, v = (torch.randn(T, n, hd, dtype=torch.float64) for n in (H, Hkv, Hkv))
    got = plain.causal_gqa_attention(q, k, v, window=3)
    for t in range(T):
        for h in range(H):
            kh = h // (H // Hkv)
            lo = max(0, t - 3 + 1)
            s = [float(q[t, h] @ k[j, kh]) / math.sqrt(hd) for j in range(lo, t + 1)]
            m = max(s)
            e = [math.exp(x - m) for x in s]
            z = sum(e)
            o = sum((ei / z) * v[lo + j, kh] for j, ei in enumerate(e))
            assert torch.allclose(got[t, h], o, atol=1e-12)


def test_rope_is_a_rotation_by_position_difference():
    torch.manual_seed(1)
    hd = 16
    q, k = torch.randn(1, 1, hd, dtype=torch.float64), torch.randn(1, 1, hd, dtype=torch.float64)
    d1 = (plain.rope_half(q, [10], 1e4) * plain.rope_half(k, [4], 1e4)).sum()
    d2 = (plain.rope_half(q, [106], 1e4) * plain.rope_half(k, [100], 1e4)).sum()
    assert abs(float(d1 - d2)) < 1e-9
    assert torch.allclose(plain.rope_half(q, [0], 1e4), q)


def _mutants(cfg, w):
    """Wrong variants of the formulas, each as (name, logits function)."""
    ids = _tokens(cfg, 40, 9)

    def no_bias():
        w2 = {k: (torch.zeros_like(v) if k.endswith("proj.bias") else v) for k, v in w.items()}
        return plain.forward(cfg, w2, ids)

    def wrong_eps():
        return plain.forward(dict(cfg, rms_norm_eps=1e-2), w, ids)

    def adjacent_pairs():
        orig = plain.rope_half

        def adj(v, positions, theta):
            hd = v.shape[-1]
            perm = torch.cat([torch.arange(0, hd, 2), torch.arange(1, hd, 2)])
            inv = torch.argsort(perm)
            return orig(v[..., perm], positions, theta)[..., inv]
        plain.rope_half = adj
        try:
            return plain.forward(cfg, w, ids)
        finally:
            plain.rope_half = orig

    def wrong_gqa():
        orig = plain.causal_gqa_attention

        def bad(q, k, v, window=None, scale=None):
            H, Hkv = q.shape[1], k.shape[1]
            # head h reads kv head h % Hkv instead of h // group
            idx = torch.tensor([(h % Hkv) for h in range(H)])
            return orig(q, k[:, idx], v[:, idx], window, scale)
        plain.causal_gqa_attention = bad
        try:
            return plain.forward(cfg, w, ids)
        finally:
            plain.causal_gqa_attention = orig

    def wrong_theta():
        return plain.forward(dict(cfg, rope_theta=cfg["rope_theta"] * 10), w, ids)

    good = plain.forward(cfg, w, ids)
    return good, {"no_bias": no_bias, "wrong_eps": wrong_eps, "adjacent_pairs": adjacent_pairs,
                  "wrong_gqa": wrong_gqa, "wrong_theta": wrong_theta}


def test_mutations_move_the_logits(models):
    # tiny-A has 2 kv heads with groups of 2, so a wrong head mapping shows
    cfg, w = models["A"]
    good, mutants = _mutants(cfg, w)
    scale = float(good.abs().max())
    for name, fn in mutants.items():
        diff = float((fn() - good).abs().max())
        print(name, diff / scale)
        # the engine's 32-bit tests hold 2e-5 of the logit scale; a wrong formula is far outside
        assert diff > 100 * 2e-5 * scale, f"mutant {name} moved logits by only {diff}"


def test_greedy_takes_the_last_of_equal_maxima(models):
    """A tie is built: two rows of the (untied) head are made equal and their gain so large that
    they are the two largest logits at every place; the larger id must be picked
    (src/generate.rs:222-263)."""
    cfg, w = models["B"]
    w = dict(w)
    head = w["lm_head.weight"].clone()
    lo, hi = 17, 301
    ids = [1, 2, 3]
    # the planted rows are multiples of the normed state that reaches the head at the last place,
    # which a first run records
    state = {}
    orig = plain.linear

    def spy(x, wt, b=None):
        if wt is head_now[0]:
            state["h"] = x.clone()
        return orig(x, wt, b)
    head_now = [head]
    plain.linear = spy
    try:
        w["lm_head.weight"] = head
        plain.forward(cfg, w, ids)
    finally:
        plain.linear = orig
    h = state["h"][-1]
    head[lo] = head[hi] = 50.0 * h / (h @ h)           # both logits exactly 50 at the last place
    w["lm_head.weight"] = head
    row = plain.forward(cfg, w, ids)[-1]
    assert row[lo] == row[hi] == row.max(), "the two planted rows must tie for the maximum"
    assert plain.greedy(cfg, w, ids, 1) == [hi]
    # and with the rows swapped in value the smaller id still loses: the rule is "last index"
    head[hi] = head[hi] * 0.5
    w["lm_head.weight"] = head
    assert plain.greedy(cfg, w, ids, 1) == [lo]


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_two_plain_implementations_agree(model_folders, models, name):
    """The torch implementation (whole sequences, masked matrices) and the numpy one (token by
    token, explicit loops, its own file reader) were written separately from the same formulas;
    they must agree to rounding of float64."""
    import numpy as np
    import plain_loops
    cfg, w = models[name]
    cfg2, w2 = plain_loops.read_folder(model_folders[name])
    assert cfg2 == cfg
    for k, v in w.items():
        assert np.array_equal(v.numpy(), w2[k]), f"the two readers differ on {k}"
    ids = _tokens(cfg, 19, 77)
    a = plain.forward(cfg, w, ids).numpy()
    b = plain_loops.forward(cfg2, w2, ids)
    assert a.shape == b.shape
    assert float(np.abs(a - b).max()) <= 1e-10 * max(1.0, float(np.abs(a).max()))
