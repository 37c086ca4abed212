"""The engine against the plain implementation, in 32-bit and in bfloat16, under every
way of cutting the work: whole prompts, the last 32 tokens one by one, portions of
changing size down to two tokens, and mixed batches with so few pages that they are
used again (the reference's batching tests: src/cuda/qwen2/tests.rs:4199-4311,
src/cuda/qwen2/slots.rs:1622-1796)."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from conftest import ROOT, TINY

pytestmark = pytest.mark.gpu

# Largest allowed |engine - plain| as a fraction of the largest |logit| of the request.
# 32-bit: float rounding through a few layers.  bfloat16: activations are rounded to 8
# bits of mantissa between kernels.  The mutation checks in test_plain.py show that a
# wrong formula moves logits by 1e-1 of the scale or more.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}

PROMPT_LENGTHS = {"A": [5, 17, 31, 70], "B": [1, 9, 40, 77], "C": [3, 33, 90, 130], "D": [2, 21, 66, 101]}


def tokens_for(name, i, n):
    g = torch.Generator().manual_seed(1000 * (ord(name) - 64) + i)
    return torch.randint(0, TINY[name]["vocab_size"], (n,), generator=g).tolist()


@pytest.fixture(scope="module")
def plain_models(model_folders):
    return {k: plain.read_model(v) for k, v in model_folders.items()}


@pytest.fixture(scope="module")
def expected(plain_models):
    """(name, i) -> float64 logits [T, V] of request i of configuration name."""
    cache = {}

    def get(name, i, n=None):
        n = n or PROMPT_LENGTHS[name][i]
        key = (name, i, n)
        if key not in cache:
            cfg, w = plain_models[name]
            cache[key] = plain.forward(cfg, w, tokens_for(name, i, n))
        return cache[key]
    return get


def build(folder, dtype, **kw):
    from axon_b200.engine.build import build_engine
    kw.setdefault("max_slots", 8)
    return build_engine(folder, dtype=dtype, **kw)


def replay(engine, steps):
    from axon_b200.engine.replay import Replayer
    r = Replayer(engine)
    out = {}
    for step, logits in r.run(steps):
        if logits is not None:
            out[step] = logits.double().cpu()
    return out


def check_rows(got, want_rows, tol, what):
    """got [n, V] vs the plain rows; error relative to the largest logit."""
    want = torch.stack(want_rows)
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    assert got.shape == want.shape, what
    assert err <= tol * scale, f"{what}: error {err:.3e} is {err / scale:.2e} of the scale (limit {tol:.0e})"


def run_and_check(engine, steps, wanted, expected_of, tol, what):
    """``wanted[step]`` lists (request key, position) in the order the step wants them."""
    got = replay(engine, steps)
    assert set(got) == set(wanted), what
    for step, pairs in wanted.items():
        rows = [expected_of(*key)[pos] for key, pos in pairs]
        check_rows(got[step], rows, tol, f"{what}, step {step}")


class Trace:
    """Builds trace steps and remembers which (request, position) each wanted row is."""

    def __init__(self):
        self.steps, self.wanted, self.pos = [], {}, {}

    def step(self, entries, end=()):
        k = len(self.steps)
        rec = {"step": k, "entries": [], "end": list(end)}
        pairs = []
        for rid, key, toks, want in entries:
            start = self.pos.get(rid, 0)
            rec["entries"].append({"id": rid, "tokens": list(toks), "want": list(want)})
            pairs += [(key, start + w) for w in want]
            self.pos[rid] = start + len(toks)
        for rid in end:
            self.pos.pop(rid, None)
        self.steps.append(rec)
        if pairs:
            self.wanted[k] = pairs
        return k


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_each_request_alone_and_whole(model_folders, expected, name, dtype):
    engine = build(model_folders[name], dtype, max_tokens=256)
    for i, n in enumerate(PROMPT_LENGTHS[name]):
        toks = tokens_for(name, i, n)
        tr = Trace()
        tr.step([("r", (name, i), toks, range(n))], end=["r"])
        run_and_check(engine, tr.steps, tr.wanted, expected, TOL[dtype], f"{name}/{dtype} request {i} whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_last_32_tokens_one_by_one(model_folders, expected, name, dtype):
    engine = build(model_folders[name], dtype, max_tokens=256)
    for i in (2, 3):
        n = PROMPT_LENGTHS[name][i]
        toks = tokens_for(name, i, n)
        head = max(n - 32, 0)
        tr = Trace()
        if head:
            tr.step([("r", (name, i), toks[:head], [head - 1])])
        for t in range(head, n):
            tr.step([("r", (name, i), [toks[t]], [0])], end=["r"] if t == n - 1 else [])
        run_and_check(engine, tr.steps, tr.wanted, expected, TOL[dtype], f"{name}/{dtype} request {i} decoded tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("sizes", [[5, 30, 3, 17, 2, 1, 33], [24, 32, 31, 2, 47], [2, 2, 2, 16, 1, 64], [16, 16, 16, 16]])
def test_portions_of_changing_size(model_folders, expected, name, dtype, sizes):
    engine = build(model_folders[name], dtype, max_tokens=256, page_size=16)
    i = 3
    n = PROMPT_LENGTHS[name][i]
    toks = tokens_for(name, i, n)
    tr, at, k = Trace(), 0, 0
    while at < n:
        size = min(sizes[k % len(sizes)], n - at)
        k += 1
        # ask for the first and the last place of every portion
        want = sorted({0, size - 1})
        tr.step([("r", (name, i), toks[at:at + size], want)], end=["r"] if at + size == n else [])
        at += size
    run_and_check(engine, tr.steps, tr.wanted, expected, TOL[dtype], f"{name}/{dtype} portions {sizes}")


def mixed_trace(name):
    """Four requests of different lengths: they join at different steps, prompts are fed
    in portions beside single decoded tokens of others, one is left out of some steps,
    they end at different steps and a fifth request then takes the pages that came free."""
    L = PROMPT_LENGTHS[name]
    lens = {"a": L[3], "b": L[2], "c": L[1] + 20, "d": L[0] + 37, "e": 50}
    keys = {"a": (name, 3, lens["a"]), "b": (name, 2, lens["b"]), "c": (name, 1, lens["c"]),
            "d": (name, 0, lens["d"]), "e": (name, 2, lens["e"])}
    toks = {r: tokens_for(name, keys[r][1], lens[r]) for r in lens}
    fed = {r: 0 for r in lens}
    tr = Trace()

    def take(r, k, want_last=True):
        k = min(k, lens[r] - fed[r])
        if k <= 0:
            return None
        part = toks[r][fed[r]:fed[r] + k]
        fed[r] += k
        return (r, keys[r], part, [k - 1] if want_last else [])

    plan = [
        [("a", 13)],
        [("a", 2), ("b", 9)],
        [("a", 1), ("b", 1), ("c", 7)],
        [("a", 1), ("b", 17), ("c", 1), ("d", 3)],
        [("a", 30), ("c", 1), ("d", 1)],            # b is left out
        [("a", 1), ("b", 2), ("c", 5), ("d", 1)],
    ]
    for row in plan:
        ents = [e for e in (take(r, k) for r, k in row) if e]
        tr.step(ents)
    # then everyone decodes one token a step until done; finished ones end, and "e" joins
    # once two of the first four are through, taking pages that came free
    joined_e = False
    while any(fed[r] < lens[r] for r in lens):
        live = [r for r in ("a", "b", "c", "d") if fed[r] < lens[r]]
        if len(live) <= 2:
            joined_e = True
        ents = [take(r, 1) for r in live]
        if joined_e and fed["e"] < lens["e"]:
            ents.append(take("e", 11 if fed["e"] < 33 else 1))
        ending = [e[0] for e in ents if fed[e[0]] == lens[e[0]]]
        tr.step(ents, end=ending)
    return tr, keys


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("shuffle", [0, 11])
def test_mixed_batches_with_pages_used_again(model_folders, plain_models, name, dtype, shuffle):
    tr, keys = mixed_trace(name)
    # the pool holds just what is live at the worst moment, so pages must be used again
    live, worst = {}, 0
    for rec in tr.steps:
        for e in rec["entries"]:
            live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-v // 16) * 16 for v in live.values()))
        for rid in rec["end"]:
            live.pop(rid)
    total = sum(-(-k[2] // 16) * 16 for k in keys.values())
    assert worst < total, "the trace must need fewer pages than all requests together"
    engine = build(model_folders[name], dtype, max_tokens=worst, page_size=16, shuffle_seed=shuffle)
    cfg, w = plain_models[name]
    full = {}

    def expected_of(nm, i, n):
        if (nm, i, n) not in full:
            full[(nm, i, n)] = plain.forward(cfg, w, tokens_for(nm, i, n))
        return full[(nm, i, n)]
    run_and_check(engine, tr.steps, tr.wanted, expected_of, TOL[dtype], f"{name}/{dtype} mixed, shuffle {shuffle}")
    engine.cache.manager.check()
    engine.cache.flush()
    assert engine.cache.manager.free_pages(0) == engine.cache.n_pages, "pages were lost"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n", [("A", 128), ("B", 200)])
def test_long_decoding(model_folders, plain_models, name, dtype, n):
    engine = build(model_folders[name], dtype, max_tokens=256, page_size=16)
    cfg, w = plain_models[name]
    toks = tokens_for(name, 7, n)
    want = plain.forward(cfg, w, toks)
    tr = Trace()
    for t in range(n):
        tr.step([("r", ("x",), [toks[t]], [0])])
    got = replay(engine, tr.steps)
    rows = torch.cat([got[t] for t in range(n)])
    check_rows(rows, list(want), TOL[dtype], f"{name}/{dtype} {n} tokens one by one")


@pytest.mark.parametrize("name,dtype", [("C", "bfloat16"), ("C", "float32"), ("B", "bfloat16"), ("D", "bfloat16")])
def test_pages_far_apart_in_a_pool_beyond_four_gib(model_folders, plain_models, name, dtype):
    """A pool of 2**32 elements (8 or 16 GiB) with pages handed out in shuffled
    order: a request's pages lie gigabytes apart, so every paged kernel's offsets (prompt and
    decode attention, the cache writes) have to be 64-bit.  A prompt whole, then tokens one by one."""
    cfg = TINY[name]
    per_token = cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * cfg["head_dim"]
    pool_tokens = -(-(2**32) // per_token // 16) * 16            # half of the pages lie beyond 2**31 elements
    engine = build(model_folders[name], dtype, max_tokens=pool_tokens, page_size=16, shuffle_seed=11)
    assert engine.cache.groups[0].pool.numel() > 2**31
    n_prompt, n_dec = PROMPT_LENGTHS[name][3], 24
    toks = tokens_for(name, 9, n_prompt + n_dec)
    cfg_w = plain_models[name]
    want = plain.forward(cfg_w[0], cfg_w[1], toks)
    tr = Trace()
    tr.step([("r", ("x",), toks[:n_prompt], range(n_prompt))])
    for t in range(n_prompt, n_prompt + n_dec):
        tr.step([("r", ("x",), [toks[t]], [0])])
    got = replay(engine, tr.steps)
    table = engine.cache.manager.table(0)[0]
    used = [int(p) for p in table[: -(-(n_prompt + n_dec) // 16)]]
    assert max(used) * 16 * per_token > 2**31, "the shuffle left this request's pages in the first gigabytes"
    rows = torch.cat([got[k] for k in range(len(tr.steps))])
    check_rows(rows, list(want), TOL[dtype], f"{name}/{dtype} in a pool of {pool_tokens} positions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(model_folders, plain_models, name, dtype):
    engine = build(model_folders[name], dtype, max_tokens=128)
    cfg, w = plain_models[name]
    for n in (1, 2, 3):
        toks = tokens_for(name, 20 + n, n)
        want = plain.forward(cfg, w, toks)
        tr = Trace()
        tr.step([("r", ("x",), toks, range(n))], end=["r"])
        check_rows(replay(engine, tr.steps)[0], list(want), TOL[dtype], f"{name}/{dtype} first {n} tokens")


def test_a_far_key_among_hundreds(tmp_path):
    """One key far back gets a large score for the last query of a long sequence: if a
    page, a position or a split is wrong anywhere along the way, the output changes by
    far more than rounding."""
    from conftest import make_model_folder
    cfg = dict(TINY["C"], num_hidden_layers=1, max_position_embeddings=1024)
    folder = make_model_folder(str(tmp_path / "far"), cfg, 77, sharpen=1.0)
    pcfg, w = plain.read_model(folder)
    n = 700
    toks = tokens_for("C", 50, n)
    # token `needle` appears once, at position 37; the last token is `probe`; make probe's
    # query and needle's key line up by planting large values in their embedding rows
    needle, probe = 998, 999
    toks = [t % 990 for t in toks]
    toks[37], toks[-1] = needle, probe
    from safetensors.torch import load_file
    from axon_b200.weights import write_safetensors
    t = load_file(os.path.join(folder, "model.safetensors"))
    e = t["model.embed_tokens.weight"].float()
    e[needle] = 0
    e[probe] = 0
    e[needle, 3] = 4.0
    e[probe, 3] = 4.0
    t["model.embed_tokens.weight"] = e.to(torch.bfloat16)
    for k in ("q_proj", "k_proj"):
        t[f"model.layers.0.self_attn.{k}.weight"] = (t[f"model.layers.0.self_attn.{k}.weight"].float() * 12).to(torch.bfloat16)
    write_safetensors(os.path.join(folder, "model.safetensors"), t)
    pcfg, w = plain.read_model(folder)
    want = plain.forward(pcfg, w, toks)
    for dtype in ("float32", "bfloat16"):
        engine = build(folder, dtype, max_tokens=1024, page_size=16, max_positions=1024)
        tr = Trace()
        tr.step([("r", ("x",), toks[:-1], [])])
        tr.step([("r", ("x",), toks[-1:], [0])], end=["r"])
        got = replay(engine, tr.steps)[1]
        check_rows(got, [want[-1]], TOL[dtype], f"far key, {dtype}, decode")
        tr = Trace()
        tr.step([("r", ("x",), toks, [n - 1, 37, 38])], end=["r"])
        got = replay(engine, tr.steps)[0]
        check_rows(got, [want[-1], want[37], want[38]], TOL[dtype], f"far key, {dtype}, whole")


def test_layer_sizes_of_the_large_model(tmp_path):
    """One layer at the widths of the 7B configuration (hidden 3584, 28 heads over 4 kv
    heads of 128, feed-forward 18944; the vocabulary is cut to 32003 so that the plain
    float64 model fits in host memory): sizes at which the tuned kernels take their
    multi-tile, split-K and multi-wave paths.  Whole, in portions, and decoded."""
    from conftest import make_model_folder
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 1,
           "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128,
           "intermediate_size": 18944, "vocab_size": 32003, "rope_theta": 1e6, "rms_norm_eps": 1e-6,
           "tie_word_embeddings": False, "max_position_embeddings": 512}
    folder = make_model_folder(str(tmp_path / "wide"), cfg, 99, sharpen=4.0)
    pcfg, w = plain.read_model(folder)
    g = torch.Generator().manual_seed(5)
    n = 150
    toks = torch.randint(0, 32003, (n,), generator=g).tolist()
    want = plain.forward(pcfg, w, toks)
    del w
    for dtype in ("float32", "bfloat16"):
        engine = build(folder, dtype, max_tokens=512, page_size=16, max_positions=512, max_slots=2)
        tr = Trace()
        tr.step([("r", ("x",), toks, [0, 1, 63, 64, 127, 128, n - 1])], end=["r"])
        got = replay(engine, tr.steps)[0]
        check_rows(got, [want[i] for i in (0, 1, 63, 64, 127, 128, n - 1)], TOL[dtype], f"7B widths, {dtype}, whole")
        tr, at = Trace(), 0
        rows, pos = [], []
        for size in (70, 2, 65, 1, 1, 1, 8, 1, 1):
            tr.step([("r", ("x",), toks[at:at + size], [size - 1])], end=["r"] if at + size == n else [])
            at += size
            pos.append(at - 1)
        assert at == n
        got = replay(engine, tr.steps)
        check_rows(torch.cat([got[k] for k in sorted(got)]), [want[p] for p in pos], TOL[dtype],
                   f"7B widths, {dtype}, portions and decoded tokens")
        del engine
        torch.cuda.empty_cache()


def test_step_refusals(model_folders):
    from axon_b200.engine.step import OutOfPages, StepEntry, StepError
    engine = build(model_folders["A"], "float32", max_tokens=32, page_size=16, max_slots=2)
    s = engine.open_request()
    with pytest.raises(StepError, match="vocabulary"):
        engine.step([StepEntry(s, [256], [0])])
    with pytest.raises(StepError, match="not open"):
        engine.step([StepEntry(5, [1], [0])])
    with pytest.raises(StepError, match="wanted place"):
        engine.step([StepEntry(s, [1, 2], [2])])
    with pytest.raises(StepError, match="twice"):
        engine.step([StepEntry(s, [1], []), StepEntry(s, [2], [])])
    assert engine.step([StepEntry(s, list(range(20)), [19])]).shape == (1, 256)
    s2 = engine.open_request()
    with pytest.raises(OutOfPages):
        engine.step([StepEntry(s2, [1], [0])])     # both pages are taken
    engine.close_request(s)
    assert engine.step([StepEntry(s2, [1], [0])]).shape == (1, 256)
    with pytest.raises(StepError, match="slots are taken"):
        engine.open_request(), engine.open_request()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_pick_inside_the_step(model_folders, dtype):
    """``step(..., greedy=True)`` returns the ids that the argmax of the same step's logits gives,
    for prompt portions (eager) and for steps of single tokens (the captured graph, replayed)."""
    from axon_b200.engine.step import StepEntry
    engine = build(model_folders["B"], dtype, max_tokens=512, page_size=16, max_slots=4)
    a, b = engine.open_request(), engine.open_request()
    prompt = tokens_for("B", 0, 21)
    want = engine.step([StepEntry(a, prompt, [3, 20])]).argmax(dim=1).tolist()
    got = engine.step([StepEntry(b, prompt, [3, 20])], greedy=True)
    assert got.dtype == torch.int32 and got.tolist() == want
    ta = tb = want[1]
    for _ in range(6):        # the first such step captures the graph, the others replay it
        ta = engine.step([StepEntry(a, [ta], [0])]).argmax(dim=1).tolist()[0]
        tb = engine.step([StepEntry(b, [tb], [0])], greedy=True).tolist()[0]
        assert ta == tb
    both = engine.step([StepEntry(a, [ta], [0]), StepEntry(b, [tb], [])], greedy=True)
    assert both.shape == (1,)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_folders, plain_models, tmp_path, dtype):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 files and `done` lines out."""
    name = "B"
    cfg, w = plain_models[name]
    toks = tokens_for(name, 3, 77)
    want = plain.forward(cfg, w, toks)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": toks[:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": toks[40:75], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": toks[75:76], "want": [0]},
                                {"id": "b", "tokens": toks[:5], "want": [4]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": toks[76:77], "want": [0]}], "end": ["a"]},
    ]
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", model_folders[name], "--dtype", dtype,
                        "--out", str(out), "--max-tokens", "192"],
                       input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    assert not (out / "1.f32").exists()
    V = cfg["vocab_size"]
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)).double()
    check_rows(got0, [want[0], want[39]], TOL[dtype], "trace_run step 0")
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V)).double()
    check_rows(got2, [want[75], want[4]], TOL[dtype], "trace_run step 2")
    got3 = torch.from_numpy(np.fromfile(out / "3.f32", dtype="<f4").reshape(-1, V)).double()
    check_rows(got3, [want[76]], TOL[dtype], "trace_run step 3")


# ---------------------------------------------------------------------------
# The schedule that serving and the bench run: many live requests decoding one token a
# step through replayed CUDA graphs, key splits that change as contexts grow and as
# requests leave and join, shuffled pages that are used again.

LONG = {
    # head size 128 (the tcgen05 prompt kernel, the fused decode kernel), 2 kv heads
    "C": dict(TINY["C"], max_position_embeddings=1536),
    # head size 32, one kv head
    "B": dict(TINY["B"], max_position_embeddings=1536),
}


@pytest.fixture(scope="module")
def long_folders(tmp_path_factory):
    from conftest import make_model_folder
    return {k: make_model_folder(str(tmp_path_factory.mktemp(f"long_{k}")), cfg, 4321 + i)
            for i, (k, cfg) in enumerate(LONG.items())}


def _long_tokens(name, i, n):
    g = torch.Generator().manual_seed(50_000 + 1000 * (ord(name) - 64) + i)
    return torch.randint(0, LONG[name]["vocab_size"], (n,), generator=g).tolist()


def _many_requests_schedule(name, n_first=24, n_late=4, decode_steps=80):
    """(requests, tokens): request r = (prompt length, first decode step, last decode step).
    The first 24 hold contexts spread over 300..1200 when decoding starts; the six longest end one
    after the other from step 17, six more at step 38 and four at step 52, and four others join
    from step 44 on the pages that came free: the number of live requests and the longest context
    both change, and with them the number of key splits."""
    reqs = {}
    for r in range(n_first):
        ctx = 300 + (r * 900) // (n_first - 1)
        last = decode_steps - 1
        if r >= n_first - 6:
            last = 17 + 2 * (n_first - 1 - r)
        elif r % 3 == 0:
            last = 38
        elif r % 3 == 1 and r < 12:
            last = 52
        reqs[r] = (ctx, 0, last)
    for j in range(n_late):
        reqs[n_first + j] = (350 + 130 * j, 44 + 8 * j, decode_steps - 1)
    toks = {r: _long_tokens(name, r, ctx + (last - first + 1)) for r, (ctx, first, last) in reqs.items()}
    return reqs, toks


def _run_many(engine, name, reqs, toks, decode_steps, greedy):
    """Feed prompts (whole, no logits wanted), then one token per live request per step.
    Returns {(request, position): row or pick} and the split counts the decode steps used."""
    from axon_b200.engine.step import StepEntry
    from axon_b200.kernels import fast
    slots, out, splits_seen, replays = {}, {}, [], 0
    kv_heads = LONG[name]["num_key_value_heads"]
    for t in range(decode_steps):
        for r, (ctx, first, last) in reqs.items():
            if first == t:
                slots[r] = engine.open_request()
                engine.step([StepEntry(slots[r], toks[r][:ctx], [])])
        live = [r for r, (ctx, first, last) in reqs.items() if first <= t <= last]
        entries, where = [], []
        for r in live:
            ctx, first, _ = reqs[r]
            pos = ctx + (t - first)
            entries.append(StepEntry(slots[r], [toks[r][pos]], [0]))
            where.append((r, pos))
        if engine.rt.dtype == torch.bfloat16:
            splits_seen.append(fast.decode_split_count(len(live), kv_heads, max(p for _, p in where) + 1))
        before = len(engine._graphs)
        res = engine.step(entries, greedy=greedy)
        replays += len(engine._graphs) == before
        res = res.cpu()
        for k, key in enumerate(where):
            out[key] = int(res[k]) if greedy else res[k].double()
        for r in live:
            if reqs[r][2] == t:
                engine.close_request(slots.pop(r))
    return out, splits_seen, replays


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "B"])
def test_many_requests_decoding_through_replayed_graphs(long_folders, name, dtype):
    """24 live requests at contexts of 300 to 1,200 decode 80 tokens, each step's logits against
    the plain implementation; requests leave and others join on their (shuffled) pages; in
    bfloat16 the steps are replayed CUDA graphs whose key-split count changes several times."""
    steps = 80
    reqs, toks = _many_requests_schedule(name)
    cfg, w = plain.read_model(long_folders[name])
    # the pool holds what is live at the worst moment, so the late requests reuse freed pages
    worst = 0
    for t in range(steps):
        live = sum(-(-(ctx + (min(t, last) - first + 1)) // 16) * 16 for ctx, first, last in reqs.values() if first <= t <= last)
        worst = max(worst, live)
    total = sum(-(-len(v) // 16) * 16 for v in toks.values())
    assert worst < total
    logits = None
    for greedy in (False, True):
        engine = build(long_folders[name], dtype, max_tokens=worst, page_size=16, max_slots=32, max_positions=1536,
                       shuffle_seed=5, max_step_tokens=2048)
        got, splits_seen, replays = _run_many(engine, name, reqs, toks, steps, greedy)
        if dtype == "bfloat16":
            assert len(set(splits_seen)) >= 3 and max(splits_seen) > 1, f"split counts {sorted(set(splits_seen))}"
            assert engine.cuda_graphs and replays >= steps // 2, f"{replays} of {steps} steps replayed a graph"
        if not greedy:
            logits = got
            want = {r: plain.forward(cfg, w, toks[r]) for r in reqs}
            worst_err = 0.0
            for (r, pos), row in got.items():
                ref = want[r][pos]
                scale = float(want[r].abs().max())
                err = float((row - ref).abs().max()) / scale
                worst_err = max(worst_err, err)
                assert err <= TOL[dtype], f"{name}/{dtype} request {r} position {pos}: {err:.2e} of the scale"
            assert len(got) == sum(last - first + 1 for _, first, last in reqs.values())
        else:
            # the pick inside the graph is the argmax of the same step's logits
            for key, pick in got.items():
                row = logits[key]
                assert pick == int((row == row.max()).nonzero().max()), f"{name}/{dtype} {key}"
        engine.cache.manager.check()
        engine.cache.flush()
        assert engine.cache.manager.free_pages(0) == engine.cache.n_pages, "pages were lost"
        del engine
        torch.cuda.empty_cache()


def test_more_decoding_requests_than_the_fused_attention_takes(tmp_path):
    """60 requests over 8 kv heads are 480 (request, kv head) pairs: more CTAs than the decode
    attention that rotates and writes by itself is used for, so the step takes the rotation
    kernel and the attention kernel.  Every request's logits against the plain implementation,
    through the captured graph."""
    from conftest import make_model_folder
    from axon_b200.engine.step import StepEntry
    from axon_b200.kernels import fast
    cfg = dict(TINY["A"], num_attention_heads=8, num_key_value_heads=8, head_dim=16, hidden_size=64,
               max_position_embeddings=160, vocab_size=300, num_hidden_layers=2)
    folder = make_model_folder(str(tmp_path / "wide_batch"), cfg, 31)
    pcfg, w = plain.read_model(folder)
    n_req, n_dec = 60, 6
    assert n_req * 8 > 3 * fast.SM_COUNT
    g = torch.Generator().manual_seed(9)
    toks = [torch.randint(0, 300, (20 + (7 * r) % 90 + n_dec,), generator=g).tolist() for r in range(n_req)]
    want = [plain.forward(pcfg, w, t) for t in toks]
    for dtype in ("bfloat16", "float32"):
        engine = build(folder, dtype, max_tokens=n_req * 128, page_size=16, max_slots=n_req, max_positions=160, shuffle_seed=3)
        slots = [engine.open_request() for _ in range(n_req)]
        for r in range(n_req):
            engine.step([StepEntry(slots[r], toks[r][:-n_dec], [])])
        for k in range(n_dec):
            res = engine.step([StepEntry(slots[r], [toks[r][len(toks[r]) - n_dec + k]], [0]) for r in range(n_req)]).double().cpu()
            for r in range(n_req):
                pos = len(toks[r]) - n_dec + k
                err = float((res[r] - want[r][pos]).abs().max()) / float(want[r].abs().max())
                assert err <= TOL[dtype], f"{dtype} request {r} step {k}: {err:.2e}"
        if dtype == "bfloat16":
            assert engine.cuda_graphs and len(engine._graphs) >= 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_token_portions_at_short_and_long_contexts(long_folders, dtype):
    """A portion of two tokens takes the decode-shape attention, whose key-split count follows the
    context: the same portion size comes at a short context (captured as a graph from the
    second time), then after a long stretch of prompt (another split count: another graph)."""
    name = "C"
    cfg, w = plain.read_model(long_folders[name])
    n = 2 * 4 + 900 + 2 * 6
    toks = _long_tokens(name, 77, n)
    want = plain.forward(cfg, w, toks)
    engine = build(long_folders[name], dtype, max_tokens=1024, page_size=16, max_slots=2, max_positions=1536)
    tr, at = Trace(), 0
    # (another request's long portion first: scratch buffers reach their size, so no graph is dropped later)
    tr.step([("w", ("x",), toks[:900], [])], end=["w"])
    sizes = [2] * 4 + [900] + [2] * 6
    for size in sizes:
        tr.step([("r", ("x",), toks[at:at + size], [0, size - 1])], end=["r"] if at + size == n else [])
        at += size
    got = replay(engine, tr.steps)
    at = 0
    for k, size in enumerate(sizes):
        check_rows(got[k + 1], [want[at], want[at + size - 1]], TOL[dtype], f"{dtype} portion {k} of {size} at {at}")
        at += size
    if dtype == "bfloat16":
        keys = [k for k in engine._graphs if k[0] == "portion" and k[1] == 2]
        assert len({k[3] for k in keys}) >= 2, f"the split count belongs to a portion's graph key: {keys}"


def test_steps_queued_without_waiting_keep_their_own_tables(model_folders):
    """Steps are queued without the host ever waiting for one: a request ends, its slot is opened
    again for another request and fed, while earlier steps' table copies may still be pending.
    Every step must see the block table it was planned with: the results equal the same
    steps run with a wait after each."""
    from axon_b200.engine.step import StepEntry
    name = "A"
    outs = {}
    for waited in (True, False):
        engine = build(model_folders[name], "bfloat16", max_tokens=96, page_size=16, max_slots=2, shuffle_seed=2)
        res = []
        big = tokens_for(name, 90, 60)
        for round_ in range(12):
            a = engine.open_request()
            # a long portion first, so that the device is behind the host
            res.append(engine.step([StepEntry(a, big, [59])]).clone())
            for k in range(3):
                res.append(engine.step([StepEntry(a, [(7 * round_ + k) % 256], [0])]).clone())
            engine.close_request(a)
            b = engine.open_request()             # the same slot, pages handed out anew
            res.append(engine.step([StepEntry(b, tokens_for(name, 91 + round_, 17), [16])]).clone())
            res.append(engine.step([StepEntry(b, [round_], [0])]).clone())
            engine.close_request(b)
            if waited:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        outs[waited] = torch.cat(res)
    assert torch.equal(outs[True], outs[False])
