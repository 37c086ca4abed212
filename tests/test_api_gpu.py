"""Generation through the entry point: greedy output equals the plain implementation's,
sampling is seeded and the same alone and in a batch, continuous batching with too few
pages preempts and still gives every request its own output, and the command line."""

import os
import subprocess

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from conftest import ROOT, TINY

pytestmark = pytest.mark.gpu


def prompt_for(name, i, n):
    g = torch.Generator().manual_seed(7000 + 100 * (ord(name) - 64) + i)
    return torch.randint(0, TINY[name]["vocab_size"], (n,), generator=g).tolist()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lengths,n_gen", [("A", [5, 17, 31], 16), ("B", [1, 9, 40], 12)])
def test_greedy_generation_matches_plain(model_folders, name, lengths, n_gen, dtype):
    import axon_b200 as axon
    cfg, w = plain.read_model(model_folders[name])
    model = axon.load(model_folders[name])
    net = axon.Backend(model, axon.BackendOptions().max_ctx(128).dtype(dtype))
    for i, n in enumerate(lengths):
        ids = prompt_for(name, i, n)
        want = plain.greedy(cfg, w, ids, n_gen)
        with net.new_cache(128) as cache:
            logits = net.prefill_logits(ids, 0, cache)
            assert logits.shape == (cfg["vocab_size"],) and logits.dtype == np.float32
            emitted = []
            st = axon.generate(net, cache, ids, logits, axon.GenOpts.greedy(n_gen, []), emit=emitted.append)
        if dtype == "float32":
            assert st.ids == want
        else:
            # bfloat16 may flip a pick where the two best logits are closer than its rounding:
            # then the continuation differs legitimately; the tokens before must agree
            ref = plain.forward(cfg, w, ids + want)
            for k, (a, b) in enumerate(zip(st.ids, want)):
                if a != b:
                    row = ref[n - 1 + k]
                    top2 = torch.topk(row, 2).values
                    assert float(top2[0] - top2[1]) < 3e-2 * float(ref.abs().max()), f"pick {k} differs"
                    break
        assert emitted == st.ids and st.passes == n_gen - 1 and st.decided == n_gen
    # batched through the scheduler: the same tokens as alone
    prompts = [prompt_for(name, i, n) for i, n in enumerate(lengths)]
    outs = net.generate_batch(prompts, n_gen)
    if dtype == "float32":
        assert outs == [plain.greedy(cfg, w, p, n_gen) for p in prompts]


def test_stop_token_and_positions(model_folders):
    import axon_b200 as axon
    cfg, w = plain.read_model(model_folders["A"])
    net = axon.Backend(axon.load(model_folders["A"]), axon.BackendOptions().max_ctx(64).dtype("float32"))
    ids = prompt_for("A", 9, 7)
    want = plain.greedy(cfg, w, ids, 10)
    with net.new_cache() as cache:
        logits = net.prefill_logits(ids, 0, cache)
        st = axon.generate(net, cache, ids, logits, axon.GenOpts.greedy(10, [want[4]]))
        assert st.ids == want[:want.index(want[4])]
        with pytest.raises(axon.StepError, match="does not continue"):
            net.forward(3, 0, cache)
    assert axon.argmax(np.array([1.0, 3.0, 3.0, np.nan])) == 2


def test_sampling_is_seeded_and_batch_equals_alone(model_folders):
    import axon_b200 as axon
    net = axon.Backend(axon.load(model_folders["B"]), axon.BackendOptions().max_ctx(128).dtype("float32").parallel(4))
    prompts = [prompt_for("B", i, n) for i, n in enumerate([1, 9, 40, 77])]
    cfgs = [axon.SampleCfg(temp=0.8, seed=11 + i) for i in range(4)]
    cfgs[2] = axon.SampleCfg(temp=1.3, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0, seed=5)   # device draw
    cfgs[3] = axon.SampleCfg(temp=0.7, top_k=300, top_p=0.95, min_p=0.01, repeat_penalty=1.3, seed=6)  # host-sorted path
    alone = []
    for p, c in zip(prompts, cfgs):
        with net.new_cache() as cache:
            logits = net.prefill_logits(p, 0, cache)
            alone.append(axon.generate(net, cache, p, logits, axon.GenOpts.sampled(24, [], c)).ids)
    again = []
    for p, c in zip(prompts, cfgs):
        with net.new_cache() as cache:
            logits = net.prefill_logits(p, 0, cache)
            again.append(axon.generate(net, cache, p, logits, axon.GenOpts.sampled(24, [], c)).ids)
    assert alone == again, "the same seed gives the same tokens"
    assert all(len(a) == 24 for a in alone)
    greedy = net.generate_batch(prompts, 24)
    assert alone != greedy, "temperature sampling differs from greedy somewhere"
    batch = net.generate_batch(prompts, 24, sample=cfgs)
    assert batch == alone, "a request samples the same tokens in a batch as alone"


def test_continuous_batching_with_too_few_pages(model_folders):
    """Eight requests, four slots, a pool that cannot hold four grown requests: some are
    preempted and fed again, and every output equals the request run alone."""
    import axon_b200 as axon
    from axon_b200.engine.serve import BatchRunner
    cfg, w = plain.read_model(model_folders["A"])
    opts = axon.BackendOptions().max_ctx(96).dtype("float32").parallel(4).kv_tokens(160).step_tokens(24)
    net = axon.Backend(axon.load(model_folders["A"]), opts)
    prompts = [prompt_for("A", 20 + i, n) for i, n in enumerate([30, 5, 44, 17, 9, 25, 3, 38])]
    n_gen = [30, 40, 20, 35, 12, 28, 45, 16]
    runner = BatchRunner(net.engine, max_batch_tokens=24, max_running=4, prefill_chunk=16)
    for i, (p, n) in enumerate(zip(prompts, n_gen)):
        runner.add(i, p, n)
    seen = {i: [] for i in range(8)}
    outs = runner.run(lambda rid, tok: seen[rid].append(tok))
    assert runner.preemptions > 0, "the pool was meant to be too small"
    for i, (p, n) in enumerate(zip(prompts, n_gen)):
        assert outs[i] == plain.greedy(cfg, w, p, n), f"request {i}"
    net.engine.cache.manager.check()
    net.engine.cache.flush()
    assert net.engine.cache.manager.free_pages(0) == net.engine.cache.n_pages
    assert net.engine.cache.manager.n_open == 0


def test_sampled_requests_survive_preemption(model_folders):
    """Greedy and sampled requests (different seeds, k, penalties; one drawing on the device, one
    sorted on the host) share four slots and a pool too small for them: some are preempted and
    fed again with their sampler state kept, and every request's tokens equal those of the
    same request run alone (the reference's test: src/cuda/qwen2/slots.rs:1622-1796)."""
    import axon_b200 as axon
    from axon_b200.engine.serve import BatchRunner
    folder = model_folders["B"]
    prompts = [prompt_for("B", 40 + i, n) for i, n in enumerate([30, 5, 44, 17, 9, 25, 3, 38])]
    n_gen = [30, 40, 20, 35, 12, 28, 45, 16]
    cfgs = [None,
            axon.SampleCfg(temp=0.8, seed=21),
            axon.SampleCfg(temp=1.0, top_k=5, top_p=1.0, repeat_penalty=1.0, seed=22),
            None,
            axon.SampleCfg(temp=1.3, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0, seed=23),      # device draw
            axon.SampleCfg(temp=0.7, top_k=300, top_p=0.95, min_p=0.01, repeat_penalty=1.3, seed=24),  # host-sorted
            axon.SampleCfg(temp=0.9, top_k=40, top_p=0.9, repeat_penalty=1.2, repeat_last_n=8, seed=25),
            None]
    roomy = axon.Backend(axon.load(folder), axon.BackendOptions().max_ctx(128).dtype("float32").parallel(2))
    alone = []
    for p, n, c in zip(prompts, n_gen, cfgs):
        with roomy.new_cache() as cache:
            logits = roomy.prefill_logits(p, 0, cache)
            opts = axon.GenOpts.greedy(n, []) if c is None else axon.GenOpts.sampled(n, [], c)
            alone.append(axon.generate(roomy, cache, p, logits, opts).ids)
    opts = axon.BackendOptions().max_ctx(96).dtype("float32").parallel(4).kv_tokens(160).step_tokens(24)
    net = axon.Backend(axon.load(folder), opts)
    runner = BatchRunner(net.engine, max_batch_tokens=24, max_running=4, prefill_chunk=16)
    for i, (p, n, c) in enumerate(zip(prompts, n_gen, cfgs)):
        runner.add(i, p, n, (), c)
    outs = runner.run()
    assert runner.preemptions > 0, "the pool was meant to be too small"
    for i in range(len(prompts)):
        assert outs[i] == alone[i], f"request {i} ({'greedy' if cfgs[i] is None else 'sampled'})"
    net.engine.cache.manager.check()
    net.engine.cache.flush()
    assert net.engine.cache.manager.free_pages(0) == net.engine.cache.n_pages


def test_command_line(model_folders):
    cfg, w = plain.read_model(model_folders["B"])
    ids = prompt_for("B", 3, 12)
    want = plain.greedy(cfg, w, ids, 6)
    axon = os.path.join(ROOT, "bin", "axon")
    p = subprocess.run([axon, "gen", model_folders["B"], " ".join(map(str, ids)), "-n", "6", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.split()] == want
    assert "prompt eval:" in p.stderr and "decode:" in p.stderr
    p = subprocess.run([axon, "logits", model_folders["B"], " ".join(map(str, ids)), "-k", "3", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    row = plain.forward(cfg, w, ids)[-1]
    lines = p.stdout.strip().splitlines()
    assert len(lines) == 3
    assert int(lines[0].split()[0]) == want[0]
    assert abs(float(lines[0].split()[1]) - float(row.max())) < 2e-5 * float(row.abs().max())
    # the oracle hooks: positions 8.. after a batched prefix of 9, each as a pass of its own, with the next token's -ln p
    env = dict(os.environ, AXON_LOGITS_IDS=",".join(map(str, ids)), AXON_LOGITS_PREFIX="9", AXON_LOGITS_NLL="1")
    full = plain.forward(cfg, w, ids)
    for each in ("0", "1"):
        p = subprocess.run([axon, "logits", model_folders["B"], "-k", "2", "--dtype", "float32"],
                           capture_output=True, text=True, timeout=600, env=dict(env, AXON_LOGITS_EACH=each))
        assert p.returncode == 0, p.stderr[-2000:]
        out = p.stdout.splitlines()
        assert out[0] == f"prompt ids (12): {ids}"
        assert [l for l in out if l.startswith("position")] == [f"position {k}:" for k in range(8, 12)]
        nll = {int(l.split()[1]): (int(l.split()[2]), float(l.split()[3])) for l in out if l.startswith("nll")}
        assert sorted(nll) == [8, 9, 10]
        for pos, (nxt, v) in nll.items():
            want_nll = float(torch.logsumexp(full[pos], 0) - full[pos][ids[pos + 1]])
            assert nxt == ids[pos + 1] and abs(v - want_nll) < 1e-3, f"each={each} position {pos}"
        best = [int(out[k + 1].split()[0]) for k, l in enumerate(out) if l.startswith("position")]
        assert best == [int(full[k].argmax()) for k in range(8, 12)]
    p = subprocess.run([axon, "logits", model_folders["B"], "-k", "1", "--dtype", "float32"], capture_output=True, text=True,
                       timeout=600, env=dict(os.environ, AXON_LOGITS_IDS=",".join(map(str, ids)), AXON_LOGITS_ALL="3"))
    assert p.returncode == 0 and [l for l in p.stdout.splitlines() if l.startswith("position")] == [f"position {k}:" for k in (9, 10, 11)]
    p = subprocess.run([axon, "gen", model_folders["B"], "1 2", "--temp", "7000"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 2 and "--temp needs a number from 0 to 100" in p.stderr
    p = subprocess.run([axon, "info", model_folders["B"]], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "layers 3 (schedule of 3 runs) / dim 96 / vocab 384 / ctx 256" in p.stdout
    assert "num_key_value_heads 1" in p.stdout and "3 x prenorm(" in p.stdout
