#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5 layer sizes, bfloat16, random
weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--rounds R] [--batch 8] [--layers L]
                    [--skip-serving] [--with-32b] [--shape 7b|1.5b|32b]

The headline is the 7B shape: a step is one decode step of a batch of requests that each hold
``--context`` positions.  ``value`` is decoded tokens per second, timed on the device with
CUDA events over K steps after W warm-up steps; ``e2e`` is the same through the Python
entry point (``Backend.decode_batch``: host token ids in, picked ids out, every step),
timed by the host clock around synchronised steps.  Everything is measured in R interleaved
rounds (decode at the main batch, at batch 1 and 64, then the 2,048-token prefill, and again);
the line reports each quantity's median over the rounds and, under ``rounds``, its smallest
and largest.  The weights (15 GB) are far larger than L2, so every step re-reads them from HBM.
``prefill.frac`` is the step's FLOPs over its time over the cuBLAS bfloat16 rate measured as a
burst; ``frac_of_sustained`` the same over the rate that cuBLAS holds through seconds under the
power cap, which is what a prefill between decode rounds (and the 0.5 s prefill at the 32B sizes)
runs under.

Contexts are synthetic: each request's cache pages are taken through the cache manager and
filled with random keys and values instead of being computed from a prompt; what a decode
step reads and computes is the same.

Two further workloads go into the same line as ``points_1p5b`` (by default; ``--skip-serving``
leaves it out) and ``points_32b`` (``--with-32b``, or alone with ``--shape 32b``):

* the 1.5B shape under continuous batching: 128 requests with prompts of 64 to 1,024 seeded
  random ids, 256 greedy tokens each, through ``Backend.generate_batch`` (the scheduler cuts
  the prompts into steps of at most 8,192 tokens beside the decoding rows);
* the 32B shape: a prefill of 8,192 tokens, then decode steps at batch 1, 8 and 32 at contexts
  of 8,192, 12,288 and 16,384 (batch 32 at the largest context the cache pool can hold beside
  65.5 GB of weights, which is less than 16,384: the line says how much).
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the layer sizes of the three Qwen2.5 shapes the measurements are quoted on
SHAPES = {
    "7b": dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
               head_dim=128, intermediate_size=18944, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6,
               tie_word_embeddings=False, max_position_embeddings=32768),
    "1.5b": dict(num_hidden_layers=28, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2,
                 head_dim=128, intermediate_size=8960, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                 tie_word_embeddings=True, max_position_embeddings=32768),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                head_dim=128, intermediate_size=27648, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-5,
                tie_word_embeddings=False, max_position_embeddings=32768),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {k: float(p.get(k, FALLBACK_PEAKS[k])) for k in FALLBACK_PEAKS}, "measured"
        except (OSError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def sizes_of(cfg):
    """Parameters of one layer's matrices, bytes a decode step reads of the weights, cache bytes per position."""
    D, H, Hkv, hd, F, V, L = (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                              cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers)
    layer_params = (H * hd + 2 * Hkv * hd) * D + D * H * hd + 3 * D * F
    weight_bytes = 2 * (L * layer_params + V * D)              # every matrix a decode step reads once
    return layer_params, weight_bytes, L * 2 * Hkv * hd * 2


def prefill_flops(cfg, T):
    """Products of every layer and the head's one row, and the causal half of the attention."""
    layer_params, _, _ = sizes_of(cfg)
    L, H, hd, V, D = cfg.num_hidden_layers, cfg.num_attention_heads, cfg.head_dim, cfg.vocab_size, cfg.hidden_size
    return 2 * L * layer_params * T + 2 * V * D + L * 2 * 2 * H * hd * T * (T + 1) / 2


class Workbench:
    """An engine of one shape with random weights, and the timed workloads on it."""

    def __init__(self, shape: str, layers: int, max_slots: int, pool_tokens, max_positions: int, max_step_tokens: int):
        import torch

        import axon_b200 as axon
        from axon_b200.config import config_from_dict
        from axon_b200.engine.build import build_engine

        cfg_d = dict(SHAPES[shape], architectures=["Qwen2ForCausalLM"], model_type="qwen2")
        self.full_layers = cfg_d["num_hidden_layers"]
        cfg_d["num_hidden_layers"] = layers or self.full_layers
        self.cfg = config_from_dict(cfg_d)
        t0 = time.time()
        self.engine = build_engine(config=self.cfg, seed=1, dtype="bfloat16", page_size=16, max_tokens=pool_tokens,
                                   max_slots=max_slots, max_positions=max_positions, max_step_tokens=max_step_tokens,
                                   gain_std=0.0)
        self.net = axon.Backend(None, axon.BackendOptions(), engine=self.engine)
        for g in self.engine.cache.groups:      # synthetic keys and values
            g.pool.normal_(0.0, 0.5)
        torch.cuda.synchronize()
        self.setup_s = time.time() - t0
        self.gen = torch.Generator().manual_seed(0)
        self.torch = torch

    def close(self):
        self.engine._graphs.clear()
        self.engine.rt.release_buffers()
        self.engine = self.net = None
        gc.collect()
        self.torch.cuda.empty_cache()

    def time_decode(self, b, context, steps, warmup, with_clocks=False, e2e=True):
        """K decode steps of b requests that each hold `context` positions: device time, end-to-end time."""
        from axon_b200.engine.step import StepEntry
        from axon_b200.kernels import lib
        torch, engine, net = self.torch, self.engine, self.net
        V = self.cfg.vocab_size
        _, weight_bytes, kv_bytes_per_pos = sizes_of(self.cfg)
        caches = [net.new_cache() for _ in range(b)]
        for c in caches:          # a synthetic context: pages taken, keys and values random
            assert engine.cache.reserve(c.slot, context), "the bench's pool is too small for its contexts"
            engine.cache.commit(c.slot, context)
        toks = torch.randint(0, V, (b,), generator=self.gen).tolist()
        for _ in range(warmup):
            toks = net.decode_batch(toks, caches)
        for _ in range(min(warmup, 3)):      # the plain step has a graph of its own: captured here, not in the timed loop
            engine.step([StepEntry(c.slot, [t], [0]) for c, t in zip(caches, toks)])
        torch.cuda.synchronize()
        launches0 = lib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler(engine.rt.device.index or 0) if with_clocks else None
        if sampler:
            sampler.__enter__()
            time.sleep(0.3)
        e0.record()
        for _ in range(steps):
            engine.step([StepEntry(c.slot, [t], [0]) for c, t in zip(caches, toks)])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = lib.launch_count() - launches0
        e2e_s = None
        if e2e:
            # end to end: host ids in, picked ids out, every step
            torch.cuda.synchronize()
            w0 = time.perf_counter()
            for _ in range(steps):
                toks = net.decode_batch(toks, caches)
            torch.cuda.synchronize()
            e2e_s = time.perf_counter() - w0
        if sampler:
            sampler.__exit__()
        ctx_mid = context + warmup + steps // 2
        for c in caches:
            c.close()
        engine.cache.flush()
        nbytes = weight_bytes + b * ctx_mid * kv_bytes_per_pos
        return {"ms_per_step": ms / steps, "tok_s": b * steps / (ms / 1e3),
                "e2e_tok_s": b * steps / e2e_s if e2e_s else None, "launches": launches, "bytes": nbytes,
                "gbs": nbytes / (ms / steps / 1e3) / 1e9, "clocks": sampler.summary() if sampler else None}

    def time_prefill(self, T, repeats=5):
        """One request, T tokens in one step (cut into steps of the engine's limit when longer); the
        times of the repeats after the third.  (The engine captures a portion size it meets a second
        time into a CUDA graph and replays it from the third; a graph's first replay still carries
        its upload.)"""
        from axon_b200.engine.step import StepEntry
        torch, engine, net = self.torch, self.engine, self.net
        ptoks = torch.randint(0, self.cfg.vocab_size, (T,), generator=self.gen).tolist()
        limit = engine.max_step_tokens
        pms = []
        for it in range(repeats):
            with net.new_cache() as c:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                for at in range(0, T, limit):
                    part = ptoks[at:at + limit]
                    engine.step([StepEntry(c.slot, part, [len(part) - 1] if at + limit >= T else [])])
                e1.record()
                torch.cuda.synchronize()
                pms.append(e0.elapsed_time(e1))
            engine.cache.flush()
        return pms[3:] if len(pms) > 3 else pms[-1:]


def med(xs):
    return statistics.median(xs)


def bench_7b(args, pk, pk_src):
    batches = [args.batch] + ([] if args.skip_points else [1, 64])
    max_b = max(batches)
    room = args.context + 2 * args.steps + args.warmup + 3 + 64      # warm-up, the timed steps, the end-to-end steps
    pool_tokens = max(max_b * (-(-room // 16) * 16), args.prefill_tokens + 64)
    wb = Workbench("7b", args.layers, max_b, pool_tokens, max(room, args.prefill_tokens + 64),
                   max(args.prefill_tokens, 64))
    cfg = wb.cfg
    if args.prefill_only:
        ms = wb.time_prefill(args.prefill_tokens, max(3, args.steps))
        print(json.dumps({"prefill_ms": [round(m, 3) for m in ms]}))
        return None
    main, points, prefill_ms = [], {b: [] for b in batches[1:]}, []
    for r in range(args.rounds):
        main.append(wb.time_decode(args.batch, args.context, args.steps, args.warmup, with_clocks=(r == args.rounds // 2)))
        for b in batches[1:]:
            points[b].append(wb.time_decode(b, args.context, args.steps, 3, e2e=False))
        if not args.skip_prefill:
            prefill_ms += wb.time_prefill(args.prefill_tokens)
    mid = sorted(main, key=lambda r: r["tok_s"])[len(main) // 2]       # the round with the median rate
    b = args.batch
    D, H, Hkv, hd, F, V, L = (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                              cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers)
    out = {
        "metric": "decode tok/s @ batch 8 (Qwen2.5-7B shape, bf16)", "value": round(mid["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(mid["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "axon_b200",
        "config": {"model": "Qwen2.5-7B shape", "layers": L, "layers_of_config": wb.full_layers, "hidden": D,
                   "heads": H, "kv_heads": Hkv, "head_dim": hd, "ffn": F, "vocab": V, "global_batch": b,
                   "seq_len": args.context, "page_size": 16, "parallelism": "1 GPU",
                   "weights": "random N(0,0.02), gains 1", "context": "synthetic cache contents",
                   "l2": "weights exceed L2, re-read every step", "peaks": pk_src, "rounds": args.rounds},
        # host to device: tokens, positions, slots, four segment rows and two work-item values per
        # request, and one wanted row each; device to host: the picked ids
        "e2e": {"value": round(med([r["e2e_tok_s"] for r in main]), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 4 * (9 * b + b), "d2h_bytes_per_step": 4 * b},
        "gpu_launches": mid["launches"],
        "roofline": {"bound": "hbm", "achieved": round(mid["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(mid["gbs"] / pk["hbm_gbs"], 4)},
        "rounds": {"n": args.rounds, "value_min": round(min(r["tok_s"] for r in main), 1),
                   "value_max": round(max(r["tok_s"] for r in main), 1),
                   "e2e_min": round(min(r["e2e_tok_s"] for r in main), 1),
                   "e2e_max": round(max(r["e2e_tok_s"] for r in main), 1)},
        "clocks": next((r["clocks"] for r in main if r["clocks"]), None),
        "setup_s": round(wb.setup_s, 1),
    }
    if prefill_ms:
        T, pm = args.prefill_tokens, med(prefill_ms)
        out["prefill"] = {"value": round(T / (pm / 1e3), 1), "tokens": T, "ms": round(pm, 3),
                          "frac": round(prefill_flops(cfg, T) / (pm / 1e3) / 1e12 / pk["bf16_tflops"], 4),
                          "frac_of_sustained": round(prefill_flops(cfg, T) / (pm / 1e3) / 1e12 / pk["bf16_tflops_sustained"], 4),
                          "ms_min": round(min(prefill_ms), 3), "ms_max": round(max(prefill_ms), 3), "timed": len(prefill_ms)}
    else:
        out["prefill"] = None
    pts = {}
    for bb, rs in points.items():
        m = sorted(rs, key=lambda r: r["tok_s"])[len(rs) // 2]
        pts[f"decode_b{bb}"] = round(m["tok_s"], 1)
        pts[f"decode_b{bb}_hbm_frac"] = round(m["gbs"] / pk["hbm_gbs"], 3)
        pts[f"decode_b{bb}_min_max"] = [round(min(r["tok_s"] for r in rs), 1), round(max(r["tok_s"] for r in rs), 1)]
    out["points"] = pts
    wb.close()
    return out


def bench_serving_1p5b(args, pk):
    """128 requests, prompts of 64..1,024 random ids, 256 greedy tokens each, continuous batching."""
    import torch
    n_req, n_gen = args.serve_requests, args.serve_tokens
    g = torch.Generator().manual_seed(1234)
    lens = torch.randint(64, 1025, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, SHAPES["1.5b"]["vocab_size"], (n,), generator=g).tolist() for n in lens]
    pool = sum(-(-(n + n_gen) // 16) * 16 for n in lens) + 64 * 16
    wb = Workbench("1.5b", 0, n_req, pool, 1024 + n_gen + 16, 8192)
    _, weight_bytes, kv_per_pos = sizes_of(wb.cfg)
    net = wb.net
    from axon_b200.engine.serve import BatchRunner

    def run_once():
        runner = BatchRunner(wb.engine, max_batch_tokens=wb.engine.max_step_tokens, max_running=n_req)
        for i, p in enumerate(prompts):
            runner.add(i, p, n_gen)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = runner.run()
        torch.cuda.synchronize()
        return time.perf_counter() - t0, runner, outs
    run_once()                                                   # warm-up: graphs of every step shape are captured
    rounds = [run_once() for _ in range(max(args.rounds, 1))]
    secs, runner, outs = sorted(rounds, key=lambda r: r[0])[len(rounds) // 2]
    # a sample of requests alone: the same tokens as in the batch, up to where bfloat16 meets a near-tie
    # (another batch cuts the products' and the attention's sums elsewhere, which moves logits by
    # rounding; two logits closer than that may swap, and the sequences part ways from there)
    import axon_b200 as axon
    same = near_tie = wrong = 0
    sample = [0, n_req // 3, 2 * n_req // 3, n_req - 1]
    for i in sample:
        with net.new_cache() as cache:
            logits = net.prefill_logits_device(prompts[i], 0, cache)
            st = axon.generate(net, cache, prompts[i], logits, axon.GenOpts.greedy(n_gen, []))
        first = next((k for k in range(min(len(st.ids), len(outs[i]))) if st.ids[k] != outs[i][k]), None)
        if first is None and len(st.ids) == len(outs[i]):
            same += 1
            continue
        with net.new_cache() as cache:
            row = net.prefill_logits_device(prompts[i] + st.ids[:first], 0, cache).float()
        margin = abs(float(row[st.ids[first]] - row[outs[i][first]]))
        if margin <= 3e-2 * float(row.abs().max()):
            near_tie += 1
        else:
            wrong += 1
    done = sum(len(outs[i]) for i in range(n_req))
    prompt_tokens = sum(lens)
    # what the steps had to read at least: the weights once per step, and every live position once per decoded token
    kv_read = sum(kv_per_pos * (n * n_gen + n_gen * (n_gen - 1) // 2) for n in lens)
    res = {"workload": f"{n_req} requests, prompts U(64,1024), {n_gen} greedy tokens each, continuous batching",
           "completion_tok_s": round(done / secs, 1), "total_tok_s": round((done + prompt_tokens) / secs, 1),
           "seconds": round(secs, 3), "seconds_min_max": [round(min(r[0] for r in rounds), 3), round(max(r[0] for r in rounds), 3)],
           "steps": runner.steps, "preemptions": runner.preemptions,
           "mean_tokens_per_step": round(runner.step_tokens / max(runner.steps, 1), 1),
           "prompt_tokens": prompt_tokens, "generated_tokens": done,
           "hbm_frac_of_all_steps": round((runner.steps * weight_bytes + kv_read) / secs / 1e9 / pk["hbm_gbs"], 3),
           "sample_alone_vs_batch": {"requests": len(sample), "equal": same, "part_at_a_near_tie": near_tie, "differ": wrong},
           "setup_s": round(wb.setup_s, 1)}
    wb.close()
    return res


def bench_32b(args, pk):
    """Prefill of 8,192 tokens, then decode steps at batch 1, 8 and 32 at contexts up to 16,384."""
    slots, top = 32, 16384
    wb = Workbench("32b", 0, slots, None, top + 2 * args.steps + 128, 8192)      # the pool: what memory allows
    cfg = wb.cfg
    _, weight_bytes, kv_per_pos = sizes_of(cfg)
    pool = wb.engine.cache.n_pages * 16
    res = {"pool_tokens": pool, "weights_gb": round(weight_bytes / 1e9, 1), "kv_bytes_per_position": kv_per_pos,
           "setup_s": round(wb.setup_s, 1)}
    pms = wb.time_prefill(8192, repeats=4 + max(args.rounds - 1, 0))
    pm = med(pms)
    res["prefill"] = {"tokens": 8192, "ms": round(pm, 2), "value": round(8192 / (pm / 1e3), 1),
                      "frac": round(prefill_flops(cfg, 8192) / (pm / 1e3) / 1e12 / pk["bf16_tflops"], 4),
                      "frac_of_sustained": round(prefill_flops(cfg, 8192) / (pm / 1e3) / 1e12 / pk["bf16_tflops_sustained"], 4),
                      "ms_min_max": [round(min(pms), 2), round(max(pms), 2)]}
    steps, warm = args.steps, max(args.warmup, 3)
    for b in (1, 8, 32):
        fits = (pool // b) // 16 * 16 - (2 * steps + warm + 3 + 16)
        for context in (8192, 12288, top):
            note = None
            if context > fits:
                if context != top:
                    continue
                # batch 32 at 16,384 needs 137 GB of cache beside 65.5 GB of weights: more than the GPU has,
                # so the point is taken at the largest context the pool holds
                context, note = fits, "largest context that fits"
            rs = [wb.time_decode(b, context, steps, warm, e2e=False) for _ in range(max(args.rounds, 1))]
            m = sorted(rs, key=lambda r: r["tok_s"])[len(rs) // 2]
            key = f"decode_b{b}_ctx{context}"
            res[key] = round(m["tok_s"], 1)
            res[key + "_ms"] = round(m["ms_per_step"], 3)
            res[key + "_hbm_frac"] = round(m["gbs"] / pk["hbm_gbs"], 3)
            if note:
                res[key + "_note"] = note
    wb.close()
    return res


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--rounds", type=int, default=3, help="interleaved repeats of every measurement (medians are reported)")
    ap.add_argument("--impl", default="axon_b200", choices=["axon_b200", "reference"])
    ap.add_argument("--shape", default="7b", choices=["7b", "1.5b", "32b"],
                    help="7b: the headline (plus the 1.5B serving run); 1.5b / 32b: that workload alone")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048, help="positions each request holds when decoding starts")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the 28 of the 7B configuration (both numbers go into `config`)")
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch 1 / 64 points")
    ap.add_argument("--skip-prefill", action="store_true", help="leave out the prefill measurement (for profiles)")
    ap.add_argument("--prefill-only", action="store_true", help="run the prefill measurement alone (for profiles)")
    ap.add_argument("--skip-serving", action="store_true", help="leave out the 1.5B continuous-batching run")
    ap.add_argument("--with-32b", action="store_true", help="add the 32B points (about two minutes more)")
    ap.add_argument("--serve-requests", type=int, default=128)
    ap.add_argument("--serve-tokens", type=int, default=256)
    args = ap.parse_args()

    if args.impl == "reference":
        # The reference is a Rust crate (Cargo.toml, no Python packaging): pip has nothing to
        # install and no Rust toolchain exists here, and its GPU backend refuses bf16 weights.
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate without Python packaging (pip: 'neither setup.py nor "
                          "pyproject.toml found'); no cargo/rustc on this machine; its GPU path runs quantized GGUF only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    args.rounds = max(args.rounds, 1)

    pk, pk_src = peaks()
    if args.shape == "1.5b":
        print(json.dumps({"impl": "axon_b200", "dtype": "bf16", "data": "synthetic", "peaks": pk_src,
                          "points_1p5b": bench_serving_1p5b(args, pk)}))
        return 0
    if args.shape == "32b":
        print(json.dumps({"impl": "axon_b200", "dtype": "bf16", "data": "synthetic", "peaks": pk_src,
                          "points_32b": bench_32b(args, pk)}))
        return 0
    out = bench_7b(args, pk, pk_src)
    if out is None:
        return 0
    if not args.skip_serving:
        out["points_1p5b"] = bench_serving_1p5b(args, pk)
    if args.with_32b:
        out["points_32b"] = bench_32b(args, pk)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
