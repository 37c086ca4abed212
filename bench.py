#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-7B layer sizes, bfloat16,
random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

A step is one decode step of a batch of requests that each hold ``--context``
positions.  ``value`` is decoded tokens per second, timed on the device with CUDA
events over K steps after W warm-up steps; ``e2e`` is the same through the Python
entry point (``Backend.decode_batch``: host token ids in, picked ids out, every
step), timed by the host clock around synchronised steps.  The line also carries a
2,048-token prefill, decode at batch 1 and 64, and the decode step's HBM roofline.
The weights (15 GB) are far larger than L2, so every step re-reads them from HBM.

Contexts are synthetic: each request's cache pages are taken through the cache
manager and filled with random keys and values instead of being computed from a
prompt; what a decode step reads and computes is the same.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Qwen2.5-7B shape
QWEN25_7B = dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
                 head_dim=128, intermediate_size=18944, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6,
                 tie_word_embeddings=False, max_position_embeddings=32768)
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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="axon_b200", choices=["axon_b200", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048, help="positions each request holds when decoding starts")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=QWEN25_7B["num_hidden_layers"],
                    help="run fewer layers than the 28 of the configuration (both numbers go into `config`)")
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch 1 / 64 points")
    ap.add_argument("--skip-prefill", action="store_true", help="leave out the prefill measurement (for profiles)")
    ap.add_argument("--prefill-only", action="store_true", help="run the prefill measurement alone (for profiles)")
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
    if args.warmup < 3:
        args.warmup = 3

    import torch

    import axon_b200 as axon
    from axon_b200.config import config_from_dict
    from axon_b200.engine.build import build_engine
    from axon_b200.engine.step import StepEntry
    from axon_b200.kernels import lib

    pk, pk_src = peaks()
    cfg_d = dict(QWEN25_7B, architectures=["Qwen2ForCausalLM"], model_type="qwen2")
    full_layers = cfg_d["num_hidden_layers"]
    cfg_d["num_hidden_layers"] = args.layers
    cfg = config_from_dict(cfg_d)
    batches = [args.batch] + ([] if args.skip_points else [1, 64])
    max_b = max(batches)
    room = args.context + 2 * args.steps + args.warmup + 3 + 64      # warm-up, the timed steps, the end-to-end steps
    pool_tokens = max(max_b * (-(-room // 16) * 16), args.prefill_tokens + 64)
    t0 = time.time()
    engine = build_engine(config=cfg, seed=1, dtype="bfloat16", page_size=16, max_tokens=pool_tokens,
                          max_slots=max_b, max_positions=max(room, args.prefill_tokens + 64),
                          max_step_tokens=max(args.prefill_tokens, 64), gain_std=0.0)
    net = axon.Backend(None, axon.BackendOptions(), engine=engine)
    dev = engine.rt.device
    for g in engine.cache.groups:      # synthetic keys and values
        g.pool.normal_(0.0, 0.5)
    torch.cuda.synchronize()
    setup_s = time.time() - t0

    D, H, Hkv, hd, F, V, L = (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                              cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers)
    layer_params = (H * hd + 2 * Hkv * hd) * D + D * H * hd + 3 * D * F
    weight_bytes = 2 * (L * layer_params + V * D)              # every matrix a decode step reads once
    kv_bytes_per_pos = L * 2 * Hkv * hd * 2
    gen = torch.Generator().manual_seed(0)

    def open_requests(b, context):
        caches = [net.new_cache() for _ in range(b)]
        for c in caches:          # a synthetic context: pages taken, keys and values random
            assert engine.cache.reserve(c.slot, context)
            engine.cache.commit(c.slot, context)
        return caches

    def time_decode(b, steps, warmup, with_clocks=False):
        caches = open_requests(b, args.context)
        toks = torch.randint(0, V, (b,), generator=gen).tolist()
        for _ in range(warmup):
            toks = net.decode_batch(toks, caches)
        for _ in range(min(warmup, 3)):      # the plain step has a graph of its own: captured here, not in the timed loop
            engine.step([StepEntry(c.slot, [t], [0]) for c, t in zip(caches, toks)])
        torch.cuda.synchronize()
        launches0 = lib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler(dev.index or 0) if with_clocks else None
        if sampler:
            sampler.__enter__()
            time.sleep(0.3)
        e0.record()
        for _ in range(steps):
            logits = engine.step([StepEntry(c.slot, [t], [0]) for c, t in zip(caches, toks)])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = lib.launch_count() - launches0
        # end to end: host ids in, picked ids out, every step
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for _ in range(steps):
            toks = net.decode_batch(toks, caches)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - w0
        if sampler:
            sampler.__exit__()
        ctx_mid = args.context + warmup + steps // 2
        for c in caches:
            c.close()
        engine.cache.flush()
        return {"ms_per_step": ms / steps, "tok_s": b * steps / (ms / 1e3), "e2e_tok_s": b * steps / e2e_s,
                "launches": launches, "bytes": weight_bytes + b * ctx_mid * kv_bytes_per_pos,
                "clocks": sampler.summary() if sampler else None}

    def time_prefill(T, repeats=6):
        """One request, T tokens in one step; the best of the repeats after the first.  (The
        engine captures a portion size it meets a second time into a CUDA graph and replays it
        from the third; a graph's first replay still carries its upload.)"""
        ptoks = torch.randint(0, V, (T,), generator=gen).tolist()
        pms = []
        for it in range(repeats):
            with net.new_cache() as c:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                engine.step([StepEntry(c.slot, ptoks, [T - 1])])
                e1.record()
                torch.cuda.synchronize()
                pms.append(e0.elapsed_time(e1))
            engine.cache.flush()
        pm = min(pms[1:]) if len(pms) > 1 else pms[0]
        flops = 2 * L * layer_params * T + 2 * V * D + L * 2 * 2 * H * hd * T * (T + 1) / 2
        return {"value": round(T / (pm / 1e3), 1), "tokens": T, "ms": round(pm, 3),
                "frac": round(flops / (pm / 1e3) / 1e12 / pk["bf16_tflops"], 4)}

    if args.prefill_only:
        print(json.dumps({"prefill": time_prefill(args.prefill_tokens, max(2, args.steps))}))
        return 0
    main_r = time_decode(args.batch, args.steps, args.warmup, with_clocks=True)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            r = time_decode(b, max(8, args.steps // 4), 3)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(r["bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 3)
    prefill = None if args.skip_prefill else time_prefill(args.prefill_tokens)

    step_s = main_r["ms_per_step"] / 1e3
    achieved = main_r["bytes"] / step_s / 1e9
    b = args.batch
    out = {
        "metric": "decode tok/s @ batch 8 (Qwen2.5-7B shape, bf16)", "value": round(main_r["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_r["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "axon_b200",
        "config": {"model": "Qwen2.5-7B shape", "layers": L, "layers_of_config": full_layers, "hidden": D,
                   "heads": H, "kv_heads": Hkv, "head_dim": hd, "ffn": F, "vocab": V, "global_batch": b,
                   "seq_len": args.context, "page_size": 16, "parallelism": "1 GPU",
                   "weights": "random N(0,0.02), gains 1", "context": "synthetic cache contents",
                   "l2": "weights exceed L2, re-read every step", "peaks": pk_src},
        "e2e": {"value": round(main_r["e2e_tok_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 4 * (3 * b + 4 * b + b), "d2h_bytes_per_step": 4 * b},
        "gpu_launches": main_r["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": main_r["clocks"],
        "setup_s": round(setup_s, 1),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
