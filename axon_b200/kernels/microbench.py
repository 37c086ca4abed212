"""Timing single kernels: ``python -m axon_b200.kernels.microbench <kernel> [sizes]``.

Each run times one kernel with CUDA events after warm-up, flushing L2 between timed
launches by writing a buffer larger than L2 (or rotating through several copies of the
operands when ``--rotate`` is given), and prints one JSON line with the median time,
the algorithmic bytes and FLOPs, and the achieved rates.  The same command under
``ncu -k regex:<kernel>`` gives the counters of exactly that launch.

Kernels: ``gemm_small_m``, ``gemm_tc``, ``attention_decode``, ``attention_prefill``,
``rmsnorm``; ``gemm_chain``: the swapped and the tiled product, each as a captured chain of
launches over distinct weights (as the layers of a step follow one another), which is what the
rule that chooses between them was fitted to; and ``mma_probe``: the cycles an SM's tensor pipe spends per 64-key step on the
products of the prompt attention when nothing else holds them up (``csrc/cuda/mma_probe.cu``).
"""

from __future__ import annotations

import argparse
import json
import math
import statistics
import sys

import torch

from . import fast, lib, ops
from ..parts.base import Runtime, StepContext

DEV = "cuda:0"
L2_BYTES = 192 * 1024 * 1024


def _time(fn, iters: int, warmup: int, flush: bool):
    scrub = torch.empty(L2_BYTES, dtype=torch.uint8, device=DEV) if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    # Everything is queued before anything is waited for: the flush in front of each timed
    # launch keeps the GPU busy while the host queues the next launch, so the events bracket
    # device time and not the host's launch latency.
    pairs = []
    for _ in range(iters):
        if scrub is not None:
            scrub.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        pairs.append((e0, e1))
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) * 1e3 for a, b in pairs]
    return statistics.median(times), min(times)


def _report(name, args, us, best, nbytes, flops):
    print(json.dumps({"kernel": name, "median_us": round(us, 2), "min_us": round(best, 2),
                      "GB_s": round(nbytes / us / 1e3, 1), "TFLOP_s": round(flops / us / 1e6, 1),
                      "bytes": nbytes, "flops": flops, "args": vars(args)}))


def _ctx(segs, items=True):
    rt = Runtime(torch.bfloat16, DEV)
    pos, slot_of, rows, at = [], [], [[], [], [], []], 0
    for slot, n, kv_len in segs:
        pos += list(range(kv_len - n, kv_len))
        slot_of += [slot] * n
        for lst, v in zip(rows, (slot, at, n, kv_len)):
            lst.append(v)
        at += n
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    unit = i32([[s, 0] for s in range(len(segs))]).flatten() if all(n == 1 for _, n, _ in segs) else None
    return StepContext(rt=rt, n_tokens=at, tokens=i32([0] * at), positions=i32(pos), token_slot=i32(slot_of),
                       seg_slot=rows[0], seg_q_start=rows[1], seg_q_len=rows[2], seg_kv_len=rows[3],
                       segments=i32(rows), unit_items=unit, host_positions=pos)


def main() -> int:
    ap = argparse.ArgumentParser(prog="microbench")
    ap.add_argument("kernel", choices=["gemm_small_m", "gemm_tc", "attention_decode", "attention_prefill", "rmsnorm", "mma_probe", "gemm_chain"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=37888)
    ap.add_argument("--k", type=int, default=3584)
    ap.add_argument("--epilogue", default="store", choices=["store", "bf16", "residual", "swiglu"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=28)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true", help="do not flush L2 between launches")
    ap.add_argument("--target-ctas", type=int, default=0, help="gemm_small_m: CTAs the split-K aims at")
    ap.add_argument("--tile", default="", help="gemm_tc: force the tile shape, e.g. 2x256 (rows/128 x columns)")
    ap.add_argument("--rows", default="64,128,256,512", help="gemm_chain: row counts, comma-separated")
    ap.add_argument("--mma-sync", action="store_true", help="attention_prefill: the mma.sync kernel, not the tcgen05 one")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        print("microbench needs a CUDA GPU", file=sys.stderr)
        return 2
    lib.cuda()
    g = torch.Generator(device=DEV).manual_seed(0)
    flush = not a.no_flush

    if a.kernel == "mma_probe":
        import ctypes
        scratch = torch.zeros(2, dtype=torch.int64, device=DEV)
        cycles = (ctypes.c_ulonglong * 2)()
        steps = 1000
        rows = {}
        for what, name in ((1, "scores (M 128, N 64, K 16; 16 a step)"), (2, "values, P in shared memory, V MN-major (8 a step)"),
                           (3, "both, P in shared memory"), (4, "values, P in tensor memory"), (5, "both, P in tensor memory"),
                           (8, "the values' shape with both operands K-major")):
            fast.check(lib.cuda().axon_mma_probe(what, steps, scratch.data_ptr(), cycles, fast._stream()))
            rows[name] = {"scores_thread_cycles_per_step": round(cycles[0] / steps, 1), "values_thread_cycles_per_step": round(cycles[1] / steps, 1)}
            print(f"{name:56s} scores thread {cycles[0] / steps:7.1f}  values thread {cycles[1] / steps:7.1f}  cycles per step")
        print(json.dumps({"kernel": "mma_probe", "steps": steps, "math_cycles_per_step": 1024, "rows": rows}))
        return 0
    if a.kernel == "gemm_chain":
        epi = {"store": fast.EPI_STORE_F32, "residual": fast.EPI_RESIDUAL, "swiglu": fast.EPI_SWIGLU, "bf16": fast.EPI_STORE_BF16}[a.epilogue]
        copies = max(6, min(40, (300 << 20) // (a.n * a.k * 2) + 1))          # more weights than L2 holds
        ws = [(torch.randn(a.n, a.k, generator=g, device=DEV) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        scrub = torch.empty(L2_BYTES, dtype=torch.uint8, device=DEV)
        side = torch.cuda.Stream()
        rows = {}
        for m in [int(v) for v in a.rows.split(",")]:
            x = torch.randn(m, a.k, generator=g, device=DEV).to(torch.bfloat16)
            out = (torch.empty(m, a.n // 2, dtype=torch.bfloat16, device=DEV) if a.epilogue == "swiglu" else
                   torch.zeros(m, a.n, dtype=torch.bfloat16 if a.epilogue == "bf16" else torch.float32, device=DEV))
            swapped = lambda w: fast._gemm_small(x, w, None, out, epi, m, a.n, a.k)
            tiled = lambda w: fast.check(lib.cuda().axon_gemm_tc(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), epi, m, a.n, a.k,
                                                                 out.stride(0), fast._stream()))
            got = {}
            for name, launch in (("swapped", swapped), ("tiled", tiled)):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.stream(side):
                    launch(ws[0])
                    torch.cuda.synchronize()
                    with torch.cuda.graph(graph, stream=side):
                        for w in ws:
                            launch(w)
                times = []
                for _ in range(a.iters):
                    scrub.zero_()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    graph.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    times.append(e0.elapsed_time(e1) * 1e3 / copies)
                got[name] = round(statistics.median(times[1:] or times), 1)
            got["rule_takes"] = "swapped" if fast._takes_swapped_kernel(m, a.n, a.k) else "tiled"
            rows[m] = got
            print(f"rows {m:5d}: swapped {got['swapped']:8.1f} us   tiled {got['tiled']:8.1f} us   (the rule takes the {got['rule_takes']} one)")
        print(json.dumps({"kernel": "gemm_chain", "n": a.n, "k": a.k, "epilogue": a.epilogue, "weights_in_chain": copies, "us_per_launch": rows}))
        assert fast.gemm_tc_status() == 0
        return 0
    if a.kernel in ("gemm_small_m", "gemm_tc"):
        x = torch.randn(a.m, a.k, generator=g, device=DEV).to(torch.bfloat16)
        w = (torch.randn(a.n, a.k, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
        if a.epilogue == "swiglu":
            out = torch.empty(a.m, a.n // 2, dtype=torch.bfloat16, device=DEV)
            fn = lambda: fast.gemm_swiglu(x, w, out)
        else:
            out = torch.zeros(a.m, a.n, dtype=torch.bfloat16 if a.epilogue == "bf16" else torch.float32, device=DEV)
            fn = lambda: fast.gemm(x, w, out, None, a.epilogue == "residual")
        if a.kernel == "gemm_small_m":
            fast.SWAP_RULE = "always"                                               # the swapped kernel at any size it takes
        if a.kernel == "gemm_tc":
            fast.SWAP_RULE = "never"                                                # the tiled kernel
        if a.tile:
            rm, bn = a.tile.split("x")
            lib.cuda().axon_gemm_tc_force_tile(int(rm), int(bn))
        if a.target_ctas:
            fast.SPLIT_TARGET_CTAS = a.target_ctas
        us, best = _time(fn, a.iters, a.warmup, flush)
        nbytes = 2 * (a.n * a.k + a.m * a.k) + out.numel() * out.element_size()
        _report(a.kernel, a, us, best, nbytes, 2 * a.m * a.n * a.k)
        if a.kernel == "gemm_tc":
            assert fast.gemm_tc_status() == 0
    elif a.kernel in ("attention_decode", "attention_prefill"):
        decode = a.kernel == "attention_decode"
        q_len = 1 if decode else a.context
        stride = -(-a.context // a.page_size)
        n_pages = a.batch * stride
        pool = (torch.randn(n_pages + 1, 1, 2, a.kv_heads, a.page_size, a.head_dim, generator=g, device=DEV) * 0.5).to(torch.bfloat16)
        table = torch.randperm(n_pages, device=DEV).to(torch.int32).view(a.batch, stride)
        view = ops.KvView(pool, table, 0, a.page_size, a.kv_heads, a.head_dim, 0)
        ctx = _ctx([(s, q_len, a.context) for s in range(a.batch)])
        q = torch.randn(ctx.n_tokens, a.heads * a.head_dim, generator=g, device=DEV).to(torch.bfloat16)
        out = torch.empty_like(q)
        scale = 1.0 / math.sqrt(a.head_dim)
        if a.mma_sync:
            fast.ENABLED["attention_tc"] = False
        fn = lambda: fast.attention(q, view, ctx, out, a.heads, scale)
        assert fn()
        us, best = _time(fn, a.iters, a.warmup, flush)
        kv_bytes = a.batch * a.context * a.kv_heads * a.head_dim * 2 * 2
        nbytes = kv_bytes + 2 * q.numel() * 2
        pairs = a.batch * (a.context if decode else a.context * (a.context + 1) // 2)
        _report(a.kernel, a, us, best, nbytes, 4 * pairs * a.heads * a.head_dim)
        assert fast.attention_tc_status() == 0
    else:
        x = torch.randn(a.m, a.k, generator=g, device=DEV)
        gain = torch.ones(a.k, device=DEV)
        out = torch.empty(a.m, a.k, dtype=torch.bfloat16, device=DEV)
        us, best = _time(lambda: ops.rmsnorm(x, gain, out, 1e-6), a.iters, a.warmup, flush)
        _report(a.kernel, a, us, best, x.numel() * 4 + out.numel() * 2, 3 * x.numel())
    return 0


if __name__ == "__main__":
    sys.exit(main())
