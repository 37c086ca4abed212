"""Kernel timeline of engine steps on the GPU (CUPTI through ``torch.profiler``).

    python -m axon_b200.kernels.timeline decode  --batch 8 --context 2048 --layers 4
    python -m axon_b200.kernels.timeline prefill --tokens 2048 --layers 4

Builds a model with the layer sizes of Qwen2.5-7B (``--shape`` for 1.5B or 32B; random weights,
``--layers`` layers), runs
a few steps, and prints for every kernel of the last one its start and end in microseconds
after the step's first kernel, its duration, and how long after the end of the kernel
before it it ended.  Under programmatic dependent launch a kernel starts early and waits
for its predecessor inside, so the last column (not the duration) is what a kernel costs in the chain.
Only CUDA activities are recorded, nothing is replayed, and clocks are left alone.
"""

from __future__ import annotations

import argparse
import sys

import torch

COMMON = dict(rms_norm_eps=1e-6, rope_theta=1000000.0, hidden_act="silu", max_position_embeddings=32768)
#: layer sizes of the Qwen2.5 models by name
SHAPES = {
    "7b": dict(COMMON, hidden_size=3584, intermediate_size=18944, num_attention_heads=28, num_key_value_heads=4,
               vocab_size=152064, tie_word_embeddings=False),
    "1.5b": dict(COMMON, hidden_size=1536, intermediate_size=8960, num_attention_heads=12, num_key_value_heads=2,
                 vocab_size=151936, tie_word_embeddings=True),
    "32b": dict(COMMON, hidden_size=5120, intermediate_size=27648, num_attention_heads=40, num_key_value_heads=8,
                vocab_size=152064, tie_word_embeddings=False),
}


def main() -> int:
    ap = argparse.ArgumentParser(prog="timeline")
    ap.add_argument("kind", choices=["decode", "prefill"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--shape", choices=sorted(SHAPES), default="7b", help="whose layer sizes")
    ap.add_argument("--rows", type=int, default=60, help="kernels of the last step to print")
    ap.add_argument("--swap-rule", choices=["model", "always", "never"], default="model",
                    help="which products take the swapped kernel (kernels.fast.SWAP_RULE)")
    ap.add_argument("--disable", action="append", default=[], metavar="KERNEL",
                    help="switch a tuned kernel off (a key of kernels.fast.ENABLED); may be repeated")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        print("timeline needs a CUDA GPU", file=sys.stderr)
        return 2
    from torch.profiler import ProfilerActivity, profile

    from . import fast
    fast.SWAP_RULE = a.swap_rule
    for name in a.disable:
        if name not in fast.ENABLED:
            ap.error(f"--disable {name}: not one of {sorted(fast.ENABLED)}")
        fast.ENABLED[name] = False
    from ..config import config_from_dict
    from ..engine.build import build_engine
    from ..engine.step import StepEntry

    cfg = config_from_dict(dict(SHAPES[a.shape], num_hidden_layers=a.layers, architectures=["Qwen2ForCausalLM"], model_type="qwen2"))
    room = max(a.context + 64, a.tokens + 64)
    slots = a.batch if a.kind == "decode" else 2
    engine = build_engine(config=cfg, seed=1, dtype="bfloat16", page_size=16, max_tokens=slots * (-(-room // 16) * 16),
                          max_slots=slots, max_positions=room, gain_std=0.0)
    if a.kind == "decode":
        reqs = [engine.open_request() for _ in range(a.batch)]
        for s in reqs:                                  # contexts of synthetic cache contents
            engine.cache.reserve(s, a.context)
            engine.cache.commit(s, a.context)
        step = lambda: engine.step([StepEntry(s, [1], [0]) for s in reqs])
    else:
        toks = [1 + i % 1000 for i in range(a.tokens)]

        def step():
            s = engine.open_request()
            engine.step([StepEntry(s, toks, [a.tokens - 1])])
            engine.close_request(s)
    for _ in range(6):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    ks = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                 if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda t: t[0])
    if not ks:
        print("no CUDA activity was recorded", file=sys.stderr)
        return 1
    t0, prev_end = ks[0][0], ks[0][0]
    print(f"{'start':>9} {'end':>9} {'dur':>7} {'after':>7}  kernel")
    for start, end, name in ks[:a.rows]:
        print(f"{start - t0:9.1f} {end - t0:9.1f} {end - start:7.1f} {end - prev_end:7.1f}  {name[:70]}")
        prev_end = max(prev_end, end)
    print(f"step: {ks[-1][1] - t0:.1f} us over {len(ks)} activities")
    return 0


if __name__ == "__main__":
    sys.exit(main())
