"""The command line, in the manner of the reference's ``axon`` (src/cli.rs:35-69, 856-1349):

    axon info   <model>                      print a summary and exit
    axon gen    <model> "<prompt>" [-n N] [--device D] [--ctx N] [--kv T] [--dtype T]
                [--verbose] [sampling flags]  generation (greedy unless --temp > 0)
    axon logits <model> "<prompt>" [-k K]    top-K next-token logits after the prompt

``<model>`` is a folder with config.json and safetensors.  The engine starts at token
ids: a prompt is a list of ids (``"1 2 3"`` or ``"1,2,3"``); when the folder holds a
``tokenizer.json`` and the ``tokenizers`` package is importable, other text is encoded
with it and the output decoded.  ``AXON_LOGITS_IDS`` gives ids in place of the prompt
(``;`` separates sequences); ``AXON_LOGITS_ALL=N``, ``AXON_LOGITS_PREFIX=N``, ``AXON_LOGITS_EACH=1``
and ``AXON_LOGITS_NLL=1`` print more positions (see ``_logits_of``): ``ALL`` prints the top-K of the last N
positions (src/cli.rs:971-1157).  Generated text goes to stdout, speeds to stderr.
"""

from __future__ import annotations

import os
import re
import sys
import time
from typing import List, Optional, Sequence

USAGE = """\
usage:
  axon <model>                              same as axon info
  axon info <model>                         print a summary and exit
  axon gen <model> "<prompt>" [-n N] [--device D] [--ctx N] [--kv T] [--dtype T] [--verbose]
            [sampling flags]
                                            generation (greedy unless --temp > 0)
  axon logits <model> "<prompt>" [-k K] [--dtype T]
                                            top-K next-token logits after the prompt
  axon -h | --help                          this help

flags:
  -n N        gen: tokens to generate (default 32)
  -k K        logits: how many candidates to print (default 10)
  --device D  cuda or cuda:N (there is no CPU path)
  --ctx N     gen: room for N positions (default: prompt + N + 1)
  --kv T      cache type: auto, bf16 or f32 (it follows --dtype)
  --dtype T   bfloat16 (default) or float32 (every kernel in true 32-bit)
  --verbose   gen: print the configuration and the kernels' library

sampling flags (gen):
  --temp T            temperature; 0 = greedy (default 0)
  --top-k K           keep the K best tokens (default 40; 0 = off)
  --top-p P           keep the smallest set whose mass reaches P (default 0.9; 1 = off)
  --min-p P           drop tokens below P times the best one's probability (default 0 = off)
  --repeat-penalty R  penalty on recent tokens (default 1.1; 1 = off)
  --repeat-last-n N   how far the penalty looks back (default 64)
  --seed S            the sampler's seed (default: from the clock; printed)
"""


def fail(msg: str) -> "NoReturn":  # noqa: F821
    print(f"axon: {msg}", file=sys.stderr)
    sys.exit(2)


def parse_ids(text: str) -> Optional[List[int]]:
    parts = [p for p in re.split(r"[,\s]+", text.strip()) if p]
    if parts and all(p.isdigit() for p in parts):
        return [int(p) for p in parts]
    return None


class _Tok:
    def __init__(self, folder: str):
        self.tok = None
        path = os.path.join(folder, "tokenizer.json")
        if os.path.exists(path):
            try:
                from tokenizers import Tokenizer
                self.tok = Tokenizer.from_file(path)
            except Exception:  # the package is optional
                self.tok = None

    def encode(self, prompt: str) -> List[int]:
        ids = parse_ids(prompt)
        if ids is not None:
            return ids
        if self.tok is None:
            fail("the prompt must be token ids (\"1 2 3\"): this model folder has no usable tokenizer.json")
        return list(self.tok.encode(prompt).ids)

    def decode(self, ids: Sequence[int]) -> str:
        if self.tok is None:
            return " ".join(str(i) for i in ids)
        return self.tok.decode(list(ids))


def cmd_info(path: str) -> int:
    """Architecture, sizes and tensors of a model folder (src/cli.rs:499-532).  Everything
    printed comes from the model's spec and its configuration's own keys, whatever the
    architecture calls them."""
    from . import api
    from .cache.manager import bytes_per_token
    from .config.base import architecture_of
    from .engine.model import layer_cache_needs
    from .parts.spec import KvNeed, StateNeed
    from .weights.loader import expected_tensors
    from .weights.safetensors_io import Checkpoint

    m = api.load(path)
    c = m.config
    spec = architecture_of(c.to_dict()).build_spec(c)
    print(f"{path}: {spec.architecture}")
    print(f"  layers {len(spec.layers)} (schedule of {len(spec.schedule)} runs) / dim {spec.hidden_size} / "
          f"vocab {spec.vocab_size} / ctx {spec.max_positions}")
    skip = ("architectures", "model_type")
    print("  config: " + ", ".join(f"{k} {v:g}" if isinstance(v, float) else f"{k} {v}"
                                   for k, v in sorted(c.to_dict().items()) if k not in skip))
    kinds = {}
    for l in spec.layers:
        sig = l.block + "(" + ", ".join(f"{n}: {p.kind}" for n, p in sorted(l.parts.items())) + ")"
        kinds[sig] = kinds.get(sig, 0) + 1
    for sig, n in kinds.items():
        print(f"  {n} x {sig}")
    needs = [layer_cache_needs(spec.layers[e.layer]) if e.cache_of is None else {} for e in spec.schedule]
    groups = {}
    for entry in needs:
        for need in entry.values():
            groups[need] = groups.get(need, 0) + 1
    for need, n in groups.items():
        if isinstance(need, KvNeed):
            rows = f"keys of {need.head_dim}" + (f" and values of {need.value_dim}" if need.planes == 2 else " (one plane)")
            print(f"  cache: {n} runs keep {rows} x {need.kv_heads} kv heads per position"
                  + (f", the last {need.window} positions" if need.window else ""))
        elif isinstance(need, StateNeed):
            print(f"  cache: {n} runs keep state {list(need.shape)} {need.dtype} per request")
    import torch
    print(f"  cache bytes per position: {bytes_per_token(needs, torch.bfloat16):,} (bfloat16)")
    print(f"  {m.n_tensors} tensors, {m.n_params:,} parameters, {m.n_bytes:,} bytes")
    ck = Checkpoint(path)
    for name, decl in sorted(expected_tensors(spec).items()):
        info = ck.infos[name]
        print(f"  {name} -> {decl.kind} {info.dtype} {list(info.shape)}")
    ck.close()
    return 0


def _env_count(name: str) -> Optional[int]:
    v = os.environ.get(name, "").strip()
    if not v:
        return None
    if not v.isdigit():
        fail(f"{name} needs a whole number, got '{v}'")
    return int(v)


def _logits_of(net, cache, ids: List[int], top_k: int, tok: "_Tok", room: int) -> None:
    """``axon logits``: the top-k (id, logit, log-probability, text) after the prompt, or, under the
    oracle hooks of the reference (src/cli.rs:1088-1157), after several of its positions:

    ``AXON_LOGITS_ALL=N``     after each of the last N positions: the rest is fed in batched passes
                              (no logits), then one decode step each;
    ``AXON_LOGITS_PREFIX=N``  after each position from N - 1 on: the first N positions in batched
                              passes (position N - 1 is the last pass's last row), the rest one
                              decode step each (0 or 1: all decode steps);
    ``AXON_LOGITS_EACH=1``    with a prefix: every position from N - 1 on is the last row of its own
                              batched pass over the tokens up to it, on a fresh cache;
    ``AXON_LOGITS_NLL=1``     also ``nll <position> <next id> <-ln p>`` of the next token of the
                              sequence, in float64.
    """
    import numpy as np
    all_n = min(_env_count("AXON_LOGITS_ALL") or 0, len(ids))
    prefix = _env_count("AXON_LOGITS_PREFIX")
    nll = os.environ.get("AXON_LOGITS_NLL") == "1"
    each = os.environ.get("AXON_LOGITS_EACH") == "1" and prefix is not None

    def show(row32: "np.ndarray", pos: Optional[int]) -> None:
        row = row32.astype(np.float64)
        lse = float(np.log(np.sum(np.exp(row - row.max()))) + row.max())
        order = np.lexsort((-np.arange(len(row)), -row))[:top_k]
        if pos is not None:
            print(f"position {pos}:")
        for t in order:
            print(f"{int(t):>8}  {row[t]:>12.6f}  {row[t] - lse:>12.6f}  {tok.decode([int(t)])!r}")
        if nll and pos is not None and pos + 1 < len(ids):
            nxt = ids[pos + 1]
            print(f"nll {pos} {nxt} {lse - row[nxt]:.9f}")

    if not all_n and prefix is None:
        show(net.prefill_logits(ids, 0, cache), None)
        cache.close()
        return
    print(f"prompt ids ({len(ids)}): {list(ids)}")
    if prefix is not None:
        first, batched = min(max(prefix, 1), len(ids)) - 1, prefix > 1
    else:
        first, batched = len(ids) - all_n, False
    last = None
    if batched:
        last = net.prefill_logits(ids[:first + 1], 0, cache)
    elif first > 0:
        net.feed_batch(ids[:first], 0, cache)
    for p in range(first, len(ids)):
        if each and p > first:
            cache.close()
            cache = net.new_cache(room)
            last = net.prefill_logits(ids[:p + 1], 0, cache)
        elif not batched or p > first:
            last = net.forward(ids[p], p, cache)[0]
        show(last, p)
    cache.close()


def run_lm(args: List[str]) -> int:
    from . import api
    from .sampling.sampler import SampleArgs

    cmd = args[0]
    if len(args) < 3 and not (len(args) == 2 and os.environ.get("AXON_LOGITS_IDS")):
        fail(f"usage: axon {cmd} <model> \"<prompt>\" [{'-n 32' if cmd == 'gen' else '-k 10'}]")
    path = args[1]
    has_prompt = len(args) > 2 and not args[2].startswith("-")
    prompt = args[2] if has_prompt else ""
    rest = args[3:] if has_prompt else args[2:]
    n_gen, top_k, device, ctx, kv, dtype, verbose = 32, 10, os.environ.get("AXON_DEVICE", "cuda"), None, \
        os.environ.get("AXON_KV", "auto"), "bfloat16", False
    sargs = SampleArgs()
    i = 0
    while i < len(rest):
        f = rest[i]
        v = rest[i + 1] if i + 1 < len(rest) else None
        if f == "--verbose":
            verbose = True
            i += 1
            continue
        if SampleArgs.is_flag(f):
            try:
                sargs.set(f, v)
            except ValueError as e:
                fail(str(e))
        elif f in ("-n", "-k", "--ctx"):
            if v is None or not v.isdigit():
                fail(f"{f} needs a whole number, got {'nothing' if v is None else repr(v)}")
            if f == "-n":
                n_gen = int(v)
            elif f == "-k":
                top_k = int(v)
            elif cmd == "gen":
                ctx = int(v)
            else:
                fail(f"unknown argument '{f}' for {cmd}")
        elif f == "--device":
            device = v or ""
            if not device.startswith("cuda"):
                fail(f"--device {device!r}: this engine runs on cuda devices only")
        elif f == "--kv":
            kv = v or ""
        elif f == "--dtype":
            dtype = v or ""
        else:
            fail(f"unknown argument '{f}' for {cmd}")
        i += 2
    cfg = sargs.resolve(0.0)  # gen is greedy unless --temp says otherwise (src/cli.rs:936-940)
    if cfg is None and cmd == "gen" and sargs.any_besides_temp():
        print("axon: note: gen is greedy without --temp > 0; the sampling flags do nothing", file=sys.stderr)
    if cfg is not None:
        print(f"sampling:    temp {cfg.temp:g} top-k {cfg.top_k} top-p {cfg.top_p:g} min-p {cfg.min_p:g} "
              f"repeat-penalty {cfg.repeat_penalty:g} repeat-last-n {cfg.repeat_last_n} seed {cfg.seed}", file=sys.stderr)

    try:
        model = api.load(path)
    except (ValueError, OSError) as e:
        fail(str(e))
    tok = _Tok(path)
    env_ids = os.environ.get("AXON_LOGITS_IDS")
    if env_ids:
        seqs = [parse_ids(s) for s in env_ids.split(";") if s.strip()]
        if any(s is None for s in seqs):
            fail("AXON_LOGITS_IDS must hold token ids")
    else:
        seqs = [tok.encode(prompt)]
    if any(len(s) == 0 for s in seqs):
        fail("the prompt is empty")

    longest = max(len(s) for s in seqs)
    trained = model.ctx_len or (longest + n_gen + 1)
    if cmd == "gen":
        n_gen = max(0, min(n_gen, trained - longest))   # the trained context caps generation (src/cli.rs:811-824)
    room = ctx or (longest + n_gen + 1)
    t_load = time.perf_counter()
    try:
        opts = api.BackendOptions().device(device).max_ctx(room).dtype(dtype).kv(kv).parallel(2)
        net = api.Backend(model, opts)
    except (ValueError, RuntimeError) as e:
        fail(str(e))
    print(f"load:        {model.n_tensors} tensors, {model.n_bytes / 1e9:.2f} GB in {time.perf_counter() - t_load:.2f} s", file=sys.stderr)
    if verbose:
        import torch
        dev = net.engine.rt.device
        print(f"model:       {model.config}", file=sys.stderr)
        print(f"placed:      {device} {dtype}, ctx {net.ctx}, page size {opts._page_size}, "
              f"cache pool of {net.engine.cache.n_pages * opts._page_size} positions", file=sys.stderr)
        print(f"device:      {torch.cuda.memory_allocated(dev) / 1e9:.2f} GB in use after loading, "
              f"{torch.cuda.max_memory_allocated(dev) / 1e9:.2f} GB at the most", file=sys.stderr)

    import numpy as np
    for ids in seqs:
        cache = net.new_cache(room)
        t0 = time.perf_counter()
        if cmd == "logits":
            _logits_of(net, cache, ids, top_k, tok, room)
            continue
        logits = net.prefill_logits_device(ids, 0, cache)
        import torch
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        # generation stops before the checkpoint's end-of-sequence token(s), when it names any
        from .config.base import read_config_json
        eos = read_config_json(path).get("eos_token_id")
        stop = [int(e) for e in (eos if isinstance(eos, list) else [eos]) if isinstance(e, int)]
        out: List[int] = []
        st = api.generate(net, cache, ids, logits,
                          api.GenOpts(n_gen, stop, cfg), emit=out.append)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        print(tok.decode(st.ids))
        print(f"prompt eval: {len(ids)} tokens in {t1 - t0:.3f} s ({len(ids) / max(t1 - t0, 1e-9):.1f} tok/s)", file=sys.stderr)
        if st.passes:
            print(f"decode:      {st.passes} tokens in {t2 - t1:.3f} s ({st.passes / max(t2 - t1, 1e-9):.1f} tok/s)", file=sys.stderr)
        cache.close()
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    if not args or args[0] in ("-h", "--help"):
        print(USAGE, end="")
        return 0 if args else 2
    if args[0] in ("-V", "--version"):
        from . import __version__
        print(f"axon_b200 {__version__}")
        return 0
    if args[0] == "info":
        if len(args) < 2:
            fail("usage: axon info <model>")
        try:
            return cmd_info(args[1])
        except BrokenPipeError:
            raise
        except (ValueError, OSError) as e:
            fail(str(e))
    if args[0] in ("gen", "logits"):
        return run_lm(args)
    if os.path.isdir(args[0]):
        try:
            return cmd_info(args[0])
        except BrokenPipeError:
            raise
        except (ValueError, OSError) as e:
            fail(str(e))
    fail(f"unknown command '{args[0]}' (info, gen, logits)")


def run() -> int:
    """``main`` for the ``axon`` program: a reader that closes the pipe early (``| head``) ends it quietly."""
    try:
        rc = main()
        sys.stdout.flush()
        return rc
    except BrokenPipeError:
        try:
            sys.stdout.close()
        except BrokenPipeError:
            pass
        return 0


if __name__ == "__main__":
    sys.exit(run())
