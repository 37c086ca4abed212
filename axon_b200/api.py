"""The programming entry point, in the manner of the reference's library API
(src/lib.rs:19-35, 90-127; src/lm.rs:54-229, 912-1025; src/generate.rs:29-220):

    model = axon_b200.load("models/tiny")
    net = axon_b200.Backend(model, axon_b200.BackendOptions().max_ctx(512))
    cache = net.new_cache(512)
    logits = net.prefill_logits(ids, 0, cache)
    st = axon_b200.generate(net, cache, ids, logits, axon_b200.GenOpts.greedy(16, stop))
    print(st.ids)

``Backend.generate_batch`` runs many requests at once through the continuous-batching
scheduler.  Token ids go in and come out on the host; everything between runs on the
GPU through the engine's own step function.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field, replace
from typing import Callable, Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from .config.base import ModelConfig, architecture_of, load_config
from .engine.build import build_engine, parse_dtype
from .engine.step import Engine, StepEntry, StepError
from .kernels import lib, ops
from .sampling.sampler import RowSampler, SampleCfg, pick_tokens
from .weights.loader import WeightsError, check_checkpoint
from .weights.safetensors_io import Checkpoint

#: most tokens of one request per prefill pass (the reference feeds prompts in passes too:
#: PREFILL_BATCH, src/generate.rs:12; src/cuda/qwen2.rs:139-145)
PREFILL_BATCH = 4096


@dataclass(frozen=True)
class Model:
    """A model folder that has been read and checked, not yet placed on a device."""

    path: str
    config: ModelConfig
    n_tensors: int
    n_params: int
    n_bytes: int
    #: the longest request the model is made for (its spec's ``max_positions``)
    ctx_len: int = 0


def load(path: str, device: str = "cuda") -> Model:
    """Read ``path/config.json``, pick the architecture, and check every tensor of the
    checkpoint against it (names, shapes, dtypes) without copying any data.  An error
    names the folder and says why it cannot be read or run (src/lib.rs:112-127)."""
    config = load_config(path)
    spec = architecture_of(config.to_dict()).build_spec(config)
    ck = Checkpoint(path)
    try:
        want = check_checkpoint(ck, spec, path)
        have = ck.infos
        params = sum(int(np.prod(have[n].shape)) for n in want)
        nbytes = sum(have[n].end - have[n].begin for n in want)
    finally:
        ck.close()
    return Model(path, config, len(want), params, nbytes, int(spec.max_positions))


@dataclass(frozen=True)
class BackendOptions:
    """How a model is placed.  Setters return new options, as the reference's do
    (src/lm.rs:912-993)."""

    _device: str = "cuda:0"
    _max_ctx: int = 4096
    _dtype: str = "bfloat16"
    _page_size: int = 16
    _parallel: int = 16
    _kv_tokens: Optional[int] = None
    _step_tokens: int = 8192

    def device(self, device: str) -> "BackendOptions":
        """Where the model runs: a CUDA device (there is no CPU path)."""
        return replace(self, _device="cuda:0" if device == "cuda" else device)

    def max_ctx(self, max_ctx: int) -> "BackendOptions":
        """Room for requests of up to ``max_ctx`` positions (default 4096)."""
        return replace(self, _max_ctx=int(max_ctx))

    def dtype(self, dtype: str) -> "BackendOptions":
        """``bfloat16`` (serving) or ``float32`` (every kernel in true 32-bit)."""
        parse_dtype(dtype)
        return replace(self, _dtype=dtype)

    def kv(self, kv: str) -> "BackendOptions":
        """The cache type.  The cache always has the model's dtype here (no quantized
        caches); ``bf16``/``f32``/``auto`` are accepted when they agree with it."""
        if kv not in ("auto", "bf16", "bfloat16", "f32", "float32"):
            raise ValueError(f"KV type '{kv}' is not supported (bf16 with a bfloat16 model, f32 with a float32 one)")
        if kv != "auto" and parse_dtype(kv) != parse_dtype(self._dtype):
            raise ValueError(f"the cache has the model's dtype ({self._dtype}); '{kv}' differs")
        return self

    def page_size(self, n: int) -> "BackendOptions":
        return replace(self, _page_size=int(n))

    def parallel(self, n: int) -> "BackendOptions":
        """Requests that may be live at once (the reference's 16 slots, src/serve.rs:2148)."""
        return replace(self, _parallel=int(n))

    def kv_tokens(self, n: int) -> "BackendOptions":
        """Positions the cache pool holds over all live requests.  Default: what the device has
        free once the weights are placed, and no more than ``parallel`` requests of ``max_ctx``
        need (the reference sizes its pool so: src/serve.rs:2411-2449)."""
        return replace(self, _kv_tokens=int(n))

    def step_tokens(self, n: int) -> "BackendOptions":
        """Most tokens one step runs (the scheduler's budget and the prefill pass size)."""
        return replace(self, _step_tokens=int(n))


class BackendCache:
    """One sequence's place in the cache (a request slot); ``close`` gives it back."""

    def __init__(self, net: "Backend", ctx: int):
        self.net, self.ctx = net, ctx
        self.slot = net.engine.open_request()

    def __len__(self) -> int:
        return self.net.engine.cache.length(self.slot) if self.slot >= 0 else 0

    def close(self) -> None:
        if self.slot >= 0:
            self.net.engine.close_request(self.slot)
            self.slot = -1

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


@dataclass
class GenStats:
    """What ``generate`` did (src/generate.rs:29-45)."""

    ids: List[int] = field(default_factory=list)   # the emitted tokens (a stop token excluded)
    passes: int = 0                                # weight passes
    decided: int = 0                               # tokens picked from logits, a final stop token included
    forward: tuple = (0, 0.0)                      # (count, seconds) of decode passes


@dataclass
class GenOpts:
    n_gen: int
    stop: Sequence[int] = ()
    sample: Optional[SampleCfg] = None

    @staticmethod
    def greedy(n_gen: int, stop: Sequence[int] = ()) -> "GenOpts":
        """Greedy decoding of up to ``n_gen`` tokens, stopping before any of ``stop``."""
        return GenOpts(n_gen, tuple(stop), None)

    @staticmethod
    def sampled(n_gen: int, stop: Sequence[int], cfg: SampleCfg) -> "GenOpts":
        return GenOpts(n_gen, tuple(stop), cfg)


class Backend:
    """A model placed on a GPU (src/lm.rs:995-1025)."""

    def __init__(self, model: Union[Model, str], options: Optional[BackendOptions] = None, *,
                 engine: Optional[Engine] = None):
        o = options or BackendOptions()
        self.options = o
        if engine is None:
            path = model.path if isinstance(model, Model) else model
            engine = build_engine(path, dtype=o._dtype, device=o._device, page_size=o._page_size,
                                  max_tokens=o._kv_tokens, max_slots=o._parallel,
                                  max_positions=o._max_ctx, max_step_tokens=o._step_tokens)
        self.engine = engine
        self.config = engine.config

    @property
    def vocab(self) -> int:
        return self.engine.model.spec.vocab_size

    @property
    def ctx(self) -> int:
        return self.engine.cache.max_positions

    def new_cache(self, ctx: Optional[int] = None) -> BackendCache:
        ctx = ctx or self.ctx
        if ctx > self.ctx:
            raise ValueError(f"a cache of {ctx} positions exceeds the context this backend was made for ({self.ctx})")
        return BackendCache(self, ctx)

    # -- one sequence -------------------------------------------------------
    def _check_pos(self, pos: int, cache: BackendCache) -> None:
        if pos != len(cache):
            raise StepError(f"position {pos} does not continue the cache, which holds {len(cache)} positions")

    def feed_batch(self, ids: Sequence[int], start: int, cache: BackendCache) -> None:
        """Put ``ids`` into cache positions ``start..`` without computing logits."""
        self._check_pos(start, cache)
        step = min(PREFILL_BATCH, self.engine.max_step_tokens)
        for at in range(0, len(ids), step):
            self.engine.step([StepEntry(cache.slot, ids[at:at + step], [])])

    def prefill_logits(self, ids: Sequence[int], start: int, cache: BackendCache) -> np.ndarray:
        """Feed ``ids`` at positions ``start..`` and return the logits after the last one."""
        return self.prefill_logits_device(ids, start, cache).cpu().numpy()

    def prefill_logits_device(self, ids: Sequence[int], start: int, cache: BackendCache) -> torch.Tensor:
        if not len(ids):
            raise StepError("prefill needs at least one token")
        self._check_pos(start, cache)
        step = min(PREFILL_BATCH, self.engine.max_step_tokens)
        logits = None
        for at in range(0, len(ids), step):
            part = ids[at:at + step]
            last = at + step >= len(ids)
            logits = self.engine.step([StepEntry(cache.slot, part, [len(part) - 1] if last else [])])
        return logits[0]

    def forward(self, token: int, pos: int, cache: BackendCache) -> np.ndarray:
        """One decode step: the logits after ``token`` at position ``pos``."""
        return self.forward_device(token, pos, cache).cpu().numpy()

    def forward_device(self, token: int, pos: int, cache: BackendCache) -> torch.Tensor:
        self._check_pos(pos, cache)
        return self.engine.step([StepEntry(cache.slot, [int(token)], [0])])

    def forward_argmax(self, token: int, pos: int, cache: BackendCache) -> int:
        """One decode step and the greedy pick, chosen on the device (4 bytes come back)."""
        logits = self.forward_device(token, pos, cache)
        best = torch.empty(1, dtype=torch.int32, device=logits.device)
        ops.argmax(logits, best)
        return int(best.item())

    # -- many sequences -----------------------------------------------------
    def decode_batch(self, tokens: Sequence[int], caches: Sequence[BackendCache]) -> List[int]:
        """One decode step for several sequences at once: ``tokens[i]`` goes to the next
        position of ``caches[i]``; the greedy picks, chosen on the device, come back as
        host integers (the batch form of ``forward_argmax``)."""
        if len(tokens) != len(caches):
            raise StepError("decode_batch needs one token per cache")
        best = self.engine.step([StepEntry(c.slot, [int(t)], [0]) for c, t in zip(caches, tokens)], greedy=True)
        picks = best.tolist()
        # a kernel that gave up on a wait returns garbage without an error: ask now and then,
        # where the host has just waited for the device anyway
        if self.engine.steps % 512 == 0:
            self.engine.check_device()
        return picks

    def generate_batch(self, prompts: Sequence[Sequence[int]], n_gen: Union[int, Sequence[int]],
                       stop: Sequence[int] = (), sample: Union[None, SampleCfg, Sequence[Optional[SampleCfg]]] = None,
                       on_token: Optional[Callable[[int, int], None]] = None,
                       prefill_chunk: int = 0) -> List[List[int]]:
        """Generate for every prompt with continuous batching; the tokens of each, in
        order of the prompts.  See :class:`axon_b200.engine.serve.BatchRunner`."""
        from .engine.serve import BatchRunner
        runner = BatchRunner(self.engine, max_batch_tokens=self.engine.max_step_tokens,
                             max_running=self.engine.cache.max_slots, prefill_chunk=prefill_chunk)
        n = [n_gen] * len(prompts) if isinstance(n_gen, int) else list(n_gen)
        cfgs = list(sample) if isinstance(sample, (list, tuple)) else [sample] * len(prompts)
        for i, p in enumerate(prompts):
            runner.add(i, p, n[i], stop, cfgs[i])
        outs = runner.run(on_token)
        return [outs[i] for i in range(len(prompts))]


def argmax(logits: np.ndarray) -> int:
    """The last index among equal maxima; NaN only when everything is NaN
    (src/generate.rs:222-263)."""
    l = np.asarray(logits)
    if np.all(np.isnan(l)):
        return len(l) - 1
    m = np.nanmax(l)
    return int(np.nonzero(l == m)[0][-1])


def generate(net: Backend, cache: BackendCache, prompt: Sequence[int], logits, opts: GenOpts,
             emit: Optional[Callable[[int], None]] = None) -> GenStats:
    """Decode up to ``opts.n_gen`` tokens after ``prompt``, whose tokens fill cache
    positions ``0..len(prompt)``; ``logits`` is the prediction after the prompt.  Every
    token goes to ``emit`` as it is picked (src/generate.rs:106-220; sampled:
    src/sample.rs:574-654)."""
    st = GenStats()
    stop = set(int(s) for s in opts.stop)
    sampler = RowSampler(opts.sample, prompt) if opts.sample is not None else None
    dev = net.engine.rt.device
    row = torch.as_tensor(np.asarray(logits), dtype=torch.float32, device=dev).reshape(1, -1) \
        if not isinstance(logits, torch.Tensor) else logits.reshape(1, -1)
    hist_len = len(prompt)
    count, secs = 0, 0.0
    picks = 0
    while len(st.ids) < opts.n_gen:
        if sampler is None:
            best = torch.empty(1, dtype=torch.int32, device=dev)
            ops.argmax(row.contiguous(), best)
            nxt = int(best.item())
        else:
            nxt = pick_tokens(row.contiguous(), [sampler])[0]      # (it copies what it changes)
        picks += 1
        if nxt in stop:
            break
        st.ids.append(nxt)
        if emit is not None:
            emit(nxt)
        if len(st.ids) >= opts.n_gen:
            break
        t0 = time.perf_counter()
        row = net.forward_device(nxt, hist_len, cache)
        hist_len += 1
        count += 1
        secs += time.perf_counter() - t0
        st.passes += 1
    st.decided = picks
    st.forward = (count, secs)
    net.engine.check_device()
    return st
