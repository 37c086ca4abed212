"""The step function: one batch of (request, its next tokens) through the model.

A step takes entries ``(slot, tokens, want)``: portions of prompts beside single
decoded tokens, cut anywhere.  It runs exactly the tokens it is given as one
flattened batch against what earlier steps left in the cache, and returns the
float32 logits at the wanted places.  The reference splits this in two calls
(``feed_slot`` for a prompt portion of one sequence, ``step`` for one row per
request: src/lm.rs:290-302); here one call holds both, flattened to per-token
(position, slot) rows like the reference's ``Place::Rows``
(src/cuda/qwen2/batch.rs:649-671).

A refused step (bad slot, token out of range, no pages) raises before any kernel
runs, as ``StepError::Input`` does (src/cuda/qwen2/slots.rs:393-438).
"""

from __future__ import annotations

from collections.abc import Sequence as SequenceABC
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import PagedCache
from ..kernels import lib
from ..parts.base import Runtime, StepContext
from .model import DecoderModel


class StepError(ValueError):
    """The step was refused; nothing ran."""


class OutOfPages(StepError):
    """A request's next tokens need more pages than are free."""


class DeviceFault(RuntimeError):
    """A kernel reported that it could not do its work (a bounded wait inside it gave up, or
    with checked tables a block-table entry lay outside the pool).  What the step returned
    is not to be trusted; the reference treats a device error as fatal too
    (``StepError::Device``, src/lm.rs:262-270)."""


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    #: places among ``tokens`` whose logits are wanted
    want: Sequence[int] = field(default_factory=tuple)


class _LazyPositions(SequenceABC):
    """The position of every token of a step, worked out when a part first asks (parts that run on
    the host side of a step do; the kernels read positions on the device)."""

    def __init__(self, seg_q_len: List[int], seg_kv_len: List[int]):
        self._q, self._kv, self._all = seg_q_len, seg_kv_len, None

    def _list(self) -> List[int]:
        if self._all is None:
            self._all = [p for n, kv in zip(self._q, self._kv) for p in range(kv - n, kv)]
        return self._all

    def __len__(self) -> int:
        return sum(self._q)

    def __getitem__(self, i):
        return self._list()[i]

    def __iter__(self):
        return iter(self._list())

    def __eq__(self, other):
        return list(self) == list(other)


class Engine:
    """A model, its cache, and the step function over both."""

    def __init__(self, model: DecoderModel, cache: PagedCache, max_step_tokens: int = 8192):
        self.model, self.cache, self.rt = model, cache, model.rt
        self.max_step_tokens = max_step_tokens
        self._staging: List[torch.Tensor] = []
        self._events: List[Optional[torch.cuda.Event]] = []
        self._turn = 0
        #: decode-only steps replay captured CUDA graphs (one per batch size, number of wanted
        #: rows and attention split count), as the reference captures its decode step
        #: (src/cuda/qwen2.rs:2978-3011; per step shape: src/cuda/qwen2/slots.rs:722-785)
        self.cuda_graphs = bool(model.graph_safe)
        #: a prompt portion of one request whose size comes a second time is captured too (chunked
        #: prefill repeats its chunk size): the host's share of such a step, about 12 us a launch,
        #: is what bounds prompts of a few hundred tokens
        self.prefill_graphs = bool(model.graph_safe)
        self._shape_seen = {}
        self.graph_max_batch = 256
        self.graph_cache_size = 64
        self._graphs = {}
        self._graph_generation = self.rt.generation
        #: steps run, for reports
        self.steps = 0
        # the metadata buffer of eager steps at its largest from the start: a buffer that grows later
        # moves, and every captured graph is dropped when any scratch buffer moves
        self.rt.buffer("step_meta", (4 * max_step_tokens + 6 * cache.max_slots,), torch.int32)

    # -- requests ---------------------------------------------------------
    def open_request(self) -> int:
        slot = self.cache.open()
        if slot < 0:
            raise StepError(f"all {self.cache.max_slots} request slots are taken")
        return slot

    def close_request(self, slot: int) -> None:
        self.cache.close(slot)

    # -- the step ---------------------------------------------------------
    def _stage(self, n_ints: int) -> torch.Tensor:
        """A pinned host buffer that no copy in flight still reads (two take turns)."""
        if not self._staging:
            self._staging = [torch.empty(0, dtype=torch.int32), torch.empty(0, dtype=torch.int32)]
            self._events = [None, None]
        i = self._turn
        self._turn ^= 1
        if self._events[i] is not None:
            self._events[i].synchronize()
        if self._staging[i].numel() < n_ints:
            self._staging[i] = torch.empty(max(n_ints, 4096), dtype=torch.int32).pin_memory()
        self._cur = i
        return self._staging[i]

    def step(self, entries: Sequence[StepEntry], greedy: bool = False) -> Optional[torch.Tensor]:
        """Run the entries' tokens; the float32 logits at the wanted places, ``[wanted, vocab]``.
        With ``greedy`` the largest logit of each wanted place is picked on the device in the same
        launch (the same CUDA graph for steps of single tokens) and the int32 ids come back instead.
        Both live in buffers of the engine: valid until the next step."""
        if not entries:
            return None
        staged = self._stage_single_tokens(entries)
        if staged is not None:
            return self._run(*staged, greedy=greedy)
        try:
            slots = np.fromiter((e.slot for e in entries), dtype=np.int32, count=len(entries))
            tok_off = np.zeros(len(entries) + 1, dtype=np.int32)
            want_off = np.zeros(len(entries) + 1, dtype=np.int32)
            np.cumsum([len(e.tokens) for e in entries], out=tok_off[1:])
            np.cumsum([len(e.want) for e in entries], out=want_off[1:])
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64).reshape(-1) for e in entries])
            wants = np.concatenate([np.asarray(list(e.want), dtype=np.int64).reshape(-1) for e in entries])
            if tokens.size and (tokens.min() < -2**31 or tokens.max() >= 2**31):
                raise OverflowError
            if wants.size and (wants.min() < -2**31 or wants.max() >= 2**31):
                raise OverflowError
        except (TypeError, ValueError, OverflowError):
            self._explain(entries)
            raise StepError("the step's entries are not lists of whole numbers")
        return self.step_flat(slots, tok_off, tokens.astype(np.int32), want_off, wants.astype(np.int32), greedy=greedy,
                              _entries=entries)

    def step_flat(self, slots, tok_off, tokens, want_off, wants, greedy: bool = False, _entries=None) -> Optional[torch.Tensor]:
        """``step`` for callers that hold the batch as arrays already (the scheduler's plans): entry
        ``i`` is the request in ``slots[i]`` with tokens ``tokens[tok_off[i]:tok_off[i+1]]`` and wanted
        places ``wants[want_off[i]:want_off[i+1]]`` (int32 arrays).  Checked and laid out for the
        device by the cache manager in one native call."""
        s = len(slots)
        if s == 0:
            return None
        n, n_want = int(tok_off[-1]), int(want_off[-1])
        stage = self._stage(3 * n + 6 * s + n_want)
        rc, bad, n, s, n_want, decode_only, total = self.cache.manager.stage_step(
            slots, tok_off, tokens, want_off, wants, self.model.spec.vocab_size, self.max_step_tokens, stage.numpy())
        if rc != 0:
            self._turn ^= 1                          # the staging buffer was not used
            entries = _entries if _entries is not None else [
                StepEntry(int(slots[i]), tokens[tok_off[i]:tok_off[i + 1]].tolist(), wants[want_off[i]:want_off[i + 1]].tolist())
                for i in range(s)]
            if rc == 2:
                e = entries[bad]
                start = self.cache.length(e.slot)
                raise OutOfPages(f"slot {e.slot}: no pages for positions {start}..{start + len(e.tokens) - 1}")
            self._explain(entries)
            raise StepError("the step was refused")
        seg = stage.numpy()[3 * n:3 * n + 4 * s].reshape(4, s)
        seg_slot, seg_q_start, seg_q_len, seg_kv_len = (row.tolist() for row in seg)
        return self._run(None, None, stage, total, n, s, n_want, bool(decode_only), seg_slot, seg_q_start, seg_q_len,
                         seg_kv_len, _LazyPositions(seg_q_len, seg_kv_len), greedy=greedy)

    def _explain(self, entries: Sequence[StepEntry]) -> None:
        """Raise the :class:`StepError` that says what is wrong with a step the native staging refused."""
        cache, vocab = self.cache, self.model.spec.vocab_size
        seen = set()
        n = 0
        for e in entries:
            if not cache.manager.is_open(e.slot):
                raise StepError(f"slot {e.slot} is not open")
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if len(e.tokens) == 0:
                raise StepError(f"slot {e.slot}: an entry needs at least one token")
            for t in e.tokens:
                if not (isinstance(t, (int, np.integer)) and 0 <= int(t) < vocab):
                    raise StepError(f"slot {e.slot}: token {t} is outside the vocabulary of {vocab}")
            for w in e.want:
                if not (isinstance(w, (int, np.integer)) and 0 <= int(w) < len(e.tokens)):
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside its {len(e.tokens)} tokens")
            if cache.length(e.slot) + len(e.tokens) > cache.max_positions:
                raise StepError(f"slot {e.slot}: {cache.length(e.slot) + len(e.tokens)} positions exceed the "
                                f"context of {cache.max_positions}")
            n += len(e.tokens)
        if n > self.max_step_tokens:
            raise StepError(f"{n} tokens exceed the step limit of {self.max_step_tokens}")

    def _stage_single_tokens(self, entries: Sequence[StepEntry]):
        """A step of one token per request given as entries: the lists go to the cache manager as
        they are (no arrays are built).  None when the step is not of that kind or something about
        it is irregular: the general path then finds the words for it."""
        s = len(entries)
        slots, toks, wanted = [], [], []
        for e in entries:
            if len(e.tokens) != 1:
                return None
            w = e.want
            if len(w) > 1 or (len(w) == 1 and w[0] != 0):
                return None
            slots.append(e.slot); toks.append(e.tokens[0]); wanted.append(len(w))
        n_want = sum(wanted)
        total = 9 * s + n_want
        stage = self._stage(total)
        try:
            rc, _ = self.cache.manager.stage_decode(slots, toks, wanted, self.model.spec.vocab_size, stage.numpy())
        except (TypeError, ValueError, OverflowError):
            rc = 1                                   # ids that are no plain integers
        if rc != 0:
            self._turn ^= 1                          # the staging buffer was not used
            return None
        buf = stage.numpy()
        starts = buf[s:2 * s].tolist()
        return (entries, starts, stage, total, s, s, n_want, True, slots, list(range(s)), [1] * s,
                buf[6 * s:7 * s].tolist(), starts)

    def _run(self, entries, starts, stage, total, n, s, n_want, decode_only, seg_slot, seg_q_start, seg_q_len,
             seg_kv_len, host_positions, greedy: bool = False) -> Optional[torch.Tensor]:
        """Copy the staged step to the device, run the model, commit the new lengths."""
        cache = self.cache
        # A decode-only step of a shape seen before replays a captured CUDA graph: every
        # kernel argument that depends on the host is in the key, everything else
        # (tokens, positions, slots, lengths, block tables) is read from device memory.
        graph_key = None
        if self.cuda_graphs and decode_only and n <= self.graph_max_batch:
            # what the parts' launches take from the host beside the batch shape (the attention's
            # split count follows the longest context) is part of the key
            probe = StepContext(rt=self.rt, n_tokens=n, tokens=None, positions=None, token_slot=None,
                                seg_slot=seg_slot, seg_q_start=seg_q_start, seg_q_len=seg_q_len, seg_kv_len=seg_kv_len)
            graph_key = (n, n_want, self.model.graph_key(probe), bool(greedy))
        elif self.cuda_graphs and self.prefill_graphs and s == 1 and n > 1:
            # one request's portion: what the host works out for it does not depend on where in
            # the request it lies (positions, lengths and tables are read from device memory),
            # except what the parts report in their keys (a portion short enough for the
            # attention's decode shape takes its split count from the context's length)
            probe = StepContext(rt=self.rt, n_tokens=n, tokens=None, positions=None, token_slot=None,
                                seg_slot=seg_slot, seg_q_start=seg_q_start, seg_q_len=seg_q_len, seg_kv_len=seg_kv_len)
            key = ("portion", n, n_want, self.model.graph_key(probe), bool(greedy))
            seen = self._shape_seen.get(key, 0) + 1
            if len(self._shape_seen) > 4096:
                self._shape_seen.clear()
            self._shape_seen[key] = seen
            if seen >= 2:
                graph_key = key
        # (a graph holds the address of the metadata it was captured with: one buffer per kind and shape)
        meta_name = "step_meta" if graph_key is None else f"step_meta_graph_{'p' if graph_key[0] == 'portion' else 'd'}_{n}_{n_want}"
        dev = self.rt.buffer(meta_name, (total,), torch.int32)
        dev.copy_(stage[:total], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[self._cur] = ev
        cache.sync_tables()

        def context() -> StepContext:
            return StepContext(
                rt=self.rt, n_tokens=n, tokens=dev[0:n], positions=dev[n:2 * n], token_slot=dev[2 * n:3 * n],
                seg_slot=seg_slot, seg_q_start=seg_q_start, seg_q_len=seg_q_len, seg_kv_len=seg_kv_len,
                segments=dev[3 * n:3 * n + 4 * s].view(4, s),
                unit_items=dev[total - 2 * s: total] if decode_only else None,
                host_positions=host_positions)
        want_rows = dev[3 * n + 4 * s: 3 * n + 4 * s + n_want] if n_want else None

        if graph_key is None:
            logits = self.model.forward(context(), cache, want_rows, n_want)
            if greedy and logits is not None:
                from ..kernels import ops
                picks = self.rt.buffer("greedy_picks", (n_want,), torch.int32)
                ops.argmax(logits, picks)
                logits = picks
        else:
            logits = self._graph_step(graph_key, context, want_rows, n_want, greedy)
        if decode_only:
            cache.manager.commit_decode(seg_slot)
        else:
            cache.manager.commit_step(stage.numpy()[3 * n:3 * n + 4 * s], s)
        self.steps += 1
        if cache.checks_tables:
            bad = cache.fault()
            if bad is not None:
                raise DeviceFault(f"a kernel met block-table entry {bad}, outside the pool of {cache.n_pages} pages "
                                  "(it used the sink page instead; the step's results are void)")
        return logits

    def check_device(self) -> None:
        """Raise :class:`DeviceFault` if a bounded wait inside a tensor-core kernel ever gave up.
        Synchronises the device, so callers ask where they wait for results anyway (at a
        request's end, every so many steps)."""
        if self.rt.precise:
            return
        from ..kernels import fast
        for what, status in (("product", fast.gemm_tc_status()), ("attention", fast.attention_tc_status())):
            if status:
                raise DeviceFault(f"a tensor-core {what} kernel gave up waiting (status {status}: 1 + the role that "
                                  "waited: 0 loads, 1 MMA, 2 epilogue; 100: misaligned shared memory)")

    def _graph_step(self, key, context, want_rows, n_want, greedy: bool = False) -> Optional[torch.Tensor]:
        """Run a decode-only step through its CUDA graph, capturing it the first time.
        The logits live in a buffer of the graph: they are valid until the next step."""
        if self._graph_generation != self.rt.generation:
            self._graphs.clear()              # a scratch buffer moved: captured addresses are stale
            self._graph_generation = self.rt.generation
        out = self.rt.buffer(f"graph_logits_{n_want}", (max(n_want, 1), self.model.spec.vocab_size), torch.float32)
        picks = self.rt.buffer(f"graph_picks_{n_want}", (max(n_want, 1),), torch.int32) if greedy else None
        result = (picks if greedy else out)[:n_want] if n_want else None

        def run() -> None:
            self.model.forward(context(), self.cache, want_rows, n_want, logits_out=out)
            if greedy and n_want:
                from ..kernels import ops
                ops.argmax(out[:n_want], picks[:n_want])

        entry = self._graphs.get(key)
        if entry is not None:
            graph, launches = entry
            graph.replay()
            lib.add_launches(launches)
            return result
        # first time: run it plainly (this also sizes every scratch buffer), then record it
        run()
        if self._graph_generation == self.rt.generation:
            try:
                graph = torch.cuda.CUDAGraph()
                before = lib.launch_count()
                with torch.cuda.graph(graph):
                    run()
                launches = lib.launch_count() - before
                lib.add_launches(-launches)       # recorded, not run
                if self._graph_generation == self.rt.generation:
                    if len(self._graphs) >= self.graph_cache_size:
                        self._graphs.pop(next(iter(self._graphs)))
                    self._graphs[key] = (graph, launches)
            except RuntimeError:
                # capture failed (for instance a part that allocates): steps of this kind stay eager
                if key[0] == "portion":
                    self.prefill_graphs = False
                else:
                    self.cuda_graphs = False
        else:
            self._graph_generation = self.rt.generation
        return result
