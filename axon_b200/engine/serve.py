"""Continuous batching: the scheduler (host library) decides, the step function runs,
the sampler picks, and the picks go back to the scheduler.

One iteration, after the reference's ``Batch::step`` (src/serve/engine.rs:1999-2181):
plan (decode rows first, then prompt portions under the token budget, preempting the
youngest request when pages run out), one mixed step, one token per request whose
last known token was in the step, finish on a stop token or on length.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..kernels import lib
from ..sampling.sampler import RowSampler, SampleCfg, pick_tokens
from .step import Engine, StepEntry


class BatchRunner:
    def __init__(self, engine: Engine, max_batch_tokens: int = 2048, max_running: int = 16,
                 prefill_chunk: int = 0):
        host = lib.host()
        self.engine = engine
        max_running = min(max_running, engine.cache.max_slots)
        self.sched = host.Scheduler(engine.cache.manager,
                                    host.SchedulerConfig(max(max_batch_tokens, max_running), max_running, prefill_chunk))
        self.samplers: Dict[int, RowSampler] = {}
        self.outputs: Dict[int, List[int]] = {}
        self.finish: Dict[int, str] = {}
        self.preemptions = 0
        self.steps = 0

    def add(self, rid: int, prompt: Sequence[int], n_gen: int, stop: Sequence[int] = (),
            sample: Optional[SampleCfg] = None) -> None:
        vocab = self.engine.model.spec.vocab_size
        for t in prompt:
            if not (0 <= int(t) < vocab):
                raise ValueError(f"request {rid}: token {t} is outside the vocabulary of {vocab}")
        self.sched.add(int(rid), [int(t) for t in prompt], int(n_gen), [int(s) for s in stop])
        self.samplers[int(rid)] = RowSampler(sample, prompt)

    def step(self, on_token: Optional[Callable[[int, int], None]] = None) -> List[int]:
        """One scheduler iteration; the ids of requests that finished in it."""
        plan = self.sched.plan()
        self.preemptions += len(plan.preempted)
        entries, wanted = [], []
        for e in plan.entries:
            entries.append(StepEntry(e.slot, e.tokens, [len(e.tokens) - 1] if e.want_logits else []))
            if e.want_logits:
                wanted.append(e.id)
        logits = self.engine.step(entries)
        picked: Dict[int, int] = {}
        if wanted:
            toks = pick_tokens(logits, [self.samplers[r] for r in wanted])
            picked = dict(zip(wanted, toks))
        done = self.sched.commit(plan, picked)
        self.steps += 1
        finished = []
        done_ids = {d.id: d.finish for d in done}
        if on_token is not None:
            for rid, tok in picked.items():
                if not (rid in done_ids and done_ids[rid] == lib.host().Finish.Stop):
                    on_token(rid, tok)
        if done:
            self.engine.check_device()      # before a request's tokens are handed out as good
        for d in done:
            self.outputs[d.id] = list(self.sched.take_output(d.id))
            self.finish[d.id] = d.finish.name
            self.samplers.pop(d.id, None)
            finished.append(d.id)
        return finished

    def run(self, on_token: Optional[Callable[[int, int], None]] = None) -> Dict[int, List[int]]:
        while not self.sched.idle():
            self.step(on_token)
        return self.outputs
