"""Continuous batching: the scheduler (host library) decides, the step function runs,
the sampler picks, and the picks go back to the scheduler.

One iteration, after the reference's ``Batch::step`` (src/serve/engine.rs:1999-2181):
plan (decode rows first, then prompt portions under the token budget, preempting the
youngest request when pages run out), one mixed step, one token per request whose
last known token was in the step, finish on a stop token or on length.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
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
        #: tokens run over all steps (prompt portions and decoded tokens), for reports
        self.step_tokens = 0

    def add(self, rid: int, prompt: Sequence[int], n_gen: int, stop: Sequence[int] = (),
            sample: Optional[SampleCfg] = None) -> None:
        vocab = self.engine.model.spec.vocab_size
        for t in prompt:
            if not (0 <= int(t) < vocab):
                raise ValueError(f"request {rid}: token {t} is outside the vocabulary of {vocab}")
        self.sched.add(int(rid), [int(t) for t in prompt], int(n_gen), [int(s) for s in stop])
        self.samplers[int(rid)] = RowSampler(sample, prompt)

    def step(self, on_token: Optional[Callable[[int, int], None]] = None) -> List[int]:
        """One scheduler iteration; the ids of requests that finished in it.  The plan goes to the
        step function as arrays (no Python object per entry or token); when every row that wants
        a token is greedy, the pick is part of the step (of its CUDA graph) and one small copy
        brings the ids back."""
        plan = self.sched.plan()
        self.preemptions += len(plan.preempted)
        ids, slots, tok_off, tokens, want_off, wants = plan.flat()
        wanted = ids[np.diff(want_off) > 0].tolist()
        self.step_tokens += int(tok_off[-1])
        all_greedy = all(self.samplers[r].greedy for r in wanted)
        out = self.engine.step_flat(slots, tok_off, tokens, want_off, wants, greedy=all_greedy and bool(wanted))
        if not wanted:
            toks = []
        elif all_greedy:
            toks = out.tolist()
            for r, t in zip(wanted, toks):
                self.samplers[r].history.append(t)
        else:
            toks = pick_tokens(out, [self.samplers[r] for r in wanted])
        done = self.sched.commit_in_order(plan, np.asarray(toks, dtype=np.int32))
        self.steps += 1
        finished = []
        if on_token is not None:
            stopped = {d.id for d in done if d.finish == lib.host().Finish.Stop}
            for rid, tok in zip(wanted, toks):
                if rid not in stopped:
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
