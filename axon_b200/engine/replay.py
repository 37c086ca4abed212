"""Replaying a trace of steps through an engine (the loop behind ``bin/trace_run``).

A trace step is ``{"step": k, "entries": [{"id", "tokens", "want"}], "end": [ids]}``.
Request ids are mapped to cache slots as they first appear and given back when a
step names them in ``end``.
"""

from __future__ import annotations

from typing import Any, Dict, Iterable, Iterator, Mapping, Optional, Tuple

import torch

from .step import Engine, StepEntry


class Replayer:
    def __init__(self, engine: Engine):
        self.engine = engine
        self.slots: Dict[Any, int] = {}

    def run_step(self, rec: Mapping[str, Any]) -> Optional[torch.Tensor]:
        """Run one trace step; the float32 logits ``[wanted, vocab]`` on the device, or
        None when nothing was wanted."""
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in self.slots:
                self.slots[rid] = self.engine.open_request()
            entries.append(StepEntry(self.slots[rid], e["tokens"], e.get("want", [])))
        logits = self.engine.step(entries) if entries else None
        for rid in rec.get("end", []):
            if rid in self.slots:
                self.engine.close_request(self.slots.pop(rid))
        return logits

    def run(self, steps: Iterable[Mapping[str, Any]]) -> Iterator[Tuple[Any, Optional[torch.Tensor]]]:
        for rec in steps:
            yield rec["step"], self.run_step(rec)
