"""Sampling: greedy, and temperature with top-k, top-p, min-p and a repeat penalty.

Order, defaults and flag names are the reference's (src/sample.rs:1-30, 101-191):
penalty -> top-k -> top-p -> min-p -> temperature -> draw; defaults temp 0.8
(``gen`` defaults to 0 = greedy), top-k 40, top-p 0.9, min-p 0, repeat-penalty 1.1 over
the last 64 tokens; the seed is random unless given.  As in the reference the work
is split: the device applies the penalty and selects the k best candidates
(``axon_b200/csrc/cuda/sampling.cu``), the host draws from them with a seeded
xoshiro256** generator, one number per decided token (``axon_b200/csrc/host/sampler.cpp``).
With top-k off, top-p and min-p off and no penalty, the draw itself runs on the
device over the whole row (inverse CDF in id order).
"""

from __future__ import annotations

import os
import time
from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..kernels import lib, ops

FLAGS = ("--temp", "--top-k", "--top-p", "--min-p", "--repeat-penalty", "--repeat-last-n", "--seed")
DEFAULT_TEMP = 0.8


@dataclass(frozen=True)
class SampleCfg:
    temp: float = DEFAULT_TEMP
    top_k: int = 40            # 0 = off (every token)
    top_p: float = 0.9         # >= 1 = off
    min_p: float = 0.0         # 0 = off
    repeat_penalty: float = 1.1  # 1 = off
    repeat_last_n: int = 64    # 0 = off
    seed: int = 0

    def to_host(self):
        c = lib.host().SampleConfig()
        c.temp, c.top_k, c.top_p, c.min_p = self.temp, self.top_k, self.top_p, self.min_p
        c.repeat_penalty, c.repeat_last_n, c.seed = self.repeat_penalty, self.repeat_last_n, self.seed
        return c


@dataclass
class SampleArgs:
    """Sampling flags as given on a command line; ``resolve`` fills in the defaults."""

    temp: Optional[float] = None
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    min_p: Optional[float] = None
    repeat_penalty: Optional[float] = None
    repeat_last_n: Optional[int] = None
    seed: Optional[int] = None

    @staticmethod
    def is_flag(f: str) -> bool:
        return f in FLAGS

    def set(self, flag: str, v: Optional[str]) -> None:
        """Set ``flag`` from its value; ValueError says what is wrong (src/sample.rs:129-165)."""
        if v is None:
            raise ValueError(f"{flag} needs a value")

        def number(lo: float, hi: float) -> float:
            try:
                x = float(v)
            except ValueError:
                x = float("nan")
            if not (x == x and lo <= x <= hi):
                raise ValueError(f"{flag} needs a number from {lo:g} to {hi:g}, got '{v}'")
            return x

        def whole() -> int:
            if not v.isdigit():
                raise ValueError(f"{flag} needs a whole number, got '{v}'")
            return int(v)

        if flag == "--temp":
            self.temp = number(0.0, 100.0)
        elif flag == "--top-k":
            self.top_k = whole()
        elif flag == "--top-p":
            self.top_p = number(0.0, 1.0)
        elif flag == "--min-p":
            self.min_p = number(0.0, 1.0)
        elif flag == "--repeat-penalty":
            p = number(0.0, 100.0)
            if p == 0.0:
                raise ValueError(f"{flag} must be above 0 (1 = off)")
            self.repeat_penalty = p
        elif flag == "--repeat-last-n":
            self.repeat_last_n = whole()
        elif flag == "--seed":
            self.seed = whole()
        else:
            raise ValueError(f"unknown sampling flag '{flag}'")

    def any_besides_temp(self) -> bool:
        return any(x is not None for x in (self.top_k, self.top_p, self.min_p, self.repeat_penalty,
                                           self.repeat_last_n, self.seed))

    def resolve(self, default_temp: float) -> Optional[SampleCfg]:
        """The settings, or None for temperature 0 (greedy)."""
        temp = default_temp if self.temp is None else self.temp
        if not temp > 0.0:
            return None
        return SampleCfg(
            temp=temp,
            top_k=40 if self.top_k is None else self.top_k,
            top_p=0.9 if self.top_p is None else self.top_p,
            min_p=0.0 if self.min_p is None else self.min_p,
            repeat_penalty=1.1 if self.repeat_penalty is None else self.repeat_penalty,
            repeat_last_n=64 if self.repeat_last_n is None else self.repeat_last_n,
            seed=random_seed() if self.seed is None else self.seed)


def random_seed() -> int:
    """A seed from the clock and the process id."""
    return (time.time_ns() ^ (os.getpid() << 32)) & 0xFFFFFFFFFFFFFFFF


class RowSampler:
    """One generation stream's settings, generator state and token history."""

    def __init__(self, cfg: Optional[SampleCfg], history: Sequence[int] = ()):
        self.cfg = cfg
        self.history: List[int] = list(history)
        self.host = lib.host().Sampler(cfg.to_host()) if cfg is not None else None

    @property
    def greedy(self) -> bool:
        return self.cfg is None

    def plain_temperature(self) -> bool:
        c = self.cfg
        return (c is not None and c.top_k == 0 and c.top_p >= 1.0 and c.min_p <= 0.0
                and (c.repeat_penalty == 1.0 or c.repeat_last_n == 0))


def pick_tokens(logits: torch.Tensor, rows: Sequence[RowSampler]) -> List[int]:
    """One token per row of ``logits [len(rows), vocab]`` (float32, on the device).

    Greedy rows take the device argmax (the last index among equal maxima).  Sampled
    rows get the penalty and the k best candidates on the device and the draw on the
    host; the picked token is appended to the row's history.  Rows of one kind are read
    where they lie (the kernels take a row index); only rows that the penalty changes are
    copied first, by a kernel of this library.  Everything the kernels need from the host
    (row indices, k, penalties, penalised ids, temperatures, uniform numbers) goes to the
    device in one copy.
    """
    n, vocab = logits.shape
    assert n == len(rows)
    if not logits.is_contiguous():
        raise ValueError("pick_tokens takes contiguous logits")
    dev = logits.device
    out: List[Optional[int]] = [None] * n
    greedy = [i for i, r in enumerate(rows) if r.greedy]
    plain = [i for i, r in enumerate(rows) if not r.greedy and r.plain_temperature()]
    cand = [i for i, r in enumerate(rows) if not r.greedy and not r.plain_temperature()]
    kmax = ops.topk_max()
    host = lib.host()

    id_lists = []
    for i in cand:
        c = rows[i].cfg
        id_lists.append(host.penalty_ids(rows[i].history, c.repeat_last_n)
                        if (c.repeat_penalty != 1.0 and c.repeat_last_n > 0) else [])
    width = max((len(x) for x in id_lists), default=0)
    ks = [rows[i].cfg.top_k for i in cand]
    on_device = [j for j, k in enumerate(ks) if 0 < k <= kmax]
    ng, npl, nc = len(greedy), len(plain), len(cand)
    # layout of the one upload, in 32-bit words: row indices of the three kinds | k | penalty
    # (float bits) | penalised ids | temperatures (float bits) | pad to 8 bytes | uniforms (double)
    o_k = ng + npl + nc
    o_pen, o_ids = o_k + nc, o_k + 2 * nc
    o_temp = o_ids + nc * width
    o_uni = (o_temp + npl + 1) // 2 * 2
    flat = np.full(o_uni + 2 * npl, -1, dtype=np.int32)
    flat[:o_k] = greedy + plain + cand
    keep = set(on_device)
    flat[o_k:o_pen] = [ks[j] if j in keep else 0 for j in range(nc)]
    flat[o_pen:o_ids] = np.asarray([rows[i].cfg.repeat_penalty for i in cand], dtype=np.float32).view(np.int32)
    for j, ids in enumerate(id_lists):
        flat[o_ids + j * width: o_ids + j * width + len(ids)] = ids
    flat[o_temp:o_temp + npl] = np.asarray([rows[i].cfg.temp for i in plain], dtype=np.float32).view(np.int32)
    flat[o_uni:] = np.asarray([rows[i].host.uniform() for i in plain], dtype=np.float64).view(np.int32)
    up = torch.from_numpy(flat).to(dev)
    whole = lambda idx: None if len(idx) == n else idx       # every row, in order: no index needed

    picks = torch.empty(ng + npl, dtype=torch.int32, device=dev)
    if greedy:
        ops.argmax(logits, picks[:ng], rows=whole(up[:ng]))
    if plain:
        ops.sample_temperature(logits, up[o_temp:o_temp + npl].view(torch.float32), up[o_uni:].view(torch.float64),
                               picks[ng:], rows=whole(up[ng:ng + npl]))
    both = None
    sub = None
    if cand:
        if width or len(on_device) < nc:
            # a copy: the penalty writes into it (and rows sorted on the host are read from it)
            sub = torch.empty((nc, vocab), dtype=torch.float32, device=dev)
            ops.gather_rows(logits, whole(up[ng + npl:o_k]), sub)
        if width:
            ops.repeat_penalty(sub, up[o_ids:o_temp].view(nc, width), up[o_pen:o_ids].view(torch.float32))
        if on_device:
            both = torch.empty((2, nc, kmax), dtype=torch.int32, device=dev)   # logits and ids: one copy back
            if sub is not None:
                ops.topk(sub, up[o_k:o_pen], both[0].view(torch.float32), both[1])
            else:
                ops.topk(logits, up[o_k:o_pen], both[0].view(torch.float32), both[1], rows=whole(up[ng + npl:o_k]))
    if greedy or plain:
        got = picks.tolist()
        for i, t in zip(greedy + plain, got):
            out[i] = int(t)
    if both is not None:
        both_h = both.cpu().numpy()
        cl_h, ci_h = both_h[0].view(np.float32), both_h[1]
        for j in on_device:
            k = min(ks[j], vocab)
            out[cand[j]] = int(rows[cand[j]].host.pick(cl_h[j, :k], ci_h[j, :k]))
    for j, k in enumerate(ks):
        if 0 < k <= kmax:
            continue
        # top-k off or above what the device selects: the whole row, sorted on the host
        # (the reference's slower path, src/sample.rs:16-20)
        row = sub[j].cpu().numpy()
        order = _sorted_candidates(row)
        if k > 0:
            order = order[:k]
        out[cand[j]] = int(rows[cand[j]].host.pick(row[order], order.astype(np.int32)))
    for i, r in enumerate(rows):
        r.history.append(out[i])
    return [int(t) for t in out]


def _sorted_candidates(row: np.ndarray) -> np.ndarray:
    """Indices of a row best first: by logit, then the larger id; NaN last
    (src/sample.rs:394-401)."""
    ids = np.arange(row.shape[0])
    key = np.where(np.isnan(row), -np.inf, row)
    # lexsort sorts by the last key first: logit descending, then id descending
    order = np.lexsort((-ids, -key))
    nan = np.isnan(row[order])
    return np.concatenate([order[~nan], order[nan]])
