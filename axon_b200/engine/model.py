"""A model built from its spec: parts put together, run in the order the schedule gives."""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Union

import torch

from ..parts.base import Part, Runtime, StepContext, fold_owed, norm_owed, part_class
from ..parts.spec import KvNeed, ModelSpec, PartSpec, StateNeed
from ..weights.loader import expected_tensors


class DecoderModel:
    """Embedding, blocks, final norm and head of one :class:`ModelSpec`.

    ``weights`` maps checkpoint names to device tensors; tensors are handed to the
    parts that name them and dropped from the mapping once nobody else needs them, so
    parts that repack their weights do not keep two copies alive.
    """

    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        spec.validate()
        self.spec, self.rt = spec, rt
        #: whether every part only queues kernels (then steps may be captured into CUDA graphs)
        self.graph_safe = True
        uses: Dict[str, int] = {}
        for category, ps in _walk(spec):
            for name in ps.weights.values():
                uses[name] = uses.get(name, 0) + 1

        def build(category: str, ps: PartSpec) -> Part:
            cls = part_class(category, ps.kind)
            self.graph_safe = self.graph_safe and bool(cls.graph_safe)
            nested = getattr(cls, "nested", {})
            tensors = {}
            for local in cls.tensors(ps):
                tensors[local] = weights[ps.weights[local]]
            part = cls(ps, tensors, rt, lambda sub, _n=nested, _ps=ps: build(_category_of(_n, _ps, sub), sub))
            for local in tensors:
                name = ps.weights[local]
                uses[name] -= 1
                if uses[name] <= 0:
                    weights.pop(name, None)
            return part

        self.embedding = build("embedding", spec.embedding)
        self.blocks = [build("block", PartSpec(l.block, l.params, {}, l.parts)) for l in spec.layers]
        self.final_norm = build("norm", spec.final_norm)
        self.head = build("head", spec.head)
        #: what each schedule entry keeps in the cache: {part path: need} over the cache-keeping
        #: parts of its layer (empty when it keeps nothing of its own)
        self.needs: List[Dict[str, Union[KvNeed, StateNeed]]] = []
        per_layer = [layer_cache_needs(l) for l in spec.layers]
        for e in spec.schedule:
            self.needs.append({} if e.cache_of is not None else dict(per_layer[e.layer]))

    def cache_owner(self, entry: int) -> int:
        e = self.spec.schedule[entry]
        return entry if e.cache_of is None else e.cache_of

    def graph_key(self, ctx: StepContext):
        """The parts' host-side launch parameters for this step (see ``Part.graph_key``), once each.
        Layers of one shape (kind, sizes and constants, nested parts) are asked once: this runs
        on the host before every step of single tokens."""
        reps = self.__dict__.get("_key_parts")
        if reps is None:
            seen, reps = set(), [self.embedding, self.final_norm, self.head]
            for layer, block in zip(self.spec.layers, self.blocks):
                sig = _shape_of(PartSpec(layer.block, layer.params, {}, layer.parts))
                if sig not in seen:
                    seen.add(sig)
                    reps.append(block)
            self._key_parts = reps
        keys = set()
        for part in reps:
            keys.update(part.graph_key(ctx))
        return tuple(sorted(keys, key=repr))

    def forward(self, ctx: StepContext, cache: Any, want_rows: Optional[torch.Tensor], n_want: int,
                logits_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run the step's tokens through every schedule entry; the float32 logits of
        the wanted rows ``[n_want, vocab]`` (None when nothing is wanted)."""
        rt, n = self.rt, ctx.n_tokens
        if not rt.precise:
            from ..kernels import fast
            fast.forget_owed(rt.device)      # whatever a step that failed half way still owed is void
        x = rt.buffer("residual", (n, self.spec.hidden_size), torch.float32)
        self.embedding.forward(ctx.tokens, x)
        owed = None          # partial sums the residual is still owed by the last product into it
        for k, e in enumerate(self.spec.schedule):
            block = self.blocks[e.layer]
            if block.passes_owed:
                owed = block.forward(x, ctx, cache.view(self.cache_owner(k)), e.cache_of is None, pending=owed)
            else:
                fold_owed(owed)
                owed = None
                block.forward(x, ctx, cache.view(self.cache_owner(k)), e.cache_of is None)
        if n_want == 0:
            fold_owed(owed)
            return None
        # the head runs on the wanted rows only (src/lm.rs:114-126)
        h = rt.buffer("head_in", (n_want, self.spec.hidden_size))
        norm_owed(self.final_norm, x, h, owed, rows=want_rows)
        if logits_out is not None:
            logits = logits_out[:n_want]
        else:
            logits = torch.empty((n_want, self.spec.vocab_size), dtype=torch.float32, device=rt.device)
        self.head.forward(h, logits)
        return logits


def layer_cache_needs(layer) -> Dict[str, Union[KvNeed, StateNeed]]:
    """What a layer keeps in the cache: ``{part path: need}`` for every part of its arrangement,
    nested ones included (paths are dotted: ``"mixer"``, ``"mixer.inner"``), whose class
    answers ``cache_need`` with something.  A layer may hold several such parts (attention
    beside a mixer with state, say) or none; no part name is special."""
    out: Dict[str, Union[KvNeed, StateNeed]] = {}

    def rec(category: str, ps: PartSpec, path: str) -> None:
        cls = part_class(category, ps.kind)
        need = cls.cache_need(ps)
        if need is not None:
            out[path or ps.kind] = need
        nested = getattr(cls, "nested", {})
        for name, sub in ps.parts.items():
            rec(nested.get(name, name), sub, f"{path}.{name}" if path else name)

    rec("block", PartSpec(layer.block, layer.params, {}, layer.parts), "")
    return out


def _shape_of(spec: PartSpec):
    """What a part is apart from its weights: kind, parameters, and the same of its nested parts."""
    return (spec.kind, repr(sorted(spec.params.items(), key=lambda kv: kv[0])),
            tuple((name, _shape_of(sub)) for name, sub in sorted(spec.parts.items())))


def _category_of(nested: Dict[str, str], parent: PartSpec, sub: PartSpec) -> str:
    for name, s in parent.parts.items():
        if s is sub:
            return nested.get(name, name)
    raise KeyError("a part built a nested part that its spec does not hold")


def _walk(spec: ModelSpec):
    from ..weights.loader import walk_parts
    return walk_parts(spec)
