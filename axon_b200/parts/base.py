"""Interfaces of the parts a model is put together from, and their registry.

Categories and what each must offer:

``norm``       ``forward(x, out, rows=None)``: ``x`` float32 ``[n, D]`` (the residual
               stream), ``out`` ``[m, D]`` in the model's dtype; ``rows`` gathers.
``position``   ``rotation(ctx)``: a float32 table ``[n, rot/2, 2]`` of (cos, sin) for
               the step's positions, or None; attributes ``rot`` and ``adjacent``.
``mixer``      ``forward(h, x, ctx, cache, write_cache)``: reads the normed input ``h``
               and *adds* its output into the float32 residual ``x``.  ``cache`` is a
               :class:`axon_b200.kernels.ops.KvView` or a state tensor ``[slots, ...]``
               according to ``cache_need``.  A simple mixer may implement
               ``compute(h, ctx, cache) -> tensor`` instead and inherit the add.
``ffn``        ``forward(h, x, ctx)``: as a mixer, without a cache.
``block``      ``forward(x, ctx, cache, write_cache)``: one layer on the residual stream.
               ``cache`` is what the layer's cache-keeping parts own: the one view or slab
               when one nested part answers ``cache_need``, a dict by part name (``"mixer"``,
               dotted for deeper nesting) when several do, None when none does.
``embedding``  ``forward(tokens, x)``: token ids to float32 rows.
``head``       ``forward(h, logits)``: normed rows to float32 logits.

Every part is built from a :class:`PartSpec` alone: ``spec.params`` carries all of
its sizes and constants, ``tensors`` its weights by local name.  ``tensors(spec)``
declares which tensors it needs (shape, kind) so that the loader can check a
checkpoint before anything is copied and so that random models can be written.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, ClassVar, Dict, List, Mapping, Optional, Tuple, Type, Union

import torch

from .spec import KvNeed, PartSpec, StateNeed, TensorDecl

CATEGORIES = ("norm", "position", "mixer", "ffn", "block", "embedding", "head")


class Runtime:
    """What parts share at run time: the model's dtype and device, and named
    scratch buffers that are reused from step to step (a buffer only ever grows)."""

    def __init__(self, dtype: torch.dtype, device: Union[str, torch.device]):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine runs in float32 or bfloat16, not {dtype}")
        self.dtype = dtype
        self.device = torch.device(device)
        #: the true 32-bit path: plain FFMA kernels everywhere
        self.precise = dtype == torch.float32
        self._buffers: Dict[str, torch.Tensor] = {}
        self._pinned: Dict[str, Tuple[torch.Tensor, Optional[torch.cuda.Event]]] = {}
        self._uploads: Dict[Any, torch.Tensor] = {}
        self._uploads_held = set()
        #: raised whenever an existing scratch buffer is replaced by a larger one: addresses
        #: handed out before are stale from then on (captured CUDA graphs must be dropped)
        self.generation = 0

    def buffer(self, name: str, shape: Tuple[int, ...], dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        dtype = dtype or self.dtype
        n = 1
        for s in shape:
            n *= s
        buf = self._buffers.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            if buf is not None:
                self.generation += 1
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[name] = buf
        return buf[:n].view(shape)

    def upload_i32(self, name: str, values) -> torch.Tensor:
        """Host integers (a work list, say) as a device tensor.  The same list under the same name
        is uploaded once and kept, so steps of a shape seen before copy nothing, and a CUDA graph
        may hold the tensor's address (lists first met inside a capture are refused: the capture
        fails and the step stays eager).  New lists go through pinned memory without blocking."""
        import numpy as np
        key = (name, tuple(values))
        capturing = torch.cuda.is_current_stream_capturing()
        hit = self._uploads.get(key)
        if hit is not None:
            if capturing:
                self._uploads_held.add(key)          # a graph reads it from now on: never dropped
            else:
                self._uploads[key] = self._uploads.pop(key)      # most recently used last
            return hit
        if capturing:
            raise RuntimeError("a host list would be uploaded for the first time inside a graph capture")
        n = len(values)
        host, event = self._pinned.get(name, (None, None))
        if event is not None:
            event.synchronize()
        if host is None or host.numel() < n:
            host = torch.empty(max(n, 1024), dtype=torch.int32).pin_memory()
        host.numpy()[:n] = np.asarray(values, dtype=np.int32)
        dev = torch.empty(max(n, 1), dtype=torch.int32, device=self.device)[:n]
        dev.copy_(host[:n], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._pinned[name] = (host, event)
        self._uploads[key] = dev
        if len(self._uploads) > 256:
            for old in list(self._uploads):
                if len(self._uploads) <= 192:
                    break
                if old not in self._uploads_held and old != key:
                    del self._uploads[old]
        return dev

    def release_buffers(self) -> None:
        self._buffers.clear()


@dataclass
class StepContext:
    """One step's batch as the parts see it.

    Tokens of all entries lie flattened, each request's in order.  ``token_slot[t]``
    is the cache slot of token ``t`` and ``positions[t]`` its position in its request.
    The ``seg_*`` lists describe each entry: its slot, where its tokens start in
    the flattened batch, how many there are, and how many positions its request holds
    after this step (so its tokens sit at ``seg_kv_len - seg_q_len ...``).
    """

    rt: Runtime
    n_tokens: int
    tokens: torch.Tensor
    positions: torch.Tensor
    token_slot: torch.Tensor
    seg_slot: List[int]
    seg_q_start: List[int]
    seg_q_len: List[int]
    seg_kv_len: List[int]
    #: device copy of the four lists above as int32 ``[4, segments]`` (slot, q_start, q_len, kv_len)
    segments: Optional[torch.Tensor] = None
    #: for steps of single tokens: device int32 ``[segments, 2]`` rows ``(segment, 0)``, the
    #: attention kernels' work list (so that such a step needs no further host-to-device copy)
    unit_items: Optional[torch.Tensor] = None
    #: host copies for parts that run on the host side of a step (toy parts, tests)
    host_positions: Optional[List[int]] = None
    scratch: Dict[Any, Any] = field(default_factory=dict)

    @property
    def max_q_len(self) -> int:
        return max(self.seg_q_len) if self.seg_q_len else 0

    @property
    def max_kv_len(self) -> int:
        return max(self.seg_kv_len) if self.seg_kv_len else 0


class Part:
    category: ClassVar[str] = ""
    kind: ClassVar[str] = ""
    #: True when ``forward`` only queues kernels on the current stream with arguments that
    #: do not depend on values read back from the device: no synchronisation, no host-side
    #: branching on device data, no allocation.  Steps of a model whose parts are all safe
    #: may be captured into CUDA graphs.
    graph_safe: ClassVar[bool] = False
    #: Owed sums.  A product for few rows may be split over K and leave its partial sums in
    #: scratch for the next reader of its output (``kernels.fast.PendingFold``), which saves
    #: that product a pass.  A mixer or feed-forward whose class sets ``may_defer`` takes
    #: ``defer=True`` in ``forward`` and then returns what its last product into the residual
    #: still owes (or None); a norm whose class sets ``folds_owed`` takes ``pending=`` and adds
    #: it to the rows it reads; a block whose class sets ``passes_owed`` takes ``pending=`` for
    #: its input and returns what its output is owed.  Parts that set none of these never see
    #: a PendingFold: their caller folds first (``fold_owed``).
    may_defer: ClassVar[bool] = False
    folds_owed: ClassVar[bool] = False
    passes_owed: ClassVar[bool] = False

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        return {}

    def graph_key(self, ctx: "StepContext") -> Tuple:
        """Whatever this part's launches take from the host that differs between two steps of
        the same batch shape (a split count that follows the context length, say).  Steps of
        single tokens replay a captured CUDA graph when batch shape and these keys agree."""
        return ()

    @classmethod
    def cache_need(cls, spec: PartSpec) -> Union[KvNeed, StateNeed, None]:
        return None

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime,
                 build: Callable[[PartSpec], "Part"]):
        self.spec = spec
        self.rt = rt


class Mixer(Part):
    category = "mixer"

    def compute(self, h: torch.Tensor, ctx: StepContext, cache: Any) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Any,
                write_cache: bool = True) -> None:
        from ..kernels import ops
        out = self.compute(h, ctx, cache)
        ops.residual_add(x, out.contiguous())


class FeedForward(Part):
    category = "ffn"

    def compute(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext) -> None:
        from ..kernels import ops
        out = self.compute(h, ctx)
        ops.residual_add(x, out.contiguous())


def fold_owed(pending) -> None:
    """Bring a tensor up to date with the partial sums it is still owed (None: nothing to do)."""
    if pending is not None:
        from ..kernels import ops
        ops.fold_partials(pending)


def norm_owed(norm: Part, x: torch.Tensor, out: torch.Tensor, pending, **kw) -> None:
    """``norm.forward(x, out)`` where ``x`` may still be owed partial sums."""
    if pending is not None and norm.folds_owed:
        norm.forward(x, out, pending=pending, **kw)
    else:
        fold_owed(pending)
        norm.forward(x, out, **kw)


_REGISTRY: Dict[Tuple[str, str], Type[Part]] = {}


def register_part(cls: Type[Part]) -> Type[Part]:
    """Class decorator: make a part available under ``(category, kind)``."""
    if cls.category not in CATEGORIES or not cls.kind:
        raise ValueError(f"{cls.__name__} must name its category ({', '.join(CATEGORIES)}) and kind")
    _REGISTRY[(cls.category, cls.kind)] = cls
    return cls


def part_class(category: str, kind: str) -> Type[Part]:
    try:
        return _REGISTRY[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise KeyError(f"no {category} part of kind '{kind}' is registered (known: {', '.join(known)})") from None


def nested_categories(category: str, kind: str) -> Mapping[str, str]:
    """Category of each nested part name of a part class (``{"position": "position"}``)."""
    return getattr(part_class(category, kind), "nested", {})
