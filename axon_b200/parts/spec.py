"""What a model is made of, as data.

An architecture is a function from its configuration to a :class:`ModelSpec`:
an embedding, a list of layers (each an arrangement of parts chosen per layer),
the order in which the layers run, a final norm and a head.  The engine builds
parts from these records through the part registry; no part knows which model
it is in, and no size or constant of a model appears anywhere but here.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part needs from the checkpoint.

    ``kind`` says what it is for the loader and for random initialisation:
    ``"matrix"`` (a projection, ``[out, in]``), ``"table"`` (embedding rows),
    ``"bias"`` or ``"gain"`` (a norm's weight).  Vectors (bias, gain) are held in
    32-bit on the device whatever the model's dtype; matrices and tables keep
    the dtype the checkpoint stores (bfloat16, or 32-bit if stored so).
    """

    shape: Tuple[int, ...]
    kind: str = "matrix"


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered ``kind``, its parameters (every size and
    constant it uses), the checkpoint names of its tensors by local name, and
    nested parts (an attention mixer's position encoding, for instance)."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    weights: Mapping[str, str] = field(default_factory=dict)
    parts: Mapping[str, "PartSpec"] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A layer: an arrangement (``block`` kind) of named parts."""

    block: str
    parts: Mapping[str, PartSpec]
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers`` and may
    appear in several entries (the layer's weights run twice, each run with a
    cache of its own).  ``cache_of`` names an earlier entry of the schedule
    whose cache this run reads instead of keeping one."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    #: checkpoint tensors whose names end so are read past without being used
    ignored_suffixes: Tuple[str, ...] = ()

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer} of {len(self.layers)}")
            if e.cache_of is not None and not (0 <= e.cache_of < i):
                raise ValueError(
                    f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
            if e.cache_of is not None and self.schedule[e.cache_of].cache_of is not None:
                raise ValueError(f"schedule entry {i} reads a cache that entry {e.cache_of} does not own")


# ---------------------------------------------------------------------------
# What a part needs of the cache manager.

@dataclass(frozen=True)
class KvNeed:
    """Rows in pages, per token and kv head: a key row of ``head_dim`` elements and, with
    ``planes`` 2, a value row of ``v_dim`` (None: as wide as the key).  ``planes`` 1 keeps one
    row only (a latent that serves as key and value).  ``window`` None keeps every position,
    else only the last ``window``."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_dim: Optional[int] = None
    planes: int = 2

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.planes == 1 or not self.v_dim else self.v_dim

    @property
    def elements_per_token(self) -> int:
        """Cache elements one position takes in one schedule entry."""
        return self.kv_heads * (self.head_dim + (self.value_dim if self.planes == 2 else 0))


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size, one slot per live request."""

    shape: Tuple[int, ...]
    dtype: str = "float32"
