"""Weights by tensor name: from safetensors, or seeded random ones.

What a model needs is derived from its :class:`ModelSpec`: every part declares its
tensors, the spec maps them to checkpoint names.  A checkpoint is checked whole
before a byte is copied, and a single :class:`WeightsError` lists everything that is
missing, unexpected, misshapen or of an unusable dtype (the reference's error cases:
src/safetensors.rs:1531-1558, src/model.rs:1493-1528).

Dtypes on the device: matrices and tables keep bfloat16 (float16 is rounded to it),
a tensor stored in 32-bit stays 32-bit; vectors (biases, gains) are widened to
float32, which is exact; integer tables become int32.  The 32-bit model widens
everything to float32.
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, List, Mapping, Optional, Tuple, Union

import torch

from ..config.base import ModelConfig, architecture_of, write_config_json
from ..parts.base import part_class
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, TensorDecl
from .safetensors_io import Checkpoint, SafetensorsError, write_safetensors, write_safetensors_stream


class WeightsError(ValueError):
    """A checkpoint that does not fit the model; lists every fault found."""

    def __init__(self, where: str, missing=(), unexpected=(), shapes=(), dtypes=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.shapes, self.dtypes = list(shapes), list(dtypes)
        lines = [f"{where}: the checkpoint does not fit the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.shapes:
            lines.append(f"  tensor {name}: shape {list(got)} doesn't fit the model (expected {list(want)})")
        for name, dt in self.dtypes:
            lines.append(f"  tensor {name}: dtype {dt} is not supported (BF16, F16, F32)")
        super().__init__("\n".join(lines))


def walk_parts(spec: ModelSpec) -> Iterator[Tuple[str, PartSpec]]:
    """Every (category, PartSpec) of a model, nested ones included."""

    def rec(category: str, ps: PartSpec) -> Iterator[Tuple[str, PartSpec]]:
        yield category, ps
        nested = getattr(part_class(category, ps.kind), "nested", {})
        for name, sub in ps.parts.items():
            yield from rec(nested.get(name, name), sub)

    yield from rec("embedding", spec.embedding)
    for layer in spec.layers:
        yield from rec("block", PartSpec(layer.block, layer.params, {}, layer.parts))
    yield from rec("norm", spec.final_norm)
    yield from rec("head", spec.head)


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorDecl]:
    """Checkpoint name -> declaration, for every tensor the model reads."""
    out: Dict[str, TensorDecl] = {}
    for category, ps in walk_parts(spec):
        decls = part_class(category, ps.kind).tensors(ps)
        for local, decl in decls.items():
            if local not in ps.weights:
                raise ValueError(f"part '{ps.kind}' needs tensor '{local}' but the spec names none")
            name = ps.weights[local]
            if name in out and tuple(out[name].shape) != tuple(decl.shape):
                raise ValueError(f"tensor {name} is used with shapes {out[name].shape} and {decl.shape}")
            if name not in out or decl.kind != "table":
                out[name] = TensorDecl(tuple(decl.shape), decl.kind)
    return out


def _device_dtype(stored: torch.dtype, kind: str, model_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if model_dtype == torch.float32 or kind in ("bias", "gain"):
        return torch.float32
    if stored == torch.float32:
        return torch.float32  # stored in 32-bit: stays so
    return torch.bfloat16


def check_checkpoint(ckpt: Checkpoint, spec: ModelSpec, where: str) -> Dict[str, TensorDecl]:
    """Compare a checkpoint's tensors (names, shapes, dtypes; no data is read) with what the
    model needs; raises one :class:`WeightsError` that lists every fault, else returns the
    model's tensors by checkpoint name."""
    want = expected_tensors(spec)
    have = ckpt.infos
    ignored = lambda n: any(n.endswith(s) for s in spec.ignored_suffixes)
    missing = sorted(n for n in want if n not in have)
    unexpected = sorted(n for n in have if n not in want and not ignored(n))
    shapes = [(n, have[n].shape, want[n].shape) for n in sorted(want)
              if n in have and tuple(have[n].shape) != tuple(want[n].shape)]
    dtypes = [(n, have[n].dtype) for n in sorted(want)
              if n in have and have[n].dtype not in ("BF16", "F16", "F32")]
    if missing or unexpected or shapes or dtypes:
        raise WeightsError(where, missing, unexpected, shapes, dtypes)
    return want


def load_weights(folder: str, spec: ModelSpec, dtype: torch.dtype,
                 device: Union[str, torch.device]) -> Dict[str, torch.Tensor]:
    """Read the model's tensors from ``folder`` onto ``device``.  A tensor goes from the
    mapped file to the device in one copy (no staging copy on the host), and is converted
    there, so the host never holds more than the mapping."""
    ckpt = Checkpoint(folder)
    try:
        want = check_checkpoint(ckpt, spec, folder)
        out: Dict[str, torch.Tensor] = {}
        for name, decl in want.items():
            t = ckpt.tensor(name, copy=False)
            want_dt = _device_dtype(t.dtype, decl.kind, dtype)
            d = t.to(device=device)
            if d.data_ptr() == t.data_ptr():
                d = t.clone()                   # the same memory (a host "device"): the mapping will be closed
            out[name] = d.to(want_dt).contiguous()
            del t, d
        if torch.device(device).type == "cuda":
            torch.cuda.synchronize(device)      # the copies read the mapping: done before it is closed
        return out
    finally:
        ckpt.close()


def _seed_of(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, decl: TensorDecl, seed: int, std: float = 0.02, gain_std: float = 0.1,
                  device: Union[str, torch.device] = "cpu") -> torch.Tensor:
    """A seeded float32 tensor: N(0, std) for matrices, tables and biases,
    1 + N(0, gain_std) for gains.  The stream depends on the seed and the tensor's name
    only, so a model's tensors do not depend on the order in which they are made."""
    g = torch.Generator(device=device)
    g.manual_seed(_seed_of(seed, name))
    t = torch.randn(tuple(decl.shape), generator=g, dtype=torch.float32, device=device)
    if decl.kind == "gain":
        return 1.0 + gain_std * t
    return std * t


def random_weights(spec: ModelSpec, seed: int, dtype: torch.dtype, device: Union[str, torch.device],
                   std: float = 0.02, gain_std: float = 0.1) -> Dict[str, torch.Tensor]:
    """Seeded random weights made on ``device`` directly (no folder): values are
    rounded to bfloat16 first, as a stored checkpoint would hold them."""
    out: Dict[str, torch.Tensor] = {}
    for name, decl in expected_tensors(spec).items():
        t = random_tensor(name, decl, seed, std, gain_std, device).to(torch.bfloat16)
        out[name] = t.to(_device_dtype(torch.bfloat16, decl.kind, dtype)).contiguous()
    return out


def write_random_model(folder: str, config: ModelConfig, seed: int, store_dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02, gain_std: float = 0.1, shards: int = 1) -> None:
    """Write ``config.json`` and the weights of a seeded random model: ``model.safetensors``, or
    with ``shards`` > 1 that many files ``model-0000i-of-0000n.safetensors`` of about equal size
    and the ``model.safetensors.index.json`` that maps every tensor to its file.  Tensors are
    made and written one at a time, so a model larger than host memory can be written."""
    arch = architecture_of(config.to_dict())
    spec = arch.build_spec(config)
    decls = expected_tensors(spec)
    names = sorted(decls)
    item = torch.empty((), dtype=store_dtype).element_size()
    size = {n: item * int(torch.Size(decls[n].shape).numel()) for n in names}
    produce = lambda n: random_tensor(n, decls[n], seed, std, gain_std).to(store_dtype)
    write_config_json(folder, config)
    if shards <= 1:
        write_safetensors_stream(os.path.join(folder, "model.safetensors"),
                                 [(n, store_dtype, tuple(decls[n].shape)) for n in names], produce, {"format": "pt"})
        return
    # contiguous runs of the sorted names, cut where the running size passes the next n-th of the whole
    total, groups, run, acc = sum(size.values()), [], [], 0
    for n in names:
        run.append(n)
        acc += size[n]
        if len(groups) < shards - 1 and acc >= total * (len(groups) + 1) / shards:
            groups.append(run)
            run = []
    if run:
        groups.append(run)
    weight_map = {}
    for i, group in enumerate(groups):
        fname = f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors"
        write_safetensors_stream(os.path.join(folder, fname), [(n, store_dtype, tuple(decls[n].shape)) for n in group],
                                 produce, {"format": "pt"})
        weight_map.update({n: fname for n in group})
    with open(os.path.join(folder, "model.safetensors.index.json"), "w", encoding="utf-8") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1, sort_keys=True)
        f.write("\n")
