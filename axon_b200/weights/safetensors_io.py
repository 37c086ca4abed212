"""Reading and writing safetensors files, with every header field checked.

The format: an 8-byte little-endian header length, a JSON header mapping each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the first byte after the header), then the data.  A header comes
from an untrusted file, so lengths, offsets, shapes and dtypes are validated
before any byte of data is touched (the reference's limits and checks:
src/safetensors.rs:33-38,177-298; shards: src/safetensors.rs:347-430).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024
MAX_SHARDS = 4096

_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_DTYPE_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors file; the message names it."""


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int
    file: str


def _parse_header(path: str, blob: bytes, data_len: int) -> Dict[str, TensorInfo]:
    try:
        header = json.loads(blob.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"{path}: the header is not JSON ({e})") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: the header is not a JSON object")
    infos: Dict[str, TensorInfo] = {}
    spans: List[Tuple[int, int, str]] = []
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        if not isinstance(rec, dict):
            raise SafetensorsError(f"{path}: tensor {name}: its record is not an object")
        dt, shape, off = rec.get("dtype"), rec.get("shape"), rec.get("data_offsets")
        if dt not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name}: dtype {dt!r} is not supported")
        if (not isinstance(shape, list)
                or any(isinstance(s, bool) or not isinstance(s, int) or s < 0 for s in shape)):
            raise SafetensorsError(f"{path}: tensor {name}: shape {shape!r} is not a list of sizes")
        if (not isinstance(off, list) or len(off) != 2
                or any(isinstance(o, bool) or not isinstance(o, int) or o < 0 for o in off)):
            raise SafetensorsError(f"{path}: tensor {name}: data_offsets {off!r} are not two offsets")
        begin, end = off
        n = 1
        for s in shape:
            n *= s
        if end < begin or end > data_len:
            raise SafetensorsError(
                f"{path}: tensor {name}: bytes {begin}..{end} lie outside the file's {data_len} data bytes")
        if end - begin != n * _DTYPES[dt][1]:
            raise SafetensorsError(
                f"{path}: tensor {name}: {end - begin} bytes do not hold shape {shape} of {dt}")
        infos[name] = TensorInfo(name, dt, tuple(shape), begin, end, path)
        if end > begin:
            spans.append((begin, end, name))
    spans.sort()
    for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
        if b1 < e0:
            raise SafetensorsError(f"{path}: tensors {n0} and {n1} overlap")
    return infos


class SafetensorsFile:
    """One mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot be read ({e.strerror})") from None
        if size < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a safetensors file")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > MAX_HEADER_BYTES or hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        blob = self._f.read(hlen)
        self.data_offset = 8 + hlen
        self.infos = _parse_header(path, blob, size - self.data_offset)
        self._map: Optional[mmap.mmap] = None

    def _mapped(self) -> mmap.mmap:
        if self._map is None:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        return self._map

    def tensor(self, name: str, copy: bool = True) -> torch.Tensor:
        """The tensor on the host, in its stored dtype.  With ``copy`` false it is a read-only
        view of the mapped file (no bytes are copied; it must not be written to and is valid
        until ``close``): what a loader wants that only copies the tensor on to a device."""
        info = self.infos[name]
        dtype, _ = _DTYPES[info.dtype]
        if info.end == info.begin:
            return torch.empty(info.shape, dtype=dtype)
        m = self._mapped()
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)     # torch warns that the buffer is read-only
            t = torch.frombuffer(m, dtype=dtype, count=(info.end - info.begin) // _DTYPES[info.dtype][1],
                                 offset=self.data_offset + info.begin).reshape(info.shape)
        return t.clone() if copy else t

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass          # a view handed out by tensor(copy=False) still lives: freed with it
            self._map = None
        self._f.close()


class Checkpoint:
    """The tensors of a model folder: ``model.safetensors`` alone, or the shards
    that ``model.safetensors.index.json`` names."""

    def __init__(self, folder: str):
        self.folder = folder
        single = os.path.join(folder, "model.safetensors")
        index = os.path.join(folder, "model.safetensors.index.json")
        self.files: Dict[str, SafetensorsFile] = {}
        self.infos: Dict[str, TensorInfo] = {}
        if os.path.exists(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    idx = json.load(f)
                wm = idx["weight_map"]
                assert isinstance(wm, dict)
            except (OSError, json.JSONDecodeError, KeyError, AssertionError, TypeError):
                raise SafetensorsError(f"{index}: not an index with a weight_map") from None
            shards = sorted(set(wm.values()))
            if len(shards) > MAX_SHARDS:
                raise SafetensorsError(f"{index}: {len(shards)} shards (at most {MAX_SHARDS})")
            for s in shards:
                if not isinstance(s, str) or os.path.basename(s) != s:
                    raise SafetensorsError(f"{index}: shard name {s!r} is not a plain file name")
                self.files[s] = SafetensorsFile(os.path.join(folder, s))
            for name, s in wm.items():
                if name not in self.files[s].infos:
                    raise SafetensorsError(f"{index}: names tensor {name} in {s}, which does not hold it")
            for s, f in self.files.items():
                for name, info in f.infos.items():
                    if name in self.infos:
                        raise SafetensorsError(
                            f"{folder}: tensor {name} is in {self.infos[name].file} and in {info.file}")
                    self.infos[name] = info
        elif os.path.exists(single):
            f = SafetensorsFile(single)
            self.files["model.safetensors"] = f
            self.infos = dict(f.infos)
        else:
            raise SafetensorsError(f"{folder}: no model.safetensors and no model.safetensors.index.json")
        self._by_path = {f.path: f for f in self.files.values()}

    def names(self) -> Iterable[str]:
        return self.infos.keys()

    def tensor(self, name: str, copy: bool = True) -> torch.Tensor:
        return self._by_path[self.infos[name].file].tensor(name, copy)

    def close(self) -> None:
        for f in self.files.values():
            f.close()


def write_safetensors_stream(path: str, specs: Sequence[Tuple[str, torch.dtype, Tuple[int, ...]]],
                             produce: Callable[[str], torch.Tensor],
                             metadata: Optional[Mapping[str, str]] = None) -> int:
    """Write a safetensors file whose tensors are made one at a time: ``specs`` lists
    (name, dtype, shape) in file order, ``produce(name)`` returns each host tensor when its
    turn comes, so a file larger than memory can be written.  Data is 8-byte aligned.
    Returns the bytes of tensor data written."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    for name, dtype, shape in specs:
        if dtype not in _DTYPE_NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {dtype} cannot be stored")
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * _DTYPES[_DTYPE_NAMES[dtype]][1]
        header[name] = {"dtype": _DTYPE_NAMES[dtype], "shape": [int(d) for d in shape],
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, dtype, shape in specs:
            t = produce(name).detach().cpu().contiguous()
            if t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(f"tensor {name}: made as {t.dtype} {tuple(t.shape)}, announced as {dtype} {tuple(shape)}")
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().data)
            del t
    return offset


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write host tensors to ``path`` in name order, data 8-byte aligned.  The tensors are copied
    before the file is opened, so they may be views of the very file that is being replaced."""
    order = sorted(tensors)
    held = {n: tensors[n].detach().cpu().clone() for n in order}
    write_safetensors_stream(path, [(n, held[n].dtype, tuple(held[n].shape)) for n in order],
                             lambda n: held.pop(n), metadata)
