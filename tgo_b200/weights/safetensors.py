"""A safetensors reader and writer of this package's own.

Container: 8 bytes little-endian header length N, N bytes of JSON
{name: {"dtype", "shape", "data_offsets": [begin, end]}}, then the planes.
The header is treated as hostile: every length, offset and shape is checked
before a byte of tensor data is touched, and errors come in a fixed order
(safetensors/safetensors.go:114-272). A folder with `model.safetensors.index.json`
is read through its weight_map, whose shard names must be plain file names
(safetensors/repo.go:120-194).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Tuple

import torch

MAX_HEADER = 100 * 1024 * 1024

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class Entry:
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """One file, header parsed and checked; planes are read on demand from a map."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a header length")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > MAX_HEADER or 8 + hlen > size:
            self._f.close()
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file "
                                   f"({size} bytes) or the {MAX_HEADER}-byte limit")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            self._f.close()
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
        if not isinstance(header, dict):
            self._f.close()
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self.data_start = 8 + hlen
        self.entries: Dict[str, Entry] = {}
        try:
            self._parse(header, size - self.data_start)
        except SafetensorsError:
            self._f.close()
            raise
        self._map = None

    def _parse(self, header: dict, data_len: int) -> None:
        for name in sorted(header):
            if name == "__metadata__":
                continue
            ent = header[name]
            if not isinstance(ent, dict):
                raise SafetensorsError(f"{self.path}: entry {name!r} is not an object")
            dt = ent.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{self.path}: {name!r} has unknown dtype {dt!r}")
            shape = ent.get("shape")
            if not isinstance(shape, list) or any(
                    isinstance(s, bool) or not isinstance(s, int) or s < 0 for s in shape):
                raise SafetensorsError(f"{self.path}: {name!r} has a bad shape {shape!r}")
            offs = ent.get("data_offsets")
            if (not isinstance(offs, list) or len(offs) != 2
                    or any(isinstance(o, bool) or not isinstance(o, int) for o in offs)):
                raise SafetensorsError(f"{self.path}: {name!r} has bad data_offsets {offs!r}")
            begin, end = offs
            if not (0 <= begin <= end <= data_len):
                raise SafetensorsError(f"{self.path}: {name!r} spans [{begin}, {end}) outside "
                                       f"the {data_len} data bytes")
            count = 1
            for s in shape:
                count *= s
            if count * _DTYPES[dt][1] != end - begin:
                raise SafetensorsError(f"{self.path}: {name!r} of shape {shape} and dtype {dt} "
                                       f"needs {count * _DTYPES[dt][1]} bytes, has {end - begin}")
            self.entries[name] = Entry(dt, tuple(shape), begin, end)
        spans = sorted((e.begin, e.end, n) for n, e in self.entries.items() if e.end > e.begin)
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{self.path}: {n0!r} and {n1!r} overlap")

    def tensor(self, name: str) -> torch.Tensor:
        """The plane of `name` as a CPU tensor backed by the file map (read-only)."""
        ent = self.entries[name]
        dtype = _DTYPES[ent.dtype][0]
        if ent.end == ent.begin:
            return torch.empty(ent.shape, dtype=dtype)
        if self._map is None:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        view = memoryview(self._map)[self.data_start + ent.begin:self.data_start + ent.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # torch warns that the buffer is read-only
            t = torch.frombuffer(view, dtype=dtype)
        return t.reshape(ent.shape)

    def close(self) -> None:
        self._map = None      # tensors handed out keep the map alive through their views
        self._f.close()


class SafetensorsRepo:
    """A model folder: one `model.safetensors`, or shards named by an index file."""

    def __init__(self, model_dir: str):
        self.files: Dict[str, SafetensorsFile] = {}
        self.where: Dict[str, str] = {}
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        if os.path.exists(index):
            with open(index) as f:
                try:
                    wm = json.load(f).get("weight_map")
                except json.JSONDecodeError as e:
                    raise SafetensorsError(f"{index}: not JSON: {e}") from None
            if not isinstance(wm, dict) or not wm:
                raise SafetensorsError(f"{index}: weight_map is missing or empty")
            for name in sorted(wm):
                shard = wm[name]
                if (not isinstance(shard, str) or not shard or os.path.basename(shard) != shard
                        or shard in (".", "..")):
                    raise SafetensorsError(f"{index}: shard name {shard!r} for {name!r} is not "
                                           "a plain file name")
                if shard not in self.files:
                    self.files[shard] = SafetensorsFile(os.path.join(model_dir, shard))
                if name not in self.files[shard].entries:
                    raise SafetensorsError(f"{index}: {name!r} is not in {shard}")
                self.where[name] = shard
            for shard, f in self.files.items():
                for name in f.entries:
                    if self.where.get(name) != shard:
                        raise SafetensorsError(f"{shard}: holds {name!r}, which the index "
                                               "does not place there")
        elif os.path.exists(single):
            self.files["model.safetensors"] = SafetensorsFile(single)
            for name in self.files["model.safetensors"].entries:
                self.where[name] = "model.safetensors"
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor "
                                   "model.safetensors.index.json is there")

    def names(self):
        return sorted(self.where)

    def entry(self, name: str) -> Entry:
        return self.files[self.where[name]].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self.files[self.where[name]].tensor(name)

    def close(self) -> None:
        for f in self.files.values():
            f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Write CPU tensors, names sorted, planes 8-byte aligned by header padding."""
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"{name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((-(8 + len(blob))) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
