"""Reading and writing safetensors files.

File layout (as the reference parses it, src/storage/safetensors.rs:211-318):
8 bytes little-endian header length, a JSON header mapping tensor names to
``{"dtype", "shape", "data_offsets"}``, then the raw little-endian data.
A folder may hold several ``*.safetensors`` shards; they are read in sorted
order and the first file that holds a name wins (src/storage/mmap_store.rs:148-211).
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_TAGS = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One memory-mapped shard."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: file of {size} bytes is too short for a header length")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: malformed header ({e})") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self._data_start = 8 + hlen
        data_size = size - self._data_start
        self.entries: dict[str, tuple[torch.dtype, tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                tag, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError) as ex:
                raise SafetensorsError(f"{path}: entry {name!r} is malformed ({ex})") from ex
            if tag not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype tag {tag!r}")
            dt = _DTYPES[tag]
            numel = 1
            for s in shape:
                numel *= s
            nbytes = numel * torch.empty((), dtype=dt).element_size()
            if not (0 <= b <= e <= data_size):
                raise SafetensorsError(f"{path}: tensor {name!r} lies outside the file ({b}..{e} of {data_size})")
            if e - b != nbytes:
                raise SafetensorsError(f"{path}: tensor {name!r}: shape {list(shape)} x {tag} needs {nbytes} "
                                       f"bytes, entry spans {e - b}")
            self.entries[name] = (dt, shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self):
        return self.entries.keys()

    def info(self, name: str):
        dt, shape, _, _ = self.entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A host tensor that owns its memory (copied out of the mapping)."""
        dt, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        buf = self._mm[self._data_start + b:self._data_start + e]
        return torch.frombuffer(bytearray(buf), dtype=dt).reshape(shape)

    def close(self):
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()


class TensorStore:
    """Every shard of a model folder behind one flat name lookup."""

    def __init__(self, folder: str):
        if os.path.isfile(folder):
            files = [folder]
        else:
            if not os.path.isdir(folder):
                raise SafetensorsError(f"{folder}: no such model folder")
            files = sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(".safetensors"))
        if not files:
            raise SafetensorsError(f"{folder}: no *.safetensors file in the folder")
        self.shards = [SafetensorsFile(f) for f in files]
        self._where: dict[str, SafetensorsFile] = {}
        for sh in self.shards:
            for n in sh.names():
                self._where.setdefault(n, sh)

    def names(self) -> list[str]:
        return list(self._where.keys())

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def info(self, name: str):
        return self._where[name].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def close(self):
        for s in self.shards:
            s.close()


def save_file(tensors: dict[str, torch.Tensor], path: str, metadata: dict[str, str] | None = None) -> None:
    """Writes one safetensors file; tensors are laid out in the order given."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _TAGS:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ({name})")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _TAGS[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    os.replace(tmp, path)
