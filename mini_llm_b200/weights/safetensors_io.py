"""Reading and writing the safetensors container, by tensor name.

File = 8-byte little-endian header length, a JSON header
{name: {dtype, shape, data_offsets}}, then the raw little-endian tensor bytes.
The reference reads one raw FP32 ``.bin`` file per tensor instead
(src/model/gpt2_model.cu:32-70).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "F64": torch.float64,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are read one by one by name."""

    def __init__(self, path: str):
        self.path = path
        if not os.path.isfile(path):
            raise SafetensorsError(f"{path}: no such file")
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        self.metadata = header.pop("__metadata__", {})
        self._entries: Dict[str, dict] = header
        self._data_start = 8 + hlen
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        data_len = size - self._data_start
        for name, e in self._entries.items():
            if e.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {e.get('dtype')!r}")
            b, en = e["data_offsets"]
            n = 1
            for s in e["shape"]:
                n *= int(s)
            want = n * torch.empty((), dtype=_DTYPES[e["dtype"]]).element_size()
            if not (0 <= b <= en <= data_len) or en - b != want:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} data_offsets {e['data_offsets']} do not match "
                    f"shape {e['shape']} of {e['dtype']}")

    def names(self) -> List[str]:
        return list(self._entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(int(s) for s in self._entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self._entries[name]["dtype"]]

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def tensor(self, name: str) -> torch.Tensor:
        """A fresh CPU tensor holding a copy of the named tensor."""
        e = self._entries[name]
        b, en = e["data_offsets"]
        dt = _DTYPES[e["dtype"]]
        shape = [int(s) for s in e["shape"]]
        if en == b:
            return torch.empty(shape, dtype=dt)
        buf = bytearray(self._mm[self._data_start + b:self._data_start + en])
        return torch.frombuffer(buf, dtype=dt).reshape(shape)

    def close(self):
        try:
            self._mm.close()
        finally:
            self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata=None) -> None:
    """Write (name, tensor) pairs in the given order."""
    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - len(hjson) % 8) % 8
    hjson += b" " * pad
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for _, t in items:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


class Checkpoint:
    """The tensors of a model folder: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` names (its ``weight_map``: tensor name -> file).  Same
    interface as one SafetensorsFile."""

    INDEX = "model.safetensors.index.json"

    def __init__(self, model_dir: str):
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, self.INDEX)
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, SafetensorsFile] = {}
        if os.path.isfile(single) or not os.path.isfile(index):
            self.path = single
            f = SafetensorsFile(single)                  # raises when neither file exists
            self._files[single] = f
            self._where = {n: f for n in f.names()}
            return
        self.path = index
        try:
            with open(index, "r", encoding="utf-8") as fh:
                weight_map = json.load(fh)["weight_map"]
            if not isinstance(weight_map, dict):
                raise TypeError("weight_map is not an object")
        except (OSError, KeyError, TypeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{index}: not a usable index: {e}") from e
        try:
            for name, fname in weight_map.items():
                fpath = os.path.join(model_dir, str(fname))
                f = self._files.get(fpath)
                if f is None:
                    f = self._files[fpath] = SafetensorsFile(fpath)
                if name not in f:
                    raise SafetensorsError(f"{index}: tensor {name!r} is not in {fname!r}")
                self._where[name] = f
            # a tensor that a shard holds but the index does not list is reported as unexpected by the loader
            for f in list(self._files.values()):
                for n in f.names():
                    self._where.setdefault(n, f)
        except Exception:
            self.close()
            raise

    def names(self) -> List[str]:
        return list(self._where)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._where[name].dtype(name)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def close(self):
        for f in self._files.values():
            f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

