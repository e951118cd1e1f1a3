"""Reading and writing the safetensors container.

Layout (src/store.rs:80-119): a little-endian u64 header length, a JSON header
``{name: {dtype, shape, data_offsets}}`` (``__metadata__`` skipped), then the
payload.  The header length and every tensor's byte range are checked against
the file before anything is sliced.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import torch


class SafetensorsError(ValueError):
    pass


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
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorRecord:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int      # absolute byte offsets into the file
    end: int
    file: int       # index of the shard


class SafetensorsFile:
    """One memory-mapped shard."""

    def __init__(self, path: str, index: int = 0):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: truncated safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header claims {hlen} bytes in a {size}-byte file")
        start = 8 + hlen
        try:
            head = json.loads(self._map[8:start].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: bad header: {e}") from None
        if not isinstance(head, dict):
            raise SafetensorsError(f"{path}: header is not an object")
        self.records: Dict[str, TensorRecord] = {}
        for name, v in head.items():
            if name == "__metadata__":
                continue
            try:
                dtype = v["dtype"]
                shape = tuple(int(x) for x in v["shape"])
                b, e = (int(x) for x in v["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: {name}: malformed header entry") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: {name}: dtype {dtype} is not supported")
            numel = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: {name}: negative dimension")
                numel *= s
            nbytes = numel * _DTYPES[dtype][1]
            if b < 0 or e < b or e - b != nbytes:
                raise SafetensorsError(
                    f"{path}: {name}: {dtype}{list(shape)} needs {nbytes} bytes, offsets give {e - b}"
                )
            if start + e > size:
                raise SafetensorsError(
                    f"{path}: {name}: {nbytes} bytes at offset {start + b} run past the {size}-byte file"
                )
            self.records[name] = TensorRecord(name, dtype, shape, start + b, start + e, index)

    def tensor(self, rec: TensorRecord) -> torch.Tensor:
        """A CPU tensor viewing the mapped bytes (copy before mutating)."""
        dt, size = _DTYPES[rec.dtype]
        count = (rec.end - rec.begin) // size
        if count == 0:
            return torch.empty(rec.shape, dtype=dt)
        if rec.begin % size:
            raw = bytearray(self._map[rec.begin:rec.end])
            return torch.frombuffer(raw, dtype=dt, count=count).reshape(rec.shape)
        return torch.frombuffer(self._map, dtype=dt, count=count, offset=rec.begin).reshape(rec.shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Write tensors in name order with an 8-byte padded header."""
    header, off = {}, 0
    names = sorted(tensors)
    for n in names:
        t = tensors[n]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"{n}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[n] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * ((8 - len(hb) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for n in names:
            t = tensors[n].detach().cpu().contiguous()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)


def shard_paths(model_dir: str) -> Iterable[str]:
    names = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    if not names:
        raise SafetensorsError(f"no .safetensors files in {model_dir}")
    return [os.path.join(model_dir, n) for n in names]
