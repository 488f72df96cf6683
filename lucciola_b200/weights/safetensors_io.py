"""Reader and writer for the safetensors container.

Format (the same one src/safetensors.cc:51-87 of lucciola parses): eight bytes
of little-endian header length, a JSON header that maps each tensor name to
{"dtype", "shape", "data_offsets": [begin, end]} (plus an optional
"__metadata__" entry), then the data, with offsets relative to the end of the
header.  lucciola accepts BF16 only and checks nothing; this reader takes
BF16, F16, F32, F64 and the integer types, and checks that every tensor lies
inside the file and has the byte count its shape and type ask for.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Mapping

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


_DTYPES: dict[str, tuple[torch.dtype, int]] = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
    "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "I16": (torch.int16, 2), "I32": (torch.int32, 4),
    "I64": (torch.int64, 8), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str                    # the container's name, e.g. "BF16"
    shape: tuple[int, ...]
    begin: int                    # byte offsets relative to the data section
    end: int

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]


class SafetensorsFile:
    """One file, memory-mapped; tensors are views of the mapping (copy before the file is closed)."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to hold a header")
        self._f = open(self.path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: header length {hlen} does not fit the file of {size} bytes")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self.data_offset = 8 + hlen
        data_size = size - self.data_offset
        self.tensors: dict[str, TensorInfo] = {}
        for name, e in header.items():
            try:
                dtype, shape, (b, en) = e["dtype"], tuple(int(x) for x in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError) as err:
                raise SafetensorsError(f"{self.path}: malformed entry for tensor {name!r}") from err
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {dtype!r}")
            want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dtype][1] if shape else _DTYPES[dtype][1]
            if not (0 <= b <= en <= data_size):
                raise SafetensorsError(f"{self.path}: tensor {name!r} lies outside the file ([{b}, {en}) of {data_size})")
            if en - b != want:
                raise SafetensorsError(
                    f"{self.path}: tensor {name!r} of shape {list(shape)} and type {dtype} needs {want} bytes, has {en - b}")
            self.tensors[name] = TensorInfo(name, dtype, shape, int(b), int(en))
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> list[str]:
        return list(self.tensors)

    def get(self, name: str) -> torch.Tensor:
        info = self.tensors[name]
        n = info.end - info.begin
        if n == 0:
            return torch.empty(info.shape, dtype=info.torch_dtype)
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=n, offset=self.data_offset + info.begin)
        # torch.frombuffer would warn about the read-only mapping; go through numpy.
        t = torch.from_numpy(buf.copy() if n < (1 << 16) else np.array(buf, copy=True))
        return t.view(info.torch_dtype).reshape(info.shape)

    def read_into(self, name: str, dst: torch.Tensor, start: int, n: int) -> None:
        """Bytes [start, start + n) of the tensor's data into `dst` (uint8, contiguous, on the host), read from the
        file itself: no page of a mapping is touched, and several threads may read at a time."""
        import os
        info = self.tensors[name]
        if start < 0 or n < 0 or start + n > info.end - info.begin or dst.numel() < n:
            raise SafetensorsError(f"{self.path}: bytes [{start}, {start + n}) do not lie in tensor {name!r} or in the buffer")
        view = memoryview(dst.numpy())[:n]
        at, done = self.data_offset + info.begin + start, 0
        while done < n:
            got = os.preadv(self._f.fileno(), [view[done:]], at + done)
            if got <= 0:
                raise SafetensorsError(f"{self.path}: the file ends inside tensor {name!r}")
            done += got

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def write_safetensors(path: str | Path, tensors: Mapping[str, torch.Tensor] | Iterable[tuple[str, torch.Tensor]],
                      metadata: Mapping[str, str] | None = None) -> None:
    """Write tensors (CPU, any supported dtype) in the order given."""
    items = list(tensors.items()) if isinstance(tensors, Mapping) else list(tensors)
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r} has dtype {t.dtype} that the container cannot hold")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            c = t.detach().cpu().contiguous()
            f.write(c.view(torch.uint8).numpy().tobytes() if c.numel() else b"")
