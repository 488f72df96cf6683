"""Weights by tensor name: from the *.safetensors files of a model folder to the parts of a model.

The parts say which tensors they want (name, shape).  The loader compares that list with what the
folder holds and raises ONE error that lists every missing tensor, every unexpected tensor and
every tensor of the wrong shape; lucciola prints a line for a missing tensor and carries on with
a null pointer (include/safetensores.h:39-42) and reads exactly one file (src/qwen.cc:69).

Types: in a bfloat16 engine BF16 and F16 tensors are held as bfloat16 and a tensor stored in
32-bit stays 32-bit; integer tables become int32.  In a float32 engine every floating tensor
becomes float32 (exact for BF16 and F16).
"""
from __future__ import annotations

from pathlib import Path
from typing import Iterable, Protocol

import torch

from ..parts.base import ParamSpec
from .safetensors_io import SafetensorsFile


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every mismatch."""


class WeightSource(Protocol):
    def names(self) -> list[str]: ...
    def shape_dtype(self, name: str) -> tuple[tuple[int, ...], torch.dtype]: ...
    def get(self, name: str) -> torch.Tensor: ...
    def close(self) -> None: ...


class CheckpointFolder:
    """All *.safetensors files of a folder as one source of tensors."""

    def __init__(self, folder: str | Path):
        self.folder = Path(folder)
        files = sorted(self.folder.glob("*.safetensors"))
        if not files:
            raise WeightError(f"{self.folder} holds no *.safetensors file")
        self._files = [SafetensorsFile(f) for f in files]
        self._where: dict[str, SafetensorsFile] = {}
        for f in self._files:
            for n in f.names():
                if n in self._where:
                    raise WeightError(f"tensor {n!r} is in both {self._where[n].path.name} and {f.path.name}")
                self._where[n] = f

    def names(self) -> list[str]:
        return list(self._where)

    def shape_dtype(self, name: str) -> tuple[tuple[int, ...], torch.dtype]:
        info = self._where[name].tensors[name]
        return info.shape, info.torch_dtype

    def get(self, name: str) -> torch.Tensor:
        return self._where[name].get(name)

    def read_into(self, name: str, dst: torch.Tensor, start: int, n: int) -> None:
        self._where[name].read_into(name, dst, start, n)

    def close(self) -> None:
        for f in self._files:
            f.close()


def check_weights(specs: Iterable[ParamSpec], source: WeightSource, ignored: Iterable[str] = ()) -> None:
    specs = list(specs)
    have = set(source.names())
    want = {s.name for s in specs}
    missing = sorted(want - have)
    unexpected = sorted(have - want - set(ignored))
    wrong = []
    for s in specs:
        if s.name in have:
            shape, dtype = source.shape_dtype(s.name)
            if tuple(shape) != tuple(s.shape):
                wrong.append(f"{s.name}: expected {list(s.shape)}, found {list(shape)}")
            elif s.integer == dtype.is_floating_point:
                wrong.append(f"{s.name}: expected {'an integer' if s.integer else 'a floating'} type, found {dtype}")
    if missing or unexpected or wrong:
        parts = ["the checkpoint does not fit the model"]
        if missing:
            parts.append(f"missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            parts.append(f"wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n  ".join(parts))


def engine_dtype_of(t: torch.Tensor, engine_dtype: torch.dtype) -> torch.dtype:
    if not t.dtype.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if t.dtype in (torch.float32, torch.float64):
        return torch.float32                      # stored in 32-bit (or more): stays 32-bit
    return torch.bfloat16


class Uploader:
    """Host tensors to the device through two pinned buffers.  The tensors of a checkpoint are views of memory-mapped
    files: copied straight from there the driver stages them itself, a little at a time (3 GB/s measured, 20 s for a 32B
    model).  Here a chunk is copied into pinned memory by a few threads while the DMA of the chunk before it runs."""

    CHUNK = 64 << 20
    SMALL = 1 << 20            # below this a plain copy is as fast

    def __init__(self, device: torch.device | str, threads: int = 4):
        from concurrent.futures import ThreadPoolExecutor
        self.device = torch.device(device)
        self._pinned = [torch.empty(self.CHUNK, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
        self._free = [torch.cuda.Event() for _ in range(2)]            # the DMA out of a buffer has finished
        self._stream = torch.cuda.Stream(self.device)
        self._pool = ThreadPoolExecutor(max_workers=threads)
        self._threads = threads
        self._used = 0

    def upload(self, t: torch.Tensor) -> torch.Tensor:
        """A tensor of the same shape and type on the device; ordered before what the current stream does next."""
        nbytes = t.numel() * t.element_size()
        if nbytes < self.SMALL or not t.is_contiguous():
            return t.to(self.device)
        out = torch.empty(t.shape, dtype=t.dtype, device=self.device)
        src, dst = t.view(torch.uint8).reshape(-1), out.view(torch.uint8).reshape(-1)
        self._stream.wait_stream(torch.cuda.current_stream(self.device))    # `out` was allocated on the current stream
        for off in range(0, nbytes, self.CHUNK):
            n = min(self.CHUNK, nbytes - off)
            i = self._used % 2
            self._used += 1
            self._free[i].synchronize()
            buf = self._pinned[i]
            step = -(-n // self._threads)
            jobs = [self._pool.submit(buf[a:min(n, a + step)].copy_, src[off + a:off + min(n, a + step)]) for a in range(0, n, step)]
            for j in jobs:
                j.result()
            with torch.cuda.stream(self._stream):
                dst[off:off + n].copy_(buf[:n], non_blocking=True)
                self._free[i].record()
        torch.cuda.current_stream(self.device).wait_stream(self._stream)
        return out

    def upload_named(self, source, name: str) -> torch.Tensor:
        """The same for a tensor of a source that can read ranges of its bytes (`read_into`): the threads read the file
        straight into the pinned buffers."""
        shape, dtype = source.shape_dtype(name)
        out = torch.empty(shape, dtype=dtype, device=self.device)
        nbytes = out.numel() * out.element_size()
        dst = out.view(torch.uint8).reshape(-1)
        self._stream.wait_stream(torch.cuda.current_stream(self.device))
        for off in range(0, nbytes, self.CHUNK):
            n = min(self.CHUNK, nbytes - off)
            i = self._used % 2
            self._used += 1
            self._free[i].synchronize()
            buf = self._pinned[i]
            step = -(-n // self._threads)
            jobs = [self._pool.submit(source.read_into, name, buf[a:min(n, a + step)], off + a, min(n, a + step) - a) for a in range(0, n, step)]
            for j in jobs:
                j.result()
            with torch.cuda.stream(self._stream):
                dst[off:off + n].copy_(buf[:n], non_blocking=True)
                self._free[i].record()
        torch.cuda.current_stream(self.device).wait_stream(self._stream)
        return out

    def close(self) -> None:
        for e in self._free:
            e.synchronize()
        self._pool.shutdown()
        self._pinned = []


def bind_weights(model, source: WeightSource, engine_dtype: torch.dtype, device: torch.device | str) -> None:
    """Check the source against the model's wanted tensors, then hand each part its tensors on the device."""
    check_weights(model.all_param_specs(), source, getattr(model, "ignored_names", lambda: [])())
    up = Uploader(device) if torch.device(device).type == "cuda" else None

    def get(name: str) -> torch.Tensor:
        shape, dtype = source.shape_dtype(name)
        nbytes = int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
        if up is not None and hasattr(source, "read_into") and nbytes >= up.SMALL:
            t = up.upload_named(source, name)
        else:
            t = source.get(name)
            if up is not None and t.device.type == "cpu":
                t = up.upload(t)
        return t.to(device=device, dtype=engine_dtype_of(t, engine_dtype))     # the type is changed on the device, if at all

    try:
        model.bind_all(get)
    finally:
        if up is not None:
            up.close()
