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


def bind_weights(model, source: WeightSource, engine_dtype: torch.dtype, device: torch.device | str) -> None:
    """Check the source against the model's wanted tensors, then hand each part its tensors on the device."""
    check_weights(model.all_param_specs(), source, getattr(model, "ignored_names", lambda: [])())

    def get(name: str) -> torch.Tensor:
        t = source.get(name)
        return t.to(device=device, dtype=engine_dtype_of(t, engine_dtype))

    model.bind_all(get)
