"""Random weights: a model folder (config.json, model.safetensors) from a configuration and a seed.

Linear maps and the embedding are drawn from N(0, std), norm weights from 1 + N(0, norm_std);
each tensor has its own generator seeded by (seed, tensor name), so a tensor's values do not
depend on which other tensors exist.  Values are rounded to the storage type once; whoever reads
the folder sees the rounded values.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any, Iterable, Mapping

import torch

from ..parts.base import ParamSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(spec: ParamSpec, seed: int, std: float, norm_std: float, dtype: torch.dtype,
                  device: torch.device | str = "cpu") -> torch.Tensor:
    device = torch.device(device)
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.integer:
        return torch.randint(0, 2 ** 15, spec.shape, generator=g, device=device, dtype=torch.int32)
    x = torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32)
    if spec.init == "norm":
        x = 1.0 + norm_std * x
    else:
        x = std * x
    return x.to(dtype)


class RandomWeights:
    """A source of tensors by name, like a checkpoint folder, drawn on demand on any device."""

    def __init__(self, specs: Iterable[ParamSpec], seed: int, std: float = 0.02, norm_std: float = 0.0,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device | str = "cpu"):
        self.specs = {s.name: s for s in specs}
        self.seed, self.std, self.norm_std, self.dtype, self.device = seed, std, norm_std, dtype, device

    def names(self) -> list[str]:
        return list(self.specs)

    def shape_dtype(self, name: str) -> tuple[tuple[int, ...], torch.dtype]:
        s = self.specs[name]
        return tuple(s.shape), (torch.int32 if s.integer else self.dtype)

    def get(self, name: str) -> torch.Tensor:
        return random_tensor(self.specs[name], self.seed, self.std, self.norm_std, self.dtype, self.device)

    def close(self) -> None:
        pass


def write_random_model(config_dict: Mapping[str, Any], folder: str | Path, seed: int, std: float = 0.02,
                       norm_std: float = 0.0, dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write config.json and model.safetensors for the architecture that `config_dict` names."""
    from ..config.registry import resolve_architecture
    from ..parts.base import Runtime

    arch = resolve_architecture(config_dict)
    cfg = arch.config_from_dict(config_dict)
    model = arch.build(cfg, Runtime("cpu", torch.float32))
    src = RandomWeights(model.all_param_specs(), seed, std, norm_std, dtype)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(dict(config_dict), indent=1))
    write_safetensors(folder / "model.safetensors", ((n, src.get(n)) for n in src.names()),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder


def main(argv: list[str] | None = None) -> int:
    """lucciola_random_model --config FILE --seed N --out DIR: a model folder with random weights."""
    import argparse
    ap = argparse.ArgumentParser(prog="lucciola_random_model",
                                 description="Write a model folder (config.json, model.safetensors) with random weights "
                                             "for the architecture a config.json names.")
    ap.add_argument("--config", required=True, help="a config.json (its `architectures` entry chooses the model)")
    ap.add_argument("--seed", type=int, required=True)
    ap.add_argument("--out", required=True, help="folder to write")
    ap.add_argument("--std", type=float, default=0.02, help="standard deviation of matrix weights")
    ap.add_argument("--norm-std", type=float, default=0.0, help="norm weights are 1 + N(0, this)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="type the tensors are stored in")
    args = ap.parse_args(argv)
    config = json.loads(Path(args.config).read_text())
    folder = write_random_model(config, args.out, args.seed, std=args.std, norm_std=args.norm_std,
                                dtype=torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    print(folder)
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
