"""From a model folder (or a configuration and a seed) to a runner that can step."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping, Optional

import torch

from ..config.engine_options import EngineOptions
from ..config.model_config import read_config_json
from ..config.registry import resolve_architecture
from ..csrc import KernelLibraryError, library
from ..parts.base import Runtime
from ..weights.loader import CheckpointFolder, bind_weights
from ..weights.random_init import RandomWeights
from .step import ModelRunner

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _runtime(options: EngineOptions) -> Runtime:
    options.validate()
    if not torch.cuda.is_available():
        raise KernelLibraryError("no CUDA device: this engine runs on the GPU only")
    device = torch.device(options.device)
    torch.cuda.set_device(device)
    lib = library()
    lib.lb_device_arch.restype = int
    arch = lib.lb_device_arch()
    if arch != 100:
        raise KernelLibraryError(f"the kernels are built for sm_100a; device {device} reports compute capability {arch}")
    return Runtime(device, _TORCH_DTYPES[options.dtype])


def build_runner(model_dir: str | Path, options: Optional[EngineOptions] = None, num_pages: Optional[int] = None) -> ModelRunner:
    """Read config.json, pick the model by its architecture name, load the weights by tensor name."""
    options = options or EngineOptions()
    cfg_dict = read_config_json(model_dir)
    arch = resolve_architecture(cfg_dict)
    cfg = arch.config_from_dict(cfg_dict)
    rt = _runtime(options)
    model = arch.build(cfg, rt)
    source = CheckpointFolder(model_dir)
    try:
        bind_weights(model, source, rt.act_dtype, rt.device)
    finally:
        source.close()
    return ModelRunner(model, rt, options, num_pages)


def build_runner_random(config_dict: Mapping[str, Any], seed: int, options: Optional[EngineOptions] = None,
                        std: float = 0.02, norm_std: float = 0.0, num_pages: Optional[int] = None) -> ModelRunner:
    """The same model with random weights drawn on the device (nothing is written)."""
    options = options or EngineOptions()
    arch = resolve_architecture(config_dict)
    cfg = arch.config_from_dict(config_dict)
    rt = _runtime(options)
    model = arch.build(cfg, rt)
    source = RandomWeights(model.all_param_specs(), seed, std, norm_std, torch.bfloat16, rt.device)
    bind_weights(model, source, rt.act_dtype, rt.device)
    return ModelRunner(model, rt, options, num_pages)
