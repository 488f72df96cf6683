"""lucciola_b200: a single-GPU inference engine for the Qwen3 dense decoder on B200.

    from lucciola_b200 import AsyncEngine, Engine, SamplingParams
"""
__version__ = "0.1.0"

from .config import EngineOptions, Qwen3Config  # noqa: E402,F401
from .sampling.params import SamplingParams  # noqa: E402,F401


def __getattr__(name):
    # The engines pull in torch.cuda paths; import them on first use.
    if name in ("Engine", "AsyncEngine"):
        from .engine import llm
        return getattr(llm, name)
    raise AttributeError(name)
