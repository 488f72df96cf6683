"""Options of the engine (not of the model).

Names follow lucciola where it has them: `max_blocks` and `block_size` are the
constructor arguments of its AsyncEngine (include/async_engine.h:24-25), with
max_blocks = 0 meaning "as many pages as fit" (src/qwen.cc:527-557: free
memory minus a reserve, times 0.9).  Its token budget of a step is the
constant 512 + 64 (src/scheduler.cc:48); here it is `max_tokens_per_step`.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"            # "bfloat16" or "float32" (true 32-bit everywhere)
    block_size: int = 16               # tokens in a page of the key/value cache
    max_blocks: int = 0                # pages in each cache group; 0 = from free memory
    mem_fraction: float = 0.90         # share of free memory for pages when max_blocks == 0
    max_tokens_per_step: int = 576     # token budget of one step (decoded tokens count first)
    prefill_chunk: int = 0             # largest portion of one prompt in a step; 0 = the budget
    token_tile: int = 0                # > 1: portions are shortened so that a step's tokens fill whole tiles of this many
    max_num_seqs: int = 256            # most requests that run at a time
    max_model_len: int = 0             # longest sequence; 0 = max_position_embeddings
    use_cuda_graph: bool = True        # record steps whose shape comes again as CUDA graphs and replay them
    graph_after: int = 2               # a step with portions of prompts is recorded when its shape has come this often
    max_shape_graphs: int = 32         # recordings of steps with portions kept at a time (least recently used goes)
    device: str = "cuda:0"

    def validate(self) -> None:
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")
        if self.block_size <= 0:
            raise ValueError(f"block_size must be positive, got {self.block_size}")
        if self.max_blocks < 0:
            raise ValueError(f"max_blocks must not be negative, got {self.max_blocks}")
        if not (0.0 < self.mem_fraction <= 1.0):
            raise ValueError(f"mem_fraction must be in (0, 1], got {self.mem_fraction}")
        if self.max_tokens_per_step <= 0 or self.max_num_seqs <= 0:
            raise ValueError("max_tokens_per_step and max_num_seqs must be positive")
        if self.graph_after < 1 or self.max_shape_graphs < 1:
            raise ValueError("graph_after and max_shape_graphs must be at least 1")
        if self.prefill_chunk < 0 or self.max_model_len < 0 or self.token_tile < 0:
            raise ValueError("prefill_chunk, max_model_len and token_tile must not be negative")
