"""lucciola_b200: a single-GPU inference engine for the Qwen3 dense decoder on B200."""
__version__ = "0.1.0"
