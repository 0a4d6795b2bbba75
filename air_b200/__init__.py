"""air_b200: a single-GPU inference engine for the Qwen2 dense decoder on NVIDIA B200."""
__version__ = "0.1.0"
