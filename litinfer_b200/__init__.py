"""litinfer_b200: a small, whole Qwen2 inference engine for one NVIDIA B200."""

__version__ = "0.1.0"
