"""litinfer_b200: a small, whole Qwen2 inference engine for one NVIDIA B200.

    from litinfer_b200 import Qwen2
    tokens = Qwen2(model_dir).generate(input_ids, max_new_tokens=32)
"""

__version__ = "0.1.0"

from .api import CausalLM, Qwen2, load_model
from .config import Qwen2Config, register_architecture
from .engine import Engine, EngineConfig, StepItem
from .models import DecoderModel
from .sampling import SamplingParams

__all__ = [
    "DecoderModel",
    "Engine",
    "EngineConfig",
    "CausalLM",
    "Qwen2",
    "Qwen2Config",
    "SamplingParams",
    "StepItem",
    "load_model",
    "register_architecture",
]
