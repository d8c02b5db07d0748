from .decoder import DecoderModel, declared_params, run_dtype

__all__ = ["DecoderModel", "declared_params", "run_dtype"]
