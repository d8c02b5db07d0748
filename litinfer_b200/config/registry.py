"""One registry from an architecture's name (config.json ``architectures[0]``)
to its configuration class.  The configuration class turns config.json into a
:class:`~litinfer_b200.config.spec.ModelSpec`; the model itself is always the
generic decoder assembled from registered parts.

LitInfer has no registry: its caller imports the one model class
(python/llaisys/models/__init__.py:1) and ``architectures`` is never read.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, Mapping, Type

from .qwen2 import ConfigError, Qwen2Config
from .spec import ModelSpec

_ARCHITECTURES: Dict[str, Type] = {}


def register_architecture(name: str, config_cls: Type) -> None:
    """``config_cls`` needs ``from_dict(mapping)`` and ``to_model_spec()``."""
    for attr in ("from_dict", "to_model_spec"):
        if not hasattr(config_cls, attr):
            raise TypeError(f"configuration class for '{name}' lacks {attr}()")
    _ARCHITECTURES[name] = config_cls


def supported_architectures():
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> Type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"architecture '{name}' is not supported; supported: {', '.join(supported_architectures())}"
        ) from None


def config_from_dict(d: Mapping[str, Any]):
    archs = d.get("architectures")
    if not archs:
        raise ConfigError("config.json: missing key 'architectures'")
    return config_class_for(archs[0]).from_dict(d)


def load_config(model_dir):
    path = Path(model_dir)
    if path.is_dir():
        path = path / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"config.json not found: {path}")
    return config_from_dict(json.loads(path.read_text()))


def model_spec_from_dir(model_dir) -> ModelSpec:
    return load_config(model_dir).to_model_spec()


register_architecture(Qwen2Config.ARCHITECTURE, Qwen2Config)
