"""Typed configuration of the Qwen2 dense decoder, read from config.json.

Keys and defaults follow LitInfer's loader
(python/llaisys/models/qwen2.py:243-299): ``num_key_value_heads`` defaults to
the number of heads, ``head_dim`` to hidden/heads, ``rms_norm_eps`` to 1e-6,
``rope_theta`` to 10000, ``eos_token_id`` may be an int or a list.  Keys that
LitInfer ignores but that change the mathematics are read and either honoured
(``tie_word_embeddings``, ``use_sliding_window`` / ``sliding_window`` /
``max_window_layers``) or refused with an error (``rope_scaling``, an
activation other than silu), never silently dropped.
"""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Tuple

from .spec import BlockSpec, ModelSpec, PartSpec, default_schedule


class ConfigError(ValueError):
    pass


def _positive_int(d: Mapping[str, Any], key: str, default: Optional[int] = None) -> int:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: missing key '{key}'")
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: '{key}' must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    attention_bias: Optional[bool]
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    eos_token_ids: Tuple[int, ...]
    torch_dtype: str
    architectures: Tuple[str, ...] = ("Qwen2ForCausalLM",)

    ARCHITECTURE = "Qwen2ForCausalLM"

    # ------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen2Config":
        hidden = _positive_int(d, "hidden_size")
        nh = _positive_int(d, "num_attention_heads")
        nkv = _positive_int(d, "num_key_value_heads", nh)
        if d.get("head_dim") is None:
            if hidden % nh:
                raise ConfigError(f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads {nh} and no head_dim is given")
            dh = hidden // nh
        else:
            dh = _positive_int(d, "head_dim")
        if nh % nkv:
            raise ConfigError(f"config.json: num_attention_heads {nh} is not a multiple of num_key_value_heads {nkv}")
        if dh % 2:
            raise ConfigError(f"config.json: head_dim {dh} must be even for rotary position encoding")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (silu only)")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: rope_scaling is not supported")
        eos = d.get("eos_token_id", None)
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        eos_ids = tuple(e for e in eos_ids if e >= 0)
        layers = _positive_int(d, "num_hidden_layers")
        use_win = bool(d.get("use_sliding_window", False))
        window = d.get("sliding_window", None)
        if use_win:
            if window is None:
                raise ConfigError("config.json: use_sliding_window is true but sliding_window is missing")
            window = _positive_int(d, "sliding_window")
        mwl = d.get("max_window_layers", layers)
        if isinstance(mwl, bool) or not isinstance(mwl, int) or mwl < 0:
            raise ConfigError(f"config.json: 'max_window_layers' must be a non-negative integer, got {mwl!r}")
        eps = float(d.get("rms_norm_eps", 1e-6))
        theta = float(d.get("rope_theta", 10000.0))
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {eps}")
        if not (theta > 0 and math.isfinite(theta)):
            raise ConfigError(f"config.json: rope_theta must be positive, got {theta}")
        archs = tuple(d.get("architectures") or (cls.ARCHITECTURE,))
        return cls(
            vocab_size=_positive_int(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_positive_int(d, "intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=dh,
            max_position_embeddings=_positive_int(d, "max_position_embeddings"),
            rms_norm_eps=eps,
            rope_theta=theta,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            # Qwen2's config.json has no such key: the q/k/v biases then follow the file, as in LitInfer, whose
            # loader does not require them (python/llaisys/models/qwen2.py:220-230)
            attention_bias=None if d.get("attention_bias") is None else bool(d["attention_bias"]),
            use_sliding_window=use_win,
            sliding_window=window if use_win else None,
            max_window_layers=mwl,
            eos_token_ids=eos_ids,
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            architectures=archs,
        )

    @classmethod
    def from_json(cls, path) -> "Qwen2Config":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        if not path.is_file():
            raise FileNotFoundError(f"config.json not found: {path}")
        return cls.from_dict(json.loads(path.read_text()))

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        eos = list(self.eos_token_ids)
        d.pop("eos_token_ids")
        d["eos_token_id"] = eos[0] if len(eos) == 1 else (eos if eos else None)
        d["hidden_act"] = "silu"
        d["model_type"] = "qwen2"
        if d["attention_bias"] is None:
            d.pop("attention_bias")
        return d

    # ------------------------------------------------------------------
    def layer_window(self, layer: int) -> Optional[int]:
        """Keys visible to a query on this layer (its own included), None for all."""
        if self.use_sliding_window and self.sliding_window is not None and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    def to_model_spec(self) -> ModelSpec:
        """Qwen2 as parts: pre-norm blocks of GQA attention (q/k/v bias, rotate-half
        RoPE, keys cached after rotation) and a dense SwiGLU feed-forward
        (src/llaisys/models/qwen2.cpp:272-316)."""
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        rope = PartSpec("rope", {"theta": self.rope_theta, "rotary_dim": self.head_dim, "pairing": "half"})
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
        blocks = []
        for i in range(self.num_hidden_layers):
            mixer = PartSpec(
                "attention",
                {
                    "hidden_size": self.hidden_size,
                    "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads,
                    "head_dim": self.head_dim,
                    "qkv_bias": self.attention_bias,
                    "out_bias": False,
                    "scale": 1.0 / math.sqrt(self.head_dim),
                    "window": self.layer_window(i),
                    "position": rope,
                },
            )
            blocks.append(BlockSpec.of("prenorm", f"model.layers.{i}.", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                       feed_forward_norm=norm))
        return ModelSpec(
            architecture=self.ARCHITECTURE,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            blocks=tuple(blocks),
            schedule=default_schedule(len(blocks)),
            final_norm=norm,
            tie_word_embeddings=self.tie_word_embeddings,
            max_position_embeddings=self.max_position_embeddings,
            eos_token_ids=self.eos_token_ids,
            # the other names LitInfer's loader takes (python/llaisys/models/qwen2.py:139-149)
            aliases={
                "model.embed_tokens.weight": ("transformer.wte.weight",),
                "lm_head.weight": ("model.lm_head.weight",),
                "model.norm.weight": ("transformer.ln_f.weight",),
            },
        )
