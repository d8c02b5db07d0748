"""Architecture-neutral description of a decoder: what the parts are built from.

A model configuration (config.json of some architecture) is translated once
into a :class:`ModelSpec`.  Everything below the configuration layer — parts,
cache manager, step function, weight loader — reads only these specs, so no
part knows which architecture it serves.

* :class:`PartSpec`: ``kind`` (a name in one of the part registries) plus the
  sizes and constants of that part.  Parameters are free-form so that a part
  registered from outside the package can carry its own.
* :class:`BlockSpec`: which parts one layer has, under which role names, how
  they are arranged (``kind``) and the tensor-name prefix of each.
* :class:`ScheduleEntry`: one run of a block.  The schedule is data: a block
  may appear twice, and an entry may read the cache of an earlier entry
  instead of owning one.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple


@dataclass(frozen=True)
class PartSpec:
    """``kind`` selects the implementation; ``params`` are its sizes and constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def replace(self, **changes: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(changes)
        return PartSpec(self.kind, merged)


# The four parts of a pre-norm decoder layer and LitInfer's tensor-name stems for them
# (python/llaisys/models/qwen2.py:156-190).  Other arrangements name their own roles.
DEFAULT_PREFIXES = {
    "mixer": "self_attn.",
    "feed_forward": "mlp.",
    "mixer_norm": "input_layernorm.",
    "feed_forward_norm": "post_attention_layernorm.",
}


@dataclass(frozen=True)
class BlockSpec:
    """One layer: an arrangement (``kind``) of parts, each under a role name.

    ``parts`` maps a role (``mixer``, ``feed_forward``, ``mixer_norm``, ``feed_forward_norm``, or whatever else
    the arrangement knows: a norm after the mixer, a second mixer) to the part's spec; ``prefixes`` maps a role
    to the part's tensor-name prefix below the layer's own ``prefix`` (for instance ``model.layers.3.``), with
    ``<role>.`` as the default for roles outside :data:`DEFAULT_PREFIXES`.  An arrangement takes the roles it
    wants and may do without any of them (a layer without a feed-forward has no such entry).
    """

    kind: str
    prefix: str
    parts: Mapping[str, PartSpec] = field(default_factory=dict)
    prefixes: Mapping[str, str] = field(default_factory=dict)

    @classmethod
    def of(cls, kind: str, prefix: str, prefixes: Optional[Mapping[str, str]] = None, **parts: Optional[PartSpec]) -> "BlockSpec":
        """``BlockSpec.of("prenorm", "model.layers.0.", mixer=..., feed_forward=..., mixer_norm=..., feed_forward_norm=...)``."""
        return cls(kind, prefix, {r: p for r, p in parts.items() if p is not None}, dict(prefixes or {}))

    def part(self, role: str) -> Optional[PartSpec]:
        return self.parts.get(role)

    def prefix_of(self, role: str) -> str:
        """Full tensor-name prefix of the part under ``role``."""
        return self.prefix + self.prefixes.get(role, DEFAULT_PREFIXES.get(role, role + "."))

    def with_part(self, role: str, spec: Optional[PartSpec], prefix: Optional[str] = None) -> "BlockSpec":
        """A copy with the part under ``role`` replaced (``None`` removes it) and, if given, its prefix."""
        parts = dict(self.parts)
        if spec is None:
            parts.pop(role, None)
        else:
            parts[role] = spec
        prefixes = dict(self.prefixes)
        if prefix is not None:
            prefixes[role] = prefix
        return BlockSpec(self.kind, self.prefix, parts, prefixes)

    def with_kind(self, kind: str) -> "BlockSpec":
        return BlockSpec(kind, self.prefix, dict(self.parts), dict(self.prefixes))


@dataclass(frozen=True)
class ScheduleEntry:
    """Run block ``block``.  ``cache_from`` None: this entry owns a cache (or
    state); otherwise it reads what schedule entry ``cache_from`` wrote in
    this step and writes nothing."""

    block: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_ids: Tuple[int, ...] = ()
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    lm_head_name: str = "lm_head.weight"
    # a position encoding of the whole model, applied to the residual stream right after the embedding (learned
    # absolute positions, say); None: positions are the mixers' business
    position: Optional[PartSpec] = None
    position_prefix: str = "model."
    # factor on the embedding rows and cap of the logits (cap * tanh(logits / cap)); None: neither
    embedding_scale: Optional[float] = None
    logit_cap: Optional[float] = None
    # other names under which a declared tensor may be stored: declared name -> names tried after it
    aliases: Mapping[str, Tuple[str, ...]] = field(default_factory=dict)

    def with_schedule(self, schedule: Sequence[ScheduleEntry]) -> "ModelSpec":
        from dataclasses import replace

        return replace(self, schedule=tuple(schedule))


def default_schedule(num_blocks: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(i) for i in range(num_blocks))


def validate_schedule(spec: ModelSpec) -> None:
    for i, e in enumerate(spec.schedule):
        if not 0 <= e.block < len(spec.blocks):
            raise ValueError(f"schedule entry {i} names block {e.block}, the model has {len(spec.blocks)}")
        if e.cache_from is not None:
            if not 0 <= e.cache_from < i:
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_from}, which does not run before it")
            if spec.schedule[e.cache_from].cache_from is not None:
                raise ValueError(f"schedule entry {i} reads entry {e.cache_from}, which owns no cache itself")
