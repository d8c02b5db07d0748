"""Architecture-neutral description of a decoder: what the parts are built from.

A model configuration (config.json of some architecture) is translated once
into a :class:`ModelSpec`.  Everything below the configuration layer — parts,
cache manager, step function, weight loader — reads only these specs, so no
part knows which architecture it serves.

* :class:`PartSpec`: ``kind`` (a name in one of the part registries) plus the
  sizes and constants of that part.  Parameters are free-form so that a part
  registered from outside the package can carry its own.
* :class:`BlockSpec`: how mixer, feed-forward and norms are arranged in one
  layer, and the tensor-name prefix of each.
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


@dataclass(frozen=True)
class BlockSpec:
    """One layer: an arrangement (``kind``) of a mixer, a feed-forward and norms.

    ``prefix`` is the tensor-name prefix of the layer (for instance
    ``model.layers.3.``); each part's own prefix below is appended to it.
    """

    kind: str
    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."


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
