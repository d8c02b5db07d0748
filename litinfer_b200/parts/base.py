"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a :class:`~litinfer_b200.config.spec.PartSpec` (its sizes
and constants), a tensor-name prefix, the run dtype and the device.  It

* declares its tensors (:meth:`Part.params`) so that loader and random
  initialisation need no knowledge of it,
* receives them once (:meth:`Part.bind`), where it may fuse or re-lay them,
* and runs on the tokens of one step (``forward``).

Registries map ``PartSpec.kind`` to a class.  Registering a class from outside
the package is all it takes to make a new kind available to configurations.

Interfaces:

* norm:          ``forward(x32) -> y``; ``add_forward(x32, delta) -> y`` (x32 += delta first);
                 ``gather_forward(x32, rows) -> y[rows]``
* position:      owns what the mixer needs to encode positions (tables, constants)
* mixer:         ``forward(h, ctx, cache) -> y``; ``cache_requirement()``
* feed-forward:  ``forward(h, ctx) -> y``
* block:         ``forward(x32, ctx, cache, pending) -> (x32, pending)``

``x32`` is the residual stream, always float32 ``[tokens, hidden]``; ``h`` and
``y`` are activations in the run dtype.  ``ctx`` is the step's
:class:`~litinfer_b200.engine.batch.StepContext`, ``cache`` the
:class:`~litinfer_b200.cache.manager.EntryCache` of the schedule entry.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple, Type

import torch

from ..config.spec import PartSpec
from ..weights.loader import ParamSpec


# --------------------------------------------------------------------------
# what a mixer needs from the cache manager
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every token (or of the last ``window``), in pages."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """Per-request state of fixed size, held in a slot: ``shape`` elements of ``dtype``."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# --------------------------------------------------------------------------
# base class
# --------------------------------------------------------------------------

class Part:
    def __init__(self, spec: PartSpec, prefix: str, dtype: torch.dtype, device) -> None:
        self.spec = spec
        self.prefix = prefix
        self.dtype = dtype
        self.device = torch.device(device)

    def params(self) -> List[ParamSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take this part's tensors out of ``tensors`` (keyed by full name)."""

    def parts(self) -> List["Part"]:
        """Sub-parts, so that params() and bind() reach them."""
        return []

    # helpers -----------------------------------------------------------
    def all_params(self) -> List[ParamSpec]:
        out = list(self.params())
        for p in self.parts():
            out.extend(p.all_params())
        return out

    def bind_all(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.bind(tensors)
        for p in self.parts():
            p.bind_all(tensors)


class Mixer(Part):
    def cache_requirement(self):
        """PagedKV, FixedState or None."""
        return None

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, x32: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, x32: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def gather_forward(self, x32: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Position(Part):
    pass


class Block(Part):
    def forward(self, x32, ctx, cache, pending):
        raise NotImplementedError


# --------------------------------------------------------------------------
# registries
# --------------------------------------------------------------------------

class Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._kinds: Dict[str, Type[Part]] = {}

    def register(self, kind: str, cls: Optional[Type[Part]] = None):
        def put(c):
            self._kinds[kind] = c
            return c

        return put(cls) if cls is not None else put

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def kinds(self):
        return sorted(self._kinds)

    def build(self, spec: PartSpec, prefix: str, dtype: torch.dtype, device, **extra) -> Part:
        try:
            cls = self._kinds[spec.kind]
        except KeyError:
            raise KeyError(f"no {self.what} of kind '{spec.kind}' is registered; known: {', '.join(self.kinds())}") from None
        return cls(spec, prefix, dtype, device, **extra)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
