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
                 ``gather_forward(x32, rows) -> y[rows]``; ``after_linear(linear, a, x32) -> y``
                 (x32 += linear(a) first; a norm may run it as one kernel with the product)
* position:      owns what the mixer needs to encode positions (tables, constants)
* mixer:         ``forward(h, ctx, cache) -> y``; ``cache_requirement()``;
                 optionally ``forward_into(h, ctx, cache, tail) -> h'``
* feed-forward:  ``forward(h, ctx) -> y``; optionally ``forward_into(h, ctx, tail) -> h'``
* block:         ``forward(x32, ctx, cache, carry, next_norm) -> (x32, carry)``; ``first_norm``

A :class:`Tail` says what follows a part's output: it is added to the residual stream and the
sum is normalised for the next part.  ``forward_into`` does all of that and returns the
normalised sum; the default calls ``forward`` and then the norm's ``add_forward``, and a part
whose last step is a product may hand it to the norm's ``after_linear`` instead.  If the part
that comes next says ``takes_deferred``, the norm may return a :class:`Deferred` activation:
the weighted sum with the reciprocal root still to be applied, which that part's first product
applies to its own result (``FusedLinear`` does), so that the norm costs no kernel.  A
:class:`Carry` is what a block hands to the next one: its last output not yet added to the
stream (``delta``), or, when it was told the next block's entry, the stream already
updated and normalised by that block's first norm (``normed``).

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

    def fused_decode(self) -> Optional[dict]:
        """What the fused decode step (``models/fused_decode.py``) needs of this part, tensors and constants under the
        names that file reads, or None: the part is not one the fused kernel is built for, and a model that holds it
        runs part by part.  The default is None, so that parts registered from outside are never fused by accident."""
        return None

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


@dataclass
class Deferred:
    """A normalised activation not yet multiplied out: ``h[t] / sqrt(sum_p ssq[t, p] / width + eps)``.

    ``h`` already holds the norm's weights.  A product applies the factor to its rows
    (``kernels.linear(..., row_scale=d.row_scale)``); :meth:`materialize` gives the activation itself."""

    h: torch.Tensor
    ssq: torch.Tensor
    width: int
    eps: float

    @property
    def row_scale(self):
        return (self.ssq, self.width, self.eps)

    @property
    def shape(self):
        return self.h.shape

    def materialize(self) -> torch.Tensor:
        from .. import kernels as K

        out = torch.empty_like(self.h)
        K.apply_row_scale(self.h, self.ssq, self.width, self.eps, out)
        return out


@dataclass
class Tail:
    """What follows a part's output y: ``x32 += y``, then ``norm`` of the sum feeds the next part, which may
    (``defer``) be given a :class:`Deferred` activation."""

    x32: torch.Tensor
    norm: "Norm"
    defer: bool = False

    def apply(self, y: torch.Tensor) -> torch.Tensor:
        return self.norm.add_forward(self.x32, y)

    def apply_linear(self, linear, a: torch.Tensor):
        """The same for y = linear(a), which the norm may fuse with the product."""
        return self.norm.after_linear(linear, a, self.x32, defer=self.defer)


@dataclass
class Carry:
    """From one block to the next: ``delta`` is still to be added to the residual stream;
    ``normed`` is the next block's first norm of the stream, which already holds everything."""

    delta: Optional[torch.Tensor] = None
    normed: Optional[torch.Tensor] = None


class Mixer(Part):
    takes_deferred = False           # whether forward accepts a Deferred activation as h
    # how many CTAs one entry of the step's attention work list becomes in this mixer's kernel (0: it does not read the
    # list); the step function sizes the list so that the entries of all such mixers fill the GPU (engine.batch.attention_units)
    ctas_per_work_unit = 0
    # A mixer with state of its own (FixedState) advances that state every time it runs, so the step function never
    # splits its portions and captures nothing of its model, unless the mixer sets this: it promises that in a step of
    # single tokens (ctx.max_q_len == 1: token s is sequence s) it reads the step only through the context's device
    # tensors (ctx.state_slots and the like) and launches the same kernels whatever they hold.  Such steps are then
    # captured and replayed like those of a model without state; the runs that warm a capture up point every sequence at
    # the spare slot (the one that padded sequences of a captured step name), so they advance nobody's state.
    decodes_from_device = False

    def cache_requirement(self):
        """PagedKV, FixedState or None."""
        return None

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError

    def forward_into(self, h: torch.Tensor, ctx, cache, tail: Tail) -> torch.Tensor:
        return tail.apply(self.forward(h, ctx, cache))


class FeedForward(Part):
    takes_deferred = False

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError

    def forward_into(self, h: torch.Tensor, ctx, tail: Tail) -> torch.Tensor:
        return tail.apply(self.forward(h, ctx))


class Norm(Part):
    def forward(self, x32: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, x32: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def gather_forward(self, x32: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def after_linear(self, linear, a: torch.Tensor, x32: torch.Tensor, defer: bool = False):
        """``x32 += linear(a)``; the norm of the sum, which may be :class:`Deferred` if ``defer``.
        ``linear`` is a :class:`~litinfer_b200.parts.linear.FusedLinear`."""
        return self.add_forward(x32, linear(a))


@dataclass
class Rotary:
    """What a mixer's kernels need to rotate queries and keys of this step: pair ``j`` of the first ``rotary_dim``
    elements of a head turns by ``position / denominators[j]``; ``table`` (or None) holds the cosines and sines
    of the step's tokens, ``[tokens, rotary_dim / 2, 2]`` float32, for kernels that rotate in an epilogue."""

    denominators: torch.Tensor
    rotary_dim: int
    table: Optional[torch.Tensor] = None


class Position(Part):
    """A position encoding.  It serves a mixer (``PartSpec`` of the mixer names it) or the whole model
    (``ModelSpec.position``), and says what it does through these methods; the defaults do nothing, so a
    part overrides only what it is.

    * :meth:`rotary`: for encodings that rotate queries and keys (the mixer hands the answer to its kernels);
      ``None`` means "rotate nothing": keys and values still go into the cache.
    * :meth:`add_to_stream`: for encodings that are added to the residual stream after the embedding
      (learned absolute positions); only called on the model's own position part.
    """

    def rotary(self, ctx) -> Optional[Rotary]:
        return None

    def add_to_stream(self, x32: torch.Tensor, ctx) -> None:
        return None


class Block(Part):
    """``spec`` is a :class:`~litinfer_b200.config.spec.BlockSpec`: parts by role."""

    def build(self, registry: "Registry", role: str, required: bool = True, **extra):
        """The part under ``role`` of this block's spec, built from ``registry``; None if the spec has none and it
        is not required."""
        part = self.spec.part(role)
        if part is None:
            if required:
                raise ValueError(f"block '{self.spec.kind}' at {self.spec.prefix!r} needs a part under the role '{role}'; "
                                 f"the spec has: {', '.join(sorted(self.spec.parts)) or 'none'}")
            return None
        return registry.build(part, self.spec.prefix_of(role), self.dtype, self.device, **extra)

    def cache_requirement(self):
        """What this block's schedule entry needs from the cache manager: by default its mixer's."""
        mixer = getattr(self, "mixer", None)
        return mixer.cache_requirement() if mixer is not None else None

    def entry(self) -> Optional[Tail]:
        """The norm this block applies to the residual stream first, and whether its consumer takes a deferred
        activation, as a Tail without a stream; None if the block before may not apply it in this block's place."""
        return None

    def forward(self, x32, ctx, cache, carry: Optional[Carry], next_entry: Optional[Tail] = None):
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
