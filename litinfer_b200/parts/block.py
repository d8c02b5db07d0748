"""Arrangement of a layer's parts.  ``prenorm``: x += Mixer(norm(x));
x += FeedForward(norm(x)) (src/llaisys/models/qwen2.cpp:272-316).

The residual stream x is float32.  A block does not add the output of its
last part itself: told the next block's entry (its first norm), it lets that part
add, and normalise for the next block, in the tail of its last product
(``Carry.normed``); otherwise it hands the output on (``Carry.delta``) and the next
block, or the model's tail, adds it inside its first norm kernel.  Either way
add and norm are one pass over x.

A block takes its parts from the roles of its :class:`~litinfer_b200.config.spec.BlockSpec`
(:meth:`Block.build`); ``prenorm`` wants ``mixer`` and ``mixer_norm`` and, unless the layer has
no feed-forward, ``feed_forward`` and ``feed_forward_norm``.
"""

from __future__ import annotations

from typing import List

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Carry, Tail


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.mixer_norm = self.build(NORMS, "mixer_norm")
        self.mixer = self.build(MIXERS, "mixer")
        self.feed_forward = self.build(FEED_FORWARDS, "feed_forward", required=False)
        self.feed_forward_norm = self.build(NORMS, "feed_forward_norm", required=self.feed_forward is not None)

    def parts(self) -> List:
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def entry(self):
        return Tail(None, self.mixer_norm, self.mixer.takes_deferred)

    def fused_decode(self):
        if type(self) is not PreNormBlock or self.feed_forward is None:
            return None
        mixer, ff = self.mixer.fused_decode(), self.feed_forward.fused_decode()
        n1, n2 = self.mixer_norm.fused_decode(), self.feed_forward_norm.fused_decode()
        if None in (mixer, ff, n1, n2) or mixer["hidden"] != ff["hidden"] or n1["size"] != mixer["hidden"] or n2["size"] != mixer["hidden"]:
            return None
        return dict(mixer, **ff, norm_first=n1, norm_ffn=n2)

    def forward(self, x32, ctx, cache, carry, next_entry=None):
        if carry is None:
            h = self.mixer_norm.forward(x32)
        elif carry.normed is not None:
            h = carry.normed                               # the block before applied this block's first norm
        else:
            h = self.mixer_norm.add_forward(x32, carry.delta)
        if self.feed_forward is None:
            if next_entry is None:
                return x32, Carry(delta=self.mixer.forward(h, ctx, cache))
            return x32, Carry(normed=self.mixer.forward_into(h, ctx, cache, Tail(x32, next_entry.norm, next_entry.defer)))
        h = self.mixer.forward_into(h, ctx, cache, Tail(x32, self.feed_forward_norm, self.feed_forward.takes_deferred))
        if next_entry is None:
            return x32, Carry(delta=self.feed_forward.forward(h, ctx))
        return x32, Carry(normed=self.feed_forward.forward_into(h, ctx, Tail(x32, next_entry.norm, next_entry.defer)))
