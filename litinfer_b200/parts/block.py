"""Arrangement of a layer's parts.  ``prenorm``: x += Mixer(norm(x));
x += FeedForward(norm(x)) (src/llaisys/models/qwen2.cpp:272-316).

The residual stream x is float32.  A block does not add the output of its
feed-forward itself: told the next block's entry (its first norm), it lets the feed-forward
add, and normalise for the next block, in the tail of its last product
(``Carry.normed``); otherwise it hands the output on (``Carry.delta``) and the next
block, or the model's tail, adds it inside its first norm kernel.  Either way
add and norm are one pass over x.
"""

from __future__ import annotations

from typing import List

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Carry, Tail


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec, prefix, dtype, device):
        # ``spec`` is a BlockSpec here
        self.spec = spec
        self.prefix = prefix
        self.dtype = dtype
        self.device = device
        p = spec.prefix
        self.mixer_norm = NORMS.build(spec.mixer_norm, p + spec.mixer_norm_prefix, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, p + spec.mixer_prefix, dtype, device)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, p + spec.feed_forward_norm_prefix, dtype, device)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, p + spec.feed_forward_prefix, dtype, device)

    def parts(self) -> List:
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def entry(self):
        return Tail(None, self.mixer_norm, self.mixer.takes_deferred)

    def forward(self, x32, ctx, cache, carry, next_entry=None):
        if carry is None:
            h = self.mixer_norm.forward(x32)
        elif carry.normed is not None:
            h = carry.normed                               # the block before applied this block's first norm
        else:
            h = self.mixer_norm.add_forward(x32, carry.delta)
        h = self.mixer.forward_into(h, ctx, cache, Tail(x32, self.feed_forward_norm, self.feed_forward.takes_deferred))
        if next_entry is None:
            return x32, Carry(delta=self.feed_forward.forward(h, ctx))
        return x32, Carry(normed=self.feed_forward.forward_into(h, ctx, Tail(x32, next_entry.norm, next_entry.defer)))
