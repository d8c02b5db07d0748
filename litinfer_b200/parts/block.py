"""Arrangement of a layer's parts.  ``prenorm``: x += Mixer(norm(x));
x += FeedForward(norm(x)) (src/llaisys/models/qwen2.cpp:272-316).

The residual stream x is float32.  A block hands the output of its
feed-forward back as ``pending`` instead of adding it, so that the next block
(or the model's tail) adds it inside its first norm kernel: one pass over x
for add and norm together.
"""

from __future__ import annotations

from typing import List

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block


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

    def forward(self, x32, ctx, cache, pending):
        h = self.mixer_norm.forward(x32) if pending is None else self.mixer_norm.add_forward(x32, pending)
        a = self.mixer.forward(h, ctx, cache)
        h = self.feed_forward_norm.add_forward(x32, a)
        return x32, self.feed_forward.forward(h, ctx)
