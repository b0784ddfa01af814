"""A block whose norms sit behind its sublayers, with learned row scales:

    h += s1 * N1(mixer(h))
    h += s2 * N2(feed_forward(h))           if the layer has a feed-forward

The sublayers read the stream itself (in the storage dtype for their matrix products); the stream stays 32-bit.  One
kernel per sublayer norms its output, scales it, adds it to the stream and writes the stream in the storage dtype
for whoever reads it next: the feed-forward, or the next layer's mixer, to which it is handed on as a ``CastStream``.
"""

from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, CastStream, NormedDelta
from .norm import LayerNorm


@BLOCKS.register("postnorm")
class PostNormBlock(Block):
    @classmethod
    def declare(cls, spec, prefix=None):
        p = spec.prefix
        hidden = spec.mixer_post_norm.size
        d = MIXERS.get(spec.mixer.kind).declare(spec.mixer, p) + NORMS.get(spec.mixer_post_norm.kind).declare(spec.mixer_post_norm, p)
        if spec.mixer_scale:
            d.append(TensorDecl(p + spec.mixer_scale, (hidden,), init="one_plus_normal"))
        if spec.feed_forward is not None:
            d += FEED_FORWARDS.get(spec.feed_forward.kind).declare(spec.feed_forward, p)
            d += NORMS.get(spec.feed_forward_post_norm.kind).declare(spec.feed_forward_post_norm, p)
            if spec.feed_forward_scale:
                d.append(TensorDecl(p + spec.feed_forward_scale, (hidden,), init="one_plus_normal"))
        return d

    def __init__(self, spec, weights, prefix, rt):
        p = spec.prefix
        self.spec, self.rt = spec, rt
        f32 = lambda n: weights[p + n].to(torch.float32).contiguous()
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, weights, p, rt)
        self.mixer_post_norm = NORMS.get(spec.mixer_post_norm.kind)(spec.mixer_post_norm, weights, p, rt)
        self.mixer_scale = f32(spec.mixer_scale) if spec.mixer_scale else None
        self.feed_forward = self.feed_forward_post_norm = self.feed_forward_scale = None
        if spec.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, weights, p, rt)
            self.feed_forward_post_norm = NORMS.get(spec.feed_forward_post_norm.kind)(spec.feed_forward_post_norm, weights, p, rt)
            self.feed_forward_scale = f32(spec.feed_forward_scale) if spec.feed_forward_scale else None
        for n in (self.mixer_post_norm, self.feed_forward_post_norm):
            if n is not None and not isinstance(n, LayerNorm):
                raise ValueError("a post-norm layer's norms must be layer norms (its kernel norms, scales and adds in one pass)")

    def _behind(self, h, y, norm, scale):
        """``h += scale * norm(y)``; returns the stream in the storage dtype."""
        return self.rt.kernels.post_layernorm(h, y, norm.weight, norm.bias, scale, norm.spec.eps, cast=True)

    def forward(self, h, pending, ctx, kv, state, writes_cache: bool):
        if isinstance(pending, CastStream):
            x = pending.x
        else:                                     # behind a block of another kind: add what it left, then cast
            if isinstance(pending, NormedDelta):
                pending.add_into(h, self.rt.kernels)
            elif pending is not None:
                h += pending.sum(dim=0)
            x = h.to(self.rt.dtype)
        y = self.mixer.forward(x, ctx, kv, state, writes_cache)
        x = self._behind(h, y[0], self.mixer_post_norm, self.mixer_scale)
        if self.feed_forward is not None:
            y = self.feed_forward.forward(x, ctx)
            x = self._behind(h, y[0], self.feed_forward_post_norm, self.feed_forward_scale)
        return h, CastStream(x)
