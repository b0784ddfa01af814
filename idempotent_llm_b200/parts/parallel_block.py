"""A block whose mixer and feed-forward read the same rows: ``h += mixer(norm1(h)) + feed_forward(norm2(h))``.

Both norms are taken from the stream as it stands before the layer, in one pass over the row (one root mean
square, two weights); the two outputs are added to the 32-bit stream, by the products' own epilogues where the parts
can do that, else as pending deltas that the next norm adds.  A constant row of the mixer's output (its output
projections' biases: ``mixer.stream_bias``) is added to the stream by the same pass that takes the norms.  Without a
feed-forward the layer is ``h += mixer(norm1(h))``.
"""

from __future__ import annotations

import torch

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, NormedDelta
from .norm import RMSNorm


@BLOCKS.register("parallel_residual")
class ParallelResidualBlock(Block):
    @classmethod
    def declare(cls, spec, prefix=None):
        p = spec.prefix
        d = (NORMS.get(spec.mixer_norm.kind).declare(spec.mixer_norm, p + spec.mixer_norm_prefix)
             + MIXERS.get(spec.mixer.kind).declare(spec.mixer, p))
        if spec.feed_forward is None:
            return d
        return (d + NORMS.get(spec.feed_forward_norm.kind).declare(spec.feed_forward_norm,
                                                                   p + spec.feed_forward_norm_prefix)
                + FEED_FORWARDS.get(spec.feed_forward.kind).declare(spec.feed_forward, p))

    def __init__(self, spec, weights, prefix, rt):
        p = spec.prefix
        self.spec, self.rt = spec, rt
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, weights, p + spec.mixer_norm_prefix, rt)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, weights, p, rt)
        self.feed_forward_norm = self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = NORMS.get(spec.feed_forward_norm.kind)(
                spec.feed_forward_norm, weights, p + spec.feed_forward_norm_prefix, rt)
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, weights, p, rt)
        # one pass for both norms where both are RMS norms with the same eps
        n1, n2 = self.mixer_norm, self.feed_forward_norm
        self.joint = isinstance(n1, RMSNorm) and (n2 is None or (isinstance(n2, RMSNorm) and n2.spec.eps == n1.spec.eps))

    def forward(self, h, pending, ctx, kv, state, writes_cache: bool):
        K = self.rt.kernels
        bias = getattr(self.mixer, "stream_bias", None)
        if isinstance(pending, NormedDelta):
            pending.add_into(h, K)
            pending = None
        if self.joint:
            x1, x2 = K.add_rmsnorm2(h, pending, self.mixer_norm.weight,
                                    None if self.feed_forward_norm is None else self.feed_forward_norm.weight,
                                    self.mixer_norm.spec.eps, post=bias)
        else:
            x1 = self.mixer_norm.forward(h, pending, ctx)
            x2 = None if self.feed_forward_norm is None else self.feed_forward_norm.forward(h, None, ctx)
            if bias is not None:
                h += bias
        kw = {"bias_in_stream": True} if bias is not None else {}
        if getattr(self.mixer, "accepts_residual", False):
            kw["residual"] = h
        deltas = [self.mixer.forward(x1, ctx, kv, state, writes_cache, **kw)]
        if self.feed_forward is not None:
            if getattr(self.feed_forward, "accepts_residual", False):
                deltas.append(self.feed_forward.forward(x2, ctx, residual=h))
            else:
                deltas.append(self.feed_forward.forward(x2, ctx))
        deltas = [d for d in deltas if d is not None]
        if not deltas:
            return h, None
        return h, deltas[0] if len(deltas) == 1 else torch.cat(deltas, dim=0)
