"""Token embeddings other than the plain lookup (a part kind of its own: ``EMBEDDINGS``).

``bigram_hash``: ``h_t = E[token_t] + B[r_t]`` with ``r_t = (mul_prev * token_(t-1) + mul_cur * token_t) mod buckets``
and ``r = buckets`` (the last row of ``B``) for a sequence's first token.  The token before a step's first one is part
of the sequence's state: one integer per slot, kept where the cache keeps per-sequence state, so that it is zeroed,
snapshot and put back with the mixers' state and a step may cut a sequence anywhere.  One kernel looks both rows up,
adds them in 32-bit, moves the state on and also leaves the stream in the storage dtype for a first sublayer that
reads the stream itself.
"""

from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from ..weights.loader import TensorDecl
from .base import EMBEDDINGS, CastStream, Part


@EMBEDDINGS.register("bigram_hash")
class BigramHashEmbedding(Part):
    @classmethod
    def declare(cls, spec, prefix=""):
        return [TensorDecl(prefix + spec.table, (spec.buckets + 1, spec.hidden))]

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kind="none", state_shape=(1,), state_dtype=torch.int32)

    def __init__(self, spec, weights, prefix, rt):
        if spec.buckets <= 0 or spec.mul_prev < 0 or spec.mul_cur < 0:
            raise ValueError(f"bigram embedding: buckets={spec.buckets}, factors {spec.mul_prev}, {spec.mul_cur}")
        self.spec, self.rt = spec, rt
        self.table = weights[prefix + spec.table].to(rt.dtype).contiguous()

    def forward(self, embed_table, ctx, state):
        """Returns the 32-bit stream and, as what is pending, the same rows in the storage dtype."""
        s = self.spec
        h, x = self.rt.kernels.embed_bigram(ctx, embed_table, self.table, state, s.buckets, s.mul_prev, s.mul_cur, cast=True)
        return h, CastStream(x)
