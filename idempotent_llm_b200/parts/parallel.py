"""Several mixers side by side on one input: ``sum_b scale_b * mixer_b(h)`` (a mixer).

Every branch is a registered mixer with a spec of its own.  The branches' input projections are one matrix
product (their matrices' rows one after another) and so are their output projections: each branch writes its
activations, times its constant, into its columns of one buffer, and the product of that buffer with the
branches' output matrices side by side is the weighted sum.  A branch therefore has, beside ``forward``:

    in_weight  [rows, hidden]     its input projections' rows, in the order its kernels expect
    out_weight [hidden, inner]    its output projection
    inner                         columns of its activations
    mix(proj, col0, ctx, kv, state, out, out_col, out_scale)
    out_bias                      optional: a 32-bit row [hidden] its output projection adds

The branches' biases, each times its branch's constant, are one constant row ``stream_bias``.  A block that knows of
it adds it to the stream itself (``bias_in_stream=True``); for any other caller the mixer adds it to its delta.  Given
``residual``, the output product adds into the stream in its epilogue where the kernels can.

What the branches keep is merged into one cache entry: the keys and values of the one branch that has some,
and one per-sequence state region in which every branch has its own columns.
"""

from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from .base import MIXERS, Mixer


def _state_floats(need: CacheNeed) -> int:
    if need.state_shape is None:
        return 0
    if need.state_dtype != torch.float32:
        raise ValueError("the branches of a parallel mixer keep 32-bit state")
    n = 1
    for d in need.state_shape:
        n *= int(d)
    return n


@MIXERS.register("parallel")
class ParallelMixer(Mixer):
    accepts_residual = True

    @classmethod
    def declare(cls, spec, prefix):
        d = []
        for b in spec.branches:
            d += MIXERS.get(b.mixer.kind).declare(b.mixer, prefix + spec.prefix + b.prefix)
        return d

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        needs = [MIXERS.get(b.mixer.kind).cache_need(b.mixer) for b in spec.branches]
        with_kv = [n for n in needs if n.kind != "none"]
        if len(with_kv) > 1:
            raise ValueError("at most one branch of a parallel mixer keeps keys and values")
        total = sum(_state_floats(n) for n in needs)
        kv = with_kv[0] if with_kv else CacheNeed()
        return CacheNeed(kind=kv.kind, n_kv_heads=kv.n_kv_heads, head_dim=kv.head_dim, window=kv.window,
                         k_row=kv.k_row, v_row=kv.v_row, state_shape=(total,) if total else None)

    def __init__(self, spec, weights, prefix, rt):
        self.spec, self.rt = spec, rt
        self.branches, self.scales, self.state_cols, self._rows = [], [], [], []
        off = 0
        for b in spec.branches:
            cls = MIXERS.get(b.mixer.kind)
            part = cls(b.mixer, weights, prefix + spec.prefix + b.prefix, rt)
            for attr in ("in_weight", "out_weight", "inner", "mix"):
                if not hasattr(part, attr):
                    raise ValueError(f"{cls.__name__} cannot be a branch of a parallel mixer: it has no {attr}")
            n = _state_floats(cls.cache_need(b.mixer))
            self.branches.append(part)
            self.scales.append(float(b.scale))
            self._rows.append(part.in_weight.shape[0])
            self.state_cols.append((off, off + n))
            off += n
        self.in_weight = torch.cat([p.in_weight for p in self.branches], dim=0).contiguous()
        self.out_weight = torch.cat([p.out_weight for p in self.branches], dim=1).contiguous()
        self.inner = sum(p.inner for p in self.branches)
        for p in self.branches:                     # the joint matrices are the ones that are read
            p.in_weight = p.out_weight = None
        self.graph_safe = all(getattr(p, "graph_safe", True) for p in self.branches)
        self.stream_bias = None
        for p, scale in zip(self.branches, self.scales):
            b = getattr(p, "out_bias", None)
            if b is not None:
                b = b.to(torch.float32) * scale
                self.stream_bias = b if self.stream_bias is None else self.stream_bias + b
        self._aligned = spec.hidden % 8 == 0 and self.inner % 8 == 0

    def forward(self, x, ctx, kv, state, writes_cache: bool, residual=None, bias_in_stream: bool = False):
        K = self.rt.kernels
        proj = K.gemm_store(x, self.in_weight, pad=True)                       # 32-bit [N, all branches' rows]
        out = torch.empty((x.shape[0], self.inner), dtype=self.rt.dtype, device=x.device)
        col0 = out_col = 0
        for p, scale, (a, b), rows in zip(self.branches, self.scales, self.state_cols, self._rows):
            p.mix(proj, col0, ctx, kv, state[:, a:b] if b > a else None, out, out_col, scale)
            col0 += rows
            out_col += p.inner
        add_bias = self.stream_bias is not None and not bias_in_stream
        if residual is not None and getattr(K, "fused", False) and self._aligned and not add_bias:
            K.gemm_residual(out, self.out_weight, residual)
            return None
        delta = K.gemm(out, self.out_weight, pad=True)                         # [1, N, hidden]
        if add_bias:
            delta += self.stream_bias
        return delta
