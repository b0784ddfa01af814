"""Causal grouped-query attention with normed heads and a handful of options (a mixer).

In this file's notation, for the mixer's input h of one sequence (positions t = 0 .. T-1):

    q, k, v  = Wq h (+ bq), Wk h (+ bk), Wv h (+ bv)     or, with ``values_from_keys``, v = k at this point and no Wv
    q, k    <- norm(q), norm(k)                          per head: x / sqrt(mean(x^2) + eps) * w, one w for all heads
    q, k    <- turn(q), turn(k)                          the first ``position.dim`` dims of each head, by position
    s_tj     = scale * q_t . k_j                         for t - window < j <= t, and with ``keep_first`` also for j < keep_first
    s_tj    <- cap * tanh(s_tj / cap)                    with ``softcap``
    s_tj    <- s_tj - slope_i (t - j)                    with slopes;  slope_i = 2^(-c (i + 1) / heads)
    a_tj     = exp(s_tj) / (sum_j' exp(s_tj') [+ exp(z_i)])   the added term is a sink without a value: z_i = 0
                                                         (``unit_sink``) or a learned number per head (``sink``)
    o_t      = (sum_j a_tj v_j) [* sigmoid(Wg h_t)_i]    one gate number per head
    out      = Wo o (+ bo)

Biases, norms, angles, scores and softmax run in 32-bit.  k and v are written once into the paged cache; a window is
a bound on the keys a query walks, the cache keeps every key.

The mixer can run alone (``forward``) or as a branch of a parallel mixer: ``in_weight`` / ``out_weight`` / ``inner`` /
``mix``, and ``out_bias`` (a constant row of the output, which the caller adds where it suits it).
"""

from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from ..weights.loader import TensorDecl
from .base import MIXERS, POSITIONS, Mixer


@MIXERS.register("head_attention")
class HeadAttention(Mixer):
    accepts_residual = True

    @classmethod
    def declare(cls, spec, prefix):
        s, nm = spec, spec.names
        rows = [(nm.q, s.n_heads * s.key_dim), (nm.k, s.n_kv_heads * s.key_dim)]
        if not s.values_from_keys:
            rows.append((nm.v, s.n_kv_heads * s.value_dim))
        d = [TensorDecl(prefix + n, (r, s.hidden)) for n, r in rows]
        if s.bias_in:
            d += [TensorDecl(prefix + n + nm.bias, (r,)) for n, r in rows]
        if s.qk_norm:
            d += [TensorDecl(prefix + nm.q_norm, (s.key_dim,), init="one_plus_normal"),
                  TensorDecl(prefix + nm.k_norm, (s.key_dim,), init="one_plus_normal")]
        if s.head_gate:
            d.append(TensorDecl(prefix + nm.gate, (s.n_heads, s.hidden)))
        if s.sink:
            d.append(TensorDecl(prefix + nm.sink, (s.n_heads,), init="unit_normal"))
        d.append(TensorDecl(prefix + nm.o, (s.hidden, s.n_heads * s.value_dim)))
        if s.bias_out:
            d.append(TensorDecl(prefix + nm.o + nm.bias, (s.hidden,)))
        return d

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        s = spec
        return CacheNeed(kind="full", n_kv_heads=s.n_kv_heads, head_dim=s.key_dim,
                         k_row=(s.n_kv_heads, s.key_dim), v_row=(s.n_kv_heads, s.value_dim))

    def __init__(self, spec, weights, prefix, rt):
        s, nm = spec, spec.names
        if s.n_heads % s.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if s.values_from_keys and s.value_dim != s.key_dim:
            raise ValueError("keys that double as values have the values' size")
        if s.sink and s.unit_sink:
            raise ValueError("a softmax has one sink: a learned one or the one of score 0")
        if s.keep_first < 0 or (s.softcap is not None and not s.softcap > 0):
            raise ValueError(f"normed attention: keep_first={s.keep_first}, softcap={s.softcap}")
        self.spec, self.rt = spec, rt
        f32 = lambda n: weights[prefix + n].to(torch.float32).contiguous()
        names = [nm.q, nm.k] + ([] if s.values_from_keys else [nm.v])
        mats = [weights[prefix + n] for n in names] + ([weights[prefix + nm.gate]] if s.head_gate else [])
        self.in_weight = torch.cat([m.to(rt.dtype) for m in mats], dim=0).contiguous()
        self.out_weight = weights[prefix + nm.o].to(rt.dtype).contiguous()
        self.out_bias = f32(nm.o + nm.bias) if s.bias_out else None
        self.inner = s.n_heads * s.value_dim
        self.col_k = s.n_heads * s.key_dim
        self.col_v = None if s.values_from_keys else self.col_k + s.n_kv_heads * s.key_dim
        self.col_gate = self.col_k + s.n_kv_heads * s.key_dim + (0 if s.values_from_keys else s.n_kv_heads * s.value_dim)
        self.biases = tuple(f32(n + nm.bias) for n in names) if s.bias_in else (None, None)
        if len(self.biases) == 2:
            self.biases += (None,)
        self.gammas = (f32(nm.q_norm), f32(nm.k_norm)) if s.qk_norm else (None, None)
        self.sink = torch.zeros(s.n_heads, dtype=torch.float32, device=rt.device) if s.unit_sink else None
        if s.sink:
            self.sink = f32(nm.sink)
        self.keep_first = int(s.keep_first) if s.window else 0      # (without a window every key is seen anyway)
        self.softcap = float(s.softcap) if s.softcap else 0.0
        self.slopes = None
        if s.slope_exponent is not None:
            h = torch.arange(1, s.n_heads + 1, dtype=torch.float64)
            self.slopes = torch.pow(2.0, -float(s.slope_exponent) * h / s.n_heads).to(torch.float32).to(rt.device)
        self.position, self.magnitude = None, 1.0
        if s.position is not None:
            variant = getattr(s.position, "variant", None)
            if variant not in ("half_partial", "half_whole_head") or s.position.dim > s.key_dim or s.position.dim % 2:
                raise ValueError(f"normed attention: position encoding variant {variant!r} over {s.position.dim} of "
                                 f"{s.key_dim} dims is not built; the kernels turn dim i with dim i + dim / 2 over the "
                                 f"first `dim` dims of a head ('half_partial')")
            self.position = POSITIONS.get(s.position.kind)(s.position, weights, prefix, rt)
            self.magnitude = float(getattr(self.position, "magnitude", 1.0))

    # -- as a branch: columns [col0, col0 + in_weight rows) of `proj` are this mixer's projections of the step
    def mix(self, proj, col0, ctx, kv, state, out, out_col, out_scale):
        s, K = self.spec, self.rt.kernels
        cs = self.position.tables(ctx) if self.position is not None else None
        q = K.head_finish(proj, col0, col0 + self.col_k, None if self.col_v is None else col0 + self.col_v,
                          s.n_heads, s.n_kv_heads, s.key_dim, s.value_dim, self.biases, self.gammas, s.eps, cs,
                          self.magnitude, kv, ctx)
        gate = proj[:, col0 + self.col_gate:] if s.head_gate else None
        if K.attention_tc_fits(kv, s.key_dim, s.value_dim) and s.softmax_scale > 0:
            # on the tensor cores, for prompts and single tokens alike; gate and constant in a pass of their own
            o = K.attention_tc(q, kv, ctx, s.softmax_scale, sink=self.sink, slopes=self.slopes, window=s.window,
                               softcap=self.softcap, keep_first=self.keep_first)
            K.gate_scale(o, gate, proj.shape[1], out_scale, out, out_col, gate_group=s.value_dim)
        else:
            K.attention_biased(q, kv, ctx, s.softmax_scale, out, out_col, out_scale, sink=self.sink, slopes=self.slopes,
                               gate=gate, gate_stride=proj.shape[1], gate_per_head=True, window=s.window,
                               softcap=self.softcap, keep_first=self.keep_first)

    def forward(self, x, ctx, kv, state, writes_cache: bool, residual=None):
        """Returns the delta ``[1, N, hidden]``, or None after adding it into ``residual`` in place."""
        if not writes_cache:
            raise ValueError("this mixer writes its own keys and values")
        K = self.rt.kernels
        pad = self.spec.hidden % 8 != 0 or self.inner % 8 != 0
        proj = K.gemm_store(x, self.in_weight, pad=True)
        out = torch.empty((x.shape[0], self.inner), dtype=self.rt.dtype, device=x.device)
        self.mix(proj, 0, ctx, kv, state, out, 0, 1.0)
        if residual is not None and getattr(K, "fused", False) and not pad and self.out_bias is None:
            K.gemm_residual(out, self.out_weight, residual)
            return None
        delta = K.gemm(out, self.out_weight, pad=True)
        if self.out_bias is not None:
            delta += self.out_bias
        return delta
