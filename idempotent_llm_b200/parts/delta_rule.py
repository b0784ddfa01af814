"""Gated delta rule (a recurrent mixer).

In this file's notation, for the mixer's input h_t, with H heads of value size P, Hk key heads of size D:

    q, k, v   = silu(filter(Wq h)), silu(filter(Wk h)), silu(filter(Wv h))     per channel, ``conv_taps`` taps, causal
    q, k     <- q / sqrt(|q|^2 + 1e-6) * D^-1/2,  k / sqrt(|k|^2 + 1e-6)        per head
    beta_t    = sigmoid(Wb h_t)                                                 per head
    g_t       = exp(-exp(A_log) * softplus(Wa2 (Wa1 h_t) + dt_bias))            per head and key channel
    S        <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T      S: [D, P] per head, head i reads key head i // (H / Hk)
    y_t       = S^T q_t
    o_t       = y_t / sqrt(mean(y_t^2) + eps) * w * sigmoid(Wg2 (Wg1 h_t))      per head; w [P] for all heads
    out       = Wo o_t

The recurrence, its decays, step sizes and gates, the unit norms and the norm behind it run in 32-bit.  Per-sequence
state: the filters' last ``conv_taps - 1`` inputs and S, in 32-bit, zero at a sequence's start.  The two low-rank
projections' second halves are one product with the two matrices on the diagonal of one.

With ``decay = "head"`` the decay is one number per head, ``g_t = exp(-exp(A_log) * softplus(Wa h_t + dt_bias))`` with
a full matrix Wa [H, hidden]; with ``gate = "silu"`` the read-out is multiplied by ``silu(Wg h_t)`` with a full matrix
Wg [H P, hidden].  Both ride in the joint input projection; the recurrence is the same.

Alone (``forward``) or as a branch of a parallel mixer (``in_weight`` / ``out_weight`` / ``inner`` / ``mix``).
"""

from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from ..weights.loader import TensorDecl
from .base import MIXERS, Mixer


def _default_rank(s) -> int:
    return max(8, -(-(s.key_dim // 2) // 8) * 8)


@MIXERS.register("gated_delta")
class GatedDeltaRule(Mixer):
    @staticmethod
    def _sizes(s):
        qk, v = s.kv_heads * s.key_dim, s.heads * s.value_dim
        return qk, v, 2 * qk + v                    # one of q / k, v, filtered channels

    @classmethod
    def declare(cls, spec, prefix):
        s, nm = spec, spec.names
        qk, v, ch = cls._sizes(s)
        ra = s.decay_rank if s.decay_rank is not None else -1
        rg = s.gate_rank if s.gate_rank is not None else -1
        free = _default_rank(s)
        rows = [(nm.q, qk), (nm.k, qk), (nm.v, v)]
        d = [TensorDecl(prefix + n, (r, s.hidden)) for n, r in rows]
        d += [TensorDecl(prefix + n + nm.conv, (r, s.conv_taps), init="filter") for n, r in rows]    # (one tap: a factor)
        d += [TensorDecl(prefix + nm.beta, (s.heads, s.hidden)),
              TensorDecl(prefix + nm.a_log, (s.heads,), init="unit_normal"),
              TensorDecl(prefix + nm.norm, (s.value_dim,), init="one_plus_normal")]
        if s.decay == "head":
            d += [TensorDecl(prefix + nm.decay, (s.heads, s.hidden)),
                  TensorDecl(prefix + nm.dt_bias, (s.heads,), init="unit_normal")]
        else:
            d += [TensorDecl(prefix + nm.decay_down, (ra, s.hidden), free=free),
                  TensorDecl(prefix + nm.decay_up, (s.heads * s.key_dim, ra), free=free),
                  TensorDecl(prefix + nm.dt_bias, (s.heads * s.key_dim,), init="unit_normal")]
        if s.gate == "silu":
            d.append(TensorDecl(prefix + nm.gate, (v, s.hidden)))
        else:
            d += [TensorDecl(prefix + nm.gate_down, (rg, s.hidden), free=free),
                  TensorDecl(prefix + nm.gate_up, (v, rg), free=free)]
        d.append(TensorDecl(prefix + nm.o, (s.hidden, v)))
        return d

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        s = spec
        qk, v, ch = cls._sizes(s)
        return CacheNeed(kind="none", state_shape=((s.conv_taps - 1) * ch + s.heads * s.key_dim * s.value_dim,))

    def __init__(self, spec, weights, prefix, rt):
        s, nm = spec, spec.names
        if s.heads % s.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        qk, v, ch = self._sizes(s)
        if s.decay not in ("channel", "head") or s.gate not in ("sigmoid_low_rank", "silu"):
            raise ValueError(f"gated delta rule: decay {s.decay!r} / gate {s.gate!r} are not built; known: 'channel', 'head' / "
                             f"'sigmoid_low_rank', 'silu'")
        self.spec, self.rt = spec, rt
        self.qk, self.inner, self.channels = qk, v, ch
        self.head_decay, self.silu_gate = s.decay == "head", s.gate == "silu"
        # the joint input projection's rows: q, k, v, beta, then the full matrices (a decay per head, a silu gate), then
        # the first halves of the low-rank projections
        mats = [weights[prefix + n] for n in (nm.q, nm.k, nm.v, nm.beta)]
        self.col_beta = ch
        at = ch + s.heads
        self.col_decay = self.col_gate = None
        if self.head_decay:
            mats.append(weights[prefix + nm.decay])
            self.col_decay, at = at, at + s.heads
        if self.silu_gate:
            mats.append(weights[prefix + nm.gate])
            self.col_gate, at = at, at + v
        self.col_low = at
        a1 = a2 = g1 = g2 = None
        if not self.head_decay:
            a1, a2 = weights[prefix + nm.decay_down], weights[prefix + nm.decay_up]
        if not self.silu_gate:
            g1, g2 = weights[prefix + nm.gate_down], weights[prefix + nm.gate_up]
        ra, rg = (0 if a1 is None else a1.shape[0]), (0 if g1 is None else g1.shape[0])
        if (a2 is not None and a2.shape[1] != ra) or (g2 is not None and g2.shape[1] != rg):
            raise ValueError(f"{prefix}: the halves of a low-rank projection disagree on its inner size")
        self.ranks = (ra, rg)
        mats += [m for m in (a1, g1) if m is not None]
        self.in_weight = torch.cat([m.to(rt.dtype) for m in mats], dim=0).contiguous()
        self.out_weight = weights[prefix + nm.o].to(rt.dtype).contiguous()
        # the second halves of the low-rank projections as one matrix: [decay rows | gate rows] x [ra | rg], zero
        # elsewhere, its inner size rounded up to 8 (rows on 16-byte borders in bfloat16)
        self.low_width = -(-(ra + rg) // 8) * 8
        self.up_weight = None
        self.decay_cols = s.heads * s.key_dim
        if ra + rg:
            n_a = 0 if a2 is None else self.decay_cols
            up = torch.zeros((n_a + (0 if g2 is None else v), self.low_width), dtype=rt.dtype, device=rt.device)
            if a2 is not None:
                up[:n_a, :ra] = a2.to(rt.dtype)
            if g2 is not None:
                up[n_a:, ra:ra + rg] = g2.to(rt.dtype)
            self.up_weight = up
        f32 = lambda n: weights[prefix + n].to(torch.float32).contiguous()
        self.w_conv = torch.cat([f32(n + nm.conv) for n in (nm.q, nm.k, nm.v)], dim=0).contiguous()
        self.dt_bias, self.a_log, self.norm = f32(nm.dt_bias), f32(nm.a_log), f32(nm.norm)
        self.conv_floats = (s.conv_taps - 1) * ch

    def mix(self, proj, col0, ctx, kv, state, out, out_col, out_scale):
        s, K = self.spec, self.rt.kernels
        conv_state = state[:, :self.conv_floats] if self.conv_floats else None
        c = K.short_conv(proj, col0, self.channels, self.w_conv, None, 1, conv_state, ctx)      # [q | k | v], silu
        if s.conv_taps > 1 and not ctx.single_token:
            K.conv_state_update(proj, col0, self.channels, s.conv_taps, conv_state, ctx)
        if self.up_weight is not None:
            low = K.cols_cast(proj, col0 + self.col_low, sum(self.ranks), self.low_width)
            ag = K.gemm_store(low, self.up_weight)                                              # [decay | gate], 32-bit
            if self.head_decay:                                                                 # (gate columns only: decays beside them)
                g = torch.empty((proj.shape[0], self.decay_cols), dtype=torch.float32, device=proj.device)
            else:
                g = ag
        else:
            ag, g = None, torch.empty((proj.shape[0], self.decay_cols), dtype=torch.float32, device=proj.device)
        beta = K.delta_prep(c, 0, self.qk, g, 0, proj, col0 + self.col_beta, self.dt_bias, self.a_log, s.heads,
                            s.kv_heads, s.key_dim, head_col=col0 + self.col_decay if self.head_decay else -1)
        y = K.delta_scan(c, 0, self.qk, 2 * self.qk, g, 0, beta, state[:, self.conv_floats:], ctx, s.heads, s.kv_heads,
                         s.key_dim, s.value_dim)
        if self.silu_gate:
            K.delta_out(y, self.norm, s.norm_eps, proj, col0 + self.col_gate, out_scale, out, out_col, s.heads, s.value_dim,
                        gate_act=1)
        else:
            K.delta_out(y, self.norm, s.norm_eps, ag, 0 if self.head_decay else self.decay_cols, out_scale, out, out_col,
                        s.heads, s.value_dim)

    def forward(self, x, ctx, kv, state, writes_cache: bool):
        K = self.rt.kernels
        proj = K.gemm_store(x, self.in_weight, pad=True)
        out = torch.empty((x.shape[0], self.inner), dtype=self.rt.dtype, device=x.device)
        self.mix(proj, 0, ctx, None, state, out, 0, 1.0)
        return K.gemm(out, self.out_weight, pad=True)
