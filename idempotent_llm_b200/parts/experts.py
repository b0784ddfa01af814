"""Feed-forward experts chosen by a table over token ids (a feed-forward).

    out_t = (1 / top) * sum_k  down_e (act(gate_e x_t) * up_e x_t),   e = table[token_t, k]

There is no learned router: which experts a token uses depends on its id alone, so the host knows a step's
grouping wherever it holds the step's token ids.  Steps of many tokens use that: rows are gathered in the order of
their experts, every expert with rows runs the gated feed-forward's two matrix products on its slice, and the
outputs are added back in the order of a token's choices.  Steps of few tokens (and steps whose tokens exist on the
device only: captured single-token steps) look the experts up on the device, and every (token, choice) streams its
expert's matrices; from a few pairs per expert on, such a step instead runs every expert over all its tokens with the
library's matrix products and lets each token pick its own experts' outputs.  All add into the 32-bit stream; they
differ in the order of their sums, not in what is summed.
"""

from __future__ import annotations

import numpy as np
import torch

from ..weights.loader import TensorDecl
from .base import FEED_FORWARDS, FeedForward
from .mlp import ACTIVATIONS

# steps with at least this many (token, choice) pairs group their rows by expert (where the host has the tokens)
GROUP_FROM = 256
# steps that cannot group (their token ids are on the device only) with at least this many (token, choice) pairs per
# expert run every expert over all tokens with the library's matrix products
DENSE_FROM = 4


@FEED_FORWARDS.register("table_experts")
class TableExperts(FeedForward):
    accepts_residual = True
    same_bits_across_steps = False      # whole prompts, portions and single tokens take different kernels

    @classmethod
    def declare(cls, spec, prefix):
        s, nm = spec, spec.names
        d = [TensorDecl(prefix + s.table, (s.vocab_size, s.top), init="choices", integer=True, high=s.n_experts)]
        for e in range(s.n_experts):
            p = prefix + s.expert.format(e)
            d += [TensorDecl(p + nm.gate, (s.intermediate, s.hidden)), TensorDecl(p + nm.up, (s.intermediate, s.hidden)),
                  TensorDecl(p + nm.down, (s.hidden, s.intermediate))]
        return d

    def __init__(self, spec, weights, prefix, rt):
        s, nm = spec, spec.names
        if s.activation not in ACTIVATIONS:
            raise ValueError(f"activation {s.activation!r} is not built; known: {sorted(ACTIVATIONS)}")
        self.spec, self.rt, self.act = spec, rt, ACTIVATIONS[s.activation]

        def stack(name):
            return [weights[prefix + s.expert.format(e) + name].to(rt.dtype) for e in range(s.n_experts)]
        K = rt.kernels
        aligned = not (rt.dtype == torch.bfloat16 and (s.hidden % 8 or s.intermediate % 8))
        self.fused = bool(getattr(K, "fused", False)) and aligned
        self.can_group = aligned
        # An expert's gate and up rows are ONE matrix, which both kinds of step read: alternating (gate row of a
        # feature, then its up row: what the gated product's epilogue wants) with the fused kernels, else gate rows
        # followed by up rows.  [E, rows, W]; down [E, W, ff].
        if self.fused:
            self.gate_up = torch.stack([K.tile_gate_up(g, u) for g, u in zip(stack(nm.gate), stack(nm.up))]).contiguous()
            self.row_stride, self.up_off = 2 * s.hidden, s.hidden
        else:
            self.gate_up = torch.stack([torch.cat([g, u], dim=0) for g, u in zip(stack(nm.gate), stack(nm.up))]).contiguous()
            self.row_stride, self.up_off = s.hidden, s.intermediate * s.hidden
        self.down = torch.stack(stack(nm.down)).contiguous()
        self.table = weights[prefix + s.table].to(torch.int32).contiguous()
        self.table_host = self.table.cpu().numpy()
        bad = (self.table_host < 0) | (self.table_host >= s.n_experts)
        if bad.any():
            raise ValueError(f"{prefix + s.table}: entries outside the {s.n_experts} experts")

    def forward(self, x, ctx, residual=None):
        """Adds into ``residual`` and returns None (or returns the delta ``[1, N, hidden]``)."""
        s, K = self.spec, self.rt.kernels
        n = x.shape[0]
        h = residual if residual is not None else torch.zeros((n, s.hidden), dtype=torch.float32, device=x.device)
        toks = getattr(ctx, "host_tokens", None)
        if toks is not None and self.can_group and n * s.top >= GROUP_FROM:
            ids = ctx.memo.get("host_token_array")           # the step's token ids as one array, made once a step
            if ids is None:
                ids = ctx.memo["host_token_array"] = np.concatenate([np.asarray(t, dtype=np.int64) for t in toks])
            self._grouped(x, ids, h)
        elif self.fused and n * s.top >= DENSE_FROM * s.n_experts:
            K.experts_dense(x, ctx.tokens, self.table, self.gate_up, self.down, h, self.act, 1.0 / s.top)
        else:
            K.experts_few(x, ctx.tokens, self.table, self.gate_up, self.row_stride, self.up_off, self.down, h, self.act, 1.0 / s.top)
        return None if residual is not None else h.unsqueeze(0)

    def _grouped(self, x, tokens, h):
        s, K = self.spec, self.rt.kernels
        n, top = tokens.shape[0], s.top
        # [n * top]: expert of (token, k); as 16-bit keys where they fit (a stable sort of those is a radix sort)
        choice = self.table_host[tokens].reshape(-1).astype(np.int16 if s.n_experts < 32768 else np.int32)
        order = np.argsort(choice, kind="stable")                          # grouped rows -> (token, k)
        counts = np.bincount(choice, minlength=s.n_experts)
        place = np.empty(n * top, dtype=np.int32)
        place[order] = np.arange(n * top, dtype=np.int32)                  # (token, k) -> grouped row
        both = torch.from_numpy(np.concatenate([(order // top).astype(np.int32), place])).to(x.device, non_blocking=True)
        if self.fused:                      # gather, every expert's two products and the sum back: one call into the library
            K.experts_grouped_step(x, both[:n * top], both[n * top:].view(n, top), np.ascontiguousarray(counts, dtype=np.int32),
                                   self.gate_up, self.down, h, self.act, 1.0 / top)
            return
        xg = K.rows_gather(x, both[:n * top])
        z = torch.empty((n * top, s.hidden), dtype=torch.float32, device=x.device)
        at = 0
        for e in range(s.n_experts):
            c = int(counts[e])
            if not c:
                continue
            y = K.gated_act(K.gemm_store(xg[at:at + c], self.gate_up[e]), self.act)      # (no fused epilogue here: 32-bit)
            K.gemm_store(y, self.down[e], out=z[at:at + c])
            at += c
        K.experts_combine(z, both[n * top:].view(n, top), h, 1.0 / top)


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """Experts named by a learned router (``RoutedExpertsSpec``):

        z = Wr x;  s = softmax(z);  chosen = the ``top`` largest of s + correction inside the best groups
        out_t = sum_k w_k * expert_(chosen_k)(x_t)  +  shared(x_t),      w = s_chosen / (sum s_chosen + 1e-20) * scale

    where the last ``n_identity`` router outputs stand for experts that return x_t itself.  The router's product and
    everything behind it (softmax, groups, choice, weights) is 32-bit and runs on the device, one warp per token, so a
    captured single-token step needs nothing from the host.  The experts then run the way table-routed experts do, on
    the same kernels: a step's row numbers take the place of token ids and the step's choices the place of the table;
    every (token, choice) pair carries its weight.  Steps of many tokens, outside a captured graph, read the choices
    back and group the rows by expert for one matrix product per expert.  Returns the sum as a delta (a norm may sit
    behind the feed-forward)."""

    same_bits_across_steps = False      # whole prompts, portions and single tokens take different kernels

    @classmethod
    def declare(cls, spec, prefix):
        s, nm = spec, spec.names
        total = s.n_experts + s.n_identity
        d = [TensorDecl(prefix + s.router, (total, s.hidden)), TensorDecl(prefix + s.correction, (total,))]
        for e in range(s.n_experts):
            p = prefix + s.expert.format(e)
            d += [TensorDecl(p + nm.gate, (s.intermediate, s.hidden)), TensorDecl(p + nm.up, (s.intermediate, s.hidden)),
                  TensorDecl(p + nm.down, (s.hidden, s.intermediate))]
        if s.shared is not None:
            d += FEED_FORWARDS.get(s.shared.kind).declare(s.shared, prefix)
        return d

    def __init__(self, spec, weights, prefix, rt):
        s, nm = spec, spec.names
        total = s.n_experts + s.n_identity
        if s.activation not in ACTIVATIONS:
            raise ValueError(f"activation {s.activation!r} is not built; known: {sorted(ACTIVATIONS)}")
        if not 1 <= s.top <= total or s.groups < 1 or total % s.groups or not 1 <= s.groups_keep <= s.groups:
            raise ValueError(f"routed experts: {s.top} of {total} experts in {s.groups} groups of which {s.groups_keep} are kept")
        if s.top > s.groups_keep * (total // s.groups):
            raise ValueError(f"routed experts: {s.top} experts cannot come from {s.groups_keep} groups of {total // s.groups}")
        self.spec, self.rt, self.act = spec, rt, ACTIVATIONS[s.activation]
        K = rt.kernels

        def stack(name):
            return [weights[prefix + s.expert.format(e) + name].to(rt.dtype) for e in range(s.n_experts)]
        aligned = not (rt.dtype == torch.bfloat16 and (s.hidden % 8 or s.intermediate % 8))
        self.fused = bool(getattr(K, "fused", False)) and aligned
        self.can_group = aligned
        self.pad = {} if aligned else {"pad": True}
        if s.n_experts:
            if self.fused:      # gate and up rows alternating: what the gated product's epilogue wants
                self.gate_up = torch.stack([K.tile_gate_up(g, u) for g, u in zip(stack(nm.gate), stack(nm.up))]).contiguous()
                self.row_stride, self.up_off = 2 * s.hidden, s.hidden
            else:
                self.gate_up = torch.stack([torch.cat([g, u], dim=0) for g, u in zip(stack(nm.gate), stack(nm.up))]).contiguous()
                self.row_stride, self.up_off = s.hidden, s.intermediate * s.hidden
            self.down = torch.stack(stack(nm.down)).contiguous()
        self.w_router = weights[prefix + s.router].to(rt.dtype).contiguous()
        self.correction = weights[prefix + s.correction].to(torch.float32).contiguous()
        self.shared = None
        if s.shared is not None:
            self.shared = FEED_FORWARDS.get(s.shared.kind)(s.shared, weights, prefix, rt)
        self._rows = {}

    def _row_numbers(self, n: int, device):
        r = self._rows.get(n)
        if r is None:
            r = self._rows[n] = torch.arange(n, dtype=torch.int32, device=device)
        return r

    def route(self, x):
        """(chosen [N, top] int32, weight [N, top]) of the step's rows."""
        s, K = self.spec, self.rt.kernels
        z = K.gemm_store(x, self.w_router, pad=True)                        # 32-bit logits over all experts
        return K.route(z, self.correction, s.top, s.groups, s.groups_keep, s.scale)

    def forward(self, x, ctx):
        s, K = self.spec, self.rt.kernels
        n = x.shape[0]
        # the shared expert's output opens the sum (its product writes the buffer the experts then add into)
        if self.shared is not None:
            h = self.shared.forward(x, ctx)[0]
        else:
            h = torch.zeros((n, s.hidden), dtype=torch.float32, device=x.device)
        chosen, weight = self.route(x)
        if s.n_experts:
            rows = self._row_numbers(n, x.device)
            in_eager_step = getattr(ctx, "host_tokens", None) is not None
            if in_eager_step and self.can_group and n * s.top >= GROUP_FROM:
                self._grouped(x, chosen, weight, h)
            elif self.fused and n * s.top >= DENSE_FROM * s.n_experts:
                K.experts_dense(x, rows, chosen, self.gate_up, self.down, h, self.act, 1.0, pair_w=weight)
            else:
                K.experts_few(x, rows, chosen, self.gate_up, self.row_stride, self.up_off, self.down, h, self.act, 1.0,
                              pair_w=weight)
        if s.n_identity:
            K.experts_identity(x, chosen, weight, h, s.n_experts)
        return h.unsqueeze(0)

    def _grouped(self, x, chosen, weight, h):
        s, K = self.spec, self.rt.kernels
        n, top, E = x.shape[0], s.top, s.n_experts
        flat = chosen.cpu().numpy().reshape(-1)                             # (the step waits for its router here)
        keys = np.where((flat >= 0) & (flat < E), flat, E).astype(np.int16 if E < 32767 else np.int32)
        order = np.argsort(keys, kind="stable")                             # grouped rows -> (token, k); pairs without a
        counts = np.bincount(keys, minlength=E + 1)[:E]                     # real expert come last and belong to nobody
        n_rows = int(counts.sum())
        place = np.full(n * top, -1, dtype=np.int32)
        place[order[:n_rows]] = np.arange(n_rows, dtype=np.int32)           # (token, k) -> grouped row, or -1
        both = torch.from_numpy(np.concatenate([(order // top).astype(np.int32), place])).to(x.device, non_blocking=True)
        src, place_d = both[:n * top], both[n * top:].view(n, top)
        if self.fused:
            K.experts_grouped_step(x, src, place_d, np.ascontiguousarray(counts, dtype=np.int32), self.gate_up, self.down, h,
                                   self.act, 1.0, pair_w=weight)
            return
        xg = K.rows_gather(x, src)
        z = torch.empty((n * top, s.hidden), dtype=torch.float32, device=x.device)
        at = 0
        for e in range(E):
            c = int(counts[e])
            if not c:
                continue
            y = K.gated_act(K.gemm_store(xg[at:at + c], self.gate_up[e], **self.pad), self.act)
            K.gemm_store(y, self.down[e], out=z[at:at + c], **self.pad)
            at += c
        K.experts_combine(z, place_d, h, 1.0, pair_w=weight)
