"""A plain, slow implementation of the Pununex decoder: whole sequences, no cache, no state carried between
calls, one function per mechanism, 64-bit floats on the CPU.  It shares no code with the package: it takes the
configuration as the dict config.json holds and the tensors by name.

The design in this file's notation (T tokens, positions 0 .. T-1, stream x):

* stream:   x_0 = E[token_t] + B[r_t],  r_0 = buckets,  r_t = (a * token_(t-1) + c * token_t) mod buckets
* layer:    x <- x + s_1 * LN_1(mixer(x));  x <- x + s_2 * LN_2(ff(x))   (the sublayers read x itself; the norm
            sits behind a sublayer; s_1, s_2 are learned rows; a layer may have no feed-forward)
* mixers:   ``delta`` = a gated delta rule with one decay per head and a silu gate;
            ``parallel`` = a * capped_window_attention(x) + b * delta rule with a decay per key channel
* ff:       dense: D (relu(G h) * U h);  or routed experts (softmax router, choice by corrected scores inside the
            best groups, identity experts, a shared expert)
* output:   logits = H LN_f(x)

LN is the layer norm with weight and bias (variance = mean squared deviation, eps inside the root).
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------- small pieces
def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight + bias


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), u = 0 before the start; the last column of
    w is the factor of u_t itself."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y


# ------------------------------------------------------------------------------- embedding
def bigram_rows(tokens: Sequence[int], buckets: int, mul_prev: int, mul_cur: int):
    """Row of the bigram table per position: the last row for a sequence's first token."""
    rows = [buckets]
    for t in range(1, len(tokens)):
        rows.append((int(tokens[t - 1]) * mul_prev + int(tokens[t]) * mul_cur) % buckets)
    return rows


def embed(tokens, w, cfg) -> torch.Tensor:
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        rows = bigram_rows(tokens, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))
        x = x + w["bigram"][torch.tensor(rows, dtype=torch.long)]
    return x


# ------------------------------------------------------------------------------- attention, by scores
def seen_mask(T: int, window: Optional[int], keep_first: int) -> torch.Tensor:
    """[T, T] True where query i sees key j: j <= i and (i - j < window or j < keep_first)."""
    t = torch.arange(T)
    dist = t[:, None] - t[None, :]
    seen = dist >= 0
    if window is not None:
        seen = seen & ((dist < window) | (t[None, :] < keep_first))
    return seen


def capped_sink_attention(q, k, v, scale: float, softcap: Optional[float], window: Optional[int], keep_first: int,
                          sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv].  score = scale q.k, then cap * tanh(score / cap); softmax over the
    seen keys with exp(sink_h) added once to the denominator (no key, no value, neither scaled nor capped)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    seen = seen_mask(T, window, keep_first)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~seen, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def window_attention(h, w, p, c, eps):
    T = h.shape[0]
    H, G, d, dv = int(c["heads"]), int(c["kv_heads"]), int(c["dim"]), int(c["vdim"])
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    q, k = rms_norm(q, w[p + "q.norm"], eps), rms_norm(k, w[p + "k.norm"], eps)
    mask = c.get("mask") or {}
    window = int(mask["size"]) if mask.get("size") else None
    keep = int(mask.get("keep_first") or 0)
    o = capped_sink_attention(q, k, v, float(c["scale"]), c.get("softcap"), window, keep, w.get(p + "sink"))
    return o.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------------------- gated delta rule
def delta_recurrence(q, k, v, beta, g) -> torch.Tensor:
    """q, k [T, Hk, dk]; v [T, H, dv]; beta [T, H]; g [T, H, dk] (decay of the rows of S).  Per head, token by
    token: S <- g * S (row-wise); u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, dv = v.shape
    Hk, dk = k.shape[1], k.shape[2]
    out = torch.zeros(T, H, dv, dtype=v.dtype)
    for h in range(H):
        j = h // (H // Hk)
        S = torch.zeros(dk, dv, dtype=v.dtype)
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, j])
            S = S + torch.outer(k[t, j], u)
            out[t, h] = S.T @ q[t, j]
    return out


def delta_inputs(h, w, p, c):
    T = h.shape[0]
    H, Hk, dk, dv = int(c["heads"]), int(c["kv_heads"]), int(c["dim"]), int(c["vdim"])
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, Hk, dk)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, Hk, dk)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q, k = unit(q) * dk ** -0.5, unit(k)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    return q, k, v, beta


def delta_mixer_head_decay(h, w, p, c, eps):
    """One decay per head, a silu gate of full rank."""
    T = h.shape[0]
    H, dk, dv = int(c["heads"]), int(c["dim"]), int(c["vdim"])
    q, k, v, beta = delta_inputs(h, w, p, c)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))       # [T, H]
    o = delta_recurrence(q, k, v, beta, g[:, :, None].expand(T, H, dk))
    o = rms_norm(o, w[p + "norm"], eps) * silu(h @ w[p + "g"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def delta_mixer_channel_decay(h, w, p, c, eps):
    """One decay per head and key channel from a low-rank projection, a low-rank sigmoid gate."""
    T = h.shape[0]
    H, dk, dv = int(c["heads"]), int(c["dim"]), int(c["vdim"])
    q, k, v, beta = delta_inputs(h, w, p, c)
    dt = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, dk)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * dt)
    o = delta_recurrence(q, k, v, beta, g)
    o = rms_norm(o, w[p + "norm"], eps) * torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def parallel_mixer(h, w, p, c, eps):
    return (float(c.get("left_scale", 1.0)) * window_attention(h, w, p + "left.", c["left"], eps)
            + float(c.get("right_scale", 1.0)) * delta_mixer_channel_decay(h, w, p + "right.", c["right"], eps))


# ------------------------------------------------------------------------------- feed-forwards
def gated_ff(h, w, p, act) -> torch.Tensor:
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(z: torch.Tensor, correction: torch.Tensor, r: dict):
    """z [T, E] router logits over experts and identity experts.  Returns (chosen [T, top], weights [T, top])."""
    E = z.shape[1]
    top = int(r["top"])
    s = torch.softmax(z, dim=-1)
    choice = s + correction
    groups = r.get("groups") or {}
    count, keep = int(groups.get("count") or 1), int(groups.get("keep") or groups.get("count") or 1)
    if count > 1 and keep < count:
        per = E // count
        best = choice.view(-1, count, per).max(dim=-1).values                      # [T, count]
        kept = best.topk(keep, dim=-1).indices
        allowed = torch.zeros(z.shape[0], count, dtype=torch.bool)
        allowed.scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), -math.inf)
    chosen = choice.topk(top, dim=-1).indices
    picked = s.gather(1, chosen)
    weights = picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))
    return chosen, weights


def route_margin(z: torch.Tensor, correction: torch.Tensor, r: dict) -> torch.Tensor:
    """[T]: how far each token's choice is from falling another way: the gap between the last chosen expert's choice
    score and the best one not chosen (among the open groups), and, where groups shut experts out, the gap between the
    last kept group's score and the best one shut out; the smaller of the two."""
    E, top = z.shape[1], int(r["top"])
    choice = torch.softmax(z, dim=-1) + correction
    groups = r.get("groups") or {}
    count, keep = int(groups.get("count") or 1), int(groups.get("keep") or groups.get("count") or 1)
    margin = torch.full((z.shape[0],), math.inf, dtype=z.dtype)
    if count > 1 and keep < count:
        per = E // count
        best = choice.view(-1, count, per).max(dim=-1).values.sort(dim=-1, descending=True).values
        margin = best[:, keep - 1] - best[:, keep]
        kept = choice.view(-1, count, per).max(dim=-1).values.topk(keep, dim=-1).indices
        allowed = torch.zeros(z.shape[0], count, dtype=torch.bool).scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), -math.inf)
    ranked = choice.sort(dim=-1, descending=True).values
    if top < E:
        margin = torch.minimum(margin, ranked[:, top - 1] - ranked[:, top])
    return margin


def routed_ff(h, w, p, c, forced=None, flips=None):
    """``forced`` [T, top]: the experts every token is given instead of the router's own choice (the weights still come
    from this function's own softmax); ``flips`` then receives (token, margin of the own choice) wherever the given
    experts are not the own ones.  For comparisons in low precision, where a choice within rounding may fall either way."""
    r = c["router"]
    n_real, n_id = int(r["experts"]), int(r.get("identity") or 0)
    z = h @ w[p + "router"].T
    chosen, weights = route(z, w[p + "correction"], r)
    if forced is not None:
        own, margin = chosen, route_margin(z, w[p + "correction"], r)
        chosen = forced.long()
        picked = torch.softmax(z, dim=-1).gather(1, chosen)
        weights = picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))
        if flips is not None:
            for t in range(h.shape[0]):
                if sorted(own[t].tolist()) != sorted(chosen[t].tolist()):
                    flips.append((t, float(margin[t])))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), weights[t]):
            if e >= n_real:
                out[t] += wt * h[t]
            else:
                out[t] += wt * gated_ff(h[t:t + 1], w, f"{p}e{e}.", silu)[0]
    if c.get("shared"):
        out = out + gated_ff(h, w, p + "shared.", silu)
    return out


def feed_forward(h, w, p, c, forced=None, flips=None):
    if c["kind"] == "dense":
        return gated_ff(h, w, p, torch.relu)
    if c["kind"] == "moe":
        return routed_ff(h, w, p, c, forced, flips)
    raise ValueError(c["kind"])


# ------------------------------------------------------------------------------- the model
def load(model_dir: str):
    """(config dict, tensors by name in 64-bit; integer tensors stay integers): own reading of the folder."""
    import json
    import os
    import struct
    import numpy as np
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, m in head.items():
        if name == "__metadata__":
            continue
        a, b = m["data_offsets"]
        raw = np.frombuffer(data[a:b], dtype=np.uint8)
        if m["dtype"] == "BF16":
            u = raw.view(np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy()).to(F64)
        elif m["dtype"] == "F32":
            t = torch.from_numpy(raw.view(np.float32).copy()).to(F64)
        elif m["dtype"] == "F16":
            t = torch.from_numpy(raw.view(np.float16).copy()).to(F64)
        elif m["dtype"] == "I32":
            t = torch.from_numpy(raw.view(np.int32).copy())
        else:
            raise ValueError(m["dtype"])
        out[name] = t.reshape(m["shape"])
    return cfg, out


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[list] = None,
            routes: Optional[dict] = None, flips: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``layers_out`` receives the stream after every layer.  ``routes`` {layer: [T,
    top]} gives routed layers their experts (see ``routed_ff``); ``flips`` receives (layer, token, margin)."""
    eps = float(cfg["norm"]["eps"])
    x = embed(tokens, w, cfg)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        if L["type"] == "delta":
            y = delta_mixer_head_decay(x, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(x, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + w[p + "ls1"] * layer_norm(y, w[p + "norm1"], w[p + "norm1.b"], eps)
        if L.get("mlp"):
            mine = []
            forced = None if routes is None or i not in routes else routes[i][:len(tokens)]
            y = feed_forward(x, w, p + "mlp.", L["mlp"], forced, mine)
            if flips is not None:
                flips += [(i, t, m) for t, m in mine]
            x = x + w[p + "ls2"] * layer_norm(y, w[p + "norm2"], w[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
