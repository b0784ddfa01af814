"""A plain, slow implementation of the Fuginex decoder: whole sequences, no cache, no state carried
between calls, one function per mechanism, 64-bit floats on the CPU.  It shares no code with the
package: it takes the configuration as the dict config.json holds and the tensors by name.

The design in this file's notation (T tokens, positions 0 .. T-1, stream x):

* stream:   x_0 = E[token]
* layer:    x <- x + (mixer(N_1(x)) + ff(N_2(x))), both norms of the same x; without a feed-forward the second
            term is absent.  A layer with ``weights_of: j`` runs with layer j's tensors.
* mixers:   ``parallel`` = a * window_attention(h) + b * delta_rule(h);  ``attention`` = slope_attention(h)
* ff:       D (silu(G h) * U h)
* output:   logits = H N_f(x)

N is the RMS norm with a weight (eps inside the root).
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------- small pieces
def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j) with u = 0 at negative indices, so that
    w[:, taps - 1] is the factor of u_t itself."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y


# ------------------------------------------------------------------------------- rotation
def ramp_frequencies(rot: dict):
    """(f_i for i < dims / 2, what cos and sin are multiplied with).  Plain: f_i = base^(-2 i / dims), 1.
    With ``scaling`` {factor, original, fast, slow}: at(n) = dims ln(original / (2 pi n)) / (2 ln base) is the index
    whose wave turns n times over the original length; between lo = max(floor(at(fast)), 0) and hi =
    min(ceil(at(slow)), dims - 1) the frequency goes linearly in i from f_i to f_i / factor."""
    dims = int(rot["dims"])
    base = float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def at(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(at(float(sc["fast"]))), 0)
    hi = min(math.ceil(at(float(sc["slow"]))), dims - 1)
    out = f.clone()
    for i in range(dims // 2):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / factor * r + f[i] * (1.0 - r)
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, mag: float = 1.0) -> torch.Tensor:
    """x [T, heads, d]; the first 2 * len(freqs) dims of each head turn, dim i with dim i + len(freqs)."""
    half = freqs.numel()
    ang = positions.to(F64)[:, None] * freqs[None, :]            # [T, half]
    c, s = mag * torch.cos(ang)[:, None, :], mag * torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)


# ------------------------------------------------------------------------------- attention, by scores
def masked_attention(q, k, v, scale: float, window: Optional[int] = None, unit_sink: bool = False,
                     slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv].  Query t sees keys j <= t, with ``window`` only those with
    t - j < window.  ``slopes`` [H]: slope_h * (t - j) is taken off the score.  ``unit_sink``: the softmax's
    denominator has one more term, exp(0) = 1, with no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    t = torch.arange(T)
    dist = (t[:, None] - t[None, :])
    seen = dist >= 0
    if window is not None:
        seen = seen & (dist < window)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if slopes is not None:
            s = s - slopes[h] * dist.to(q.dtype)
        s = s.masked_fill(~seen, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if unit_sink:
            m = torch.clamp(m, min=0.0)
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if unit_sink:
            den = den + torch.exp(-m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def head_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x [T, heads, d]: RMS norm over d with one weight [d] for all heads."""
    return rms_norm(x, weight, eps)


# ------------------------------------------------------------------------------- left: window attention
def window_attention(h, w, p, c, eps):
    """Keys double as values: the value of a token is its key as projected (with bias), before norm and rotation."""
    T = h.shape[0]
    H, G, d = int(c["heads"]), int(c["kv_heads"]), int(c["dim"])
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = k
    q, k = head_norm(q, w[p + "q.norm"], eps), head_norm(k, w[p + "k.norm"], eps)
    if c.get("rot"):
        f, mag = ramp_frequencies(c["rot"])
        pos = torch.arange(T)
        q, k = rotate(q, pos, f, mag), rotate(k, pos, f, mag)
    window = int(c["mask"]["size"]) if c.get("mask") else None
    o = masked_attention(q, k, v, float(c["scale"]), window=window, unit_sink=True).reshape(T, H * d)
    return o @ w[p + "o"].T + w[p + "o.b"]


# ------------------------------------------------------------------------------- right: gated delta rule
def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g) -> torch.Tensor:
    """q, k [T, Hk, dk]; v [T, H, dv]; beta [T, H]; g [T, H, dk] (decay of the rows of S).  Per head, token by
    token: S <- g * S (row-wise); u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, dv = v.shape
    Hk, dk = k.shape[1], k.shape[2]
    rep = H // Hk
    o = torch.zeros(T, H, dv, dtype=v.dtype)
    S = torch.zeros(H, dk, dv, dtype=v.dtype)
    for t in range(T):
        kt = k[t].repeat_interleave(rep, dim=0)             # [H, dk]
        qt = q[t].repeat_interleave(rep, dim=0)
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, qt)
    return o


def delta_mixer(h, w, p, c, eps):
    T = h.shape[0]
    H, Hk, dk, dv = int(c["heads"]), int(c["kv_heads"]), int(c["dim"]), int(c["vdim"])
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, Hk, dk)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, Hk, dk)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q, k = unit(q) * dk ** -0.5, unit(k)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                           # [T, H]
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]                       # [T, H * dk]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * softplus(a).view(T, H, dk))
    o = delta_rule(q, k, v, beta, g)
    o = rms_norm(o, w[p + "norm"], eps)
    o = o * torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def parallel_mixer(h, w, p, c, eps):
    return (float(c["left_scale"]) * window_attention(h, w, p + "left.", c["left"], eps)
            + float(c["right_scale"]) * delta_mixer(h, w, p + "right.", c["right"], eps))


# ------------------------------------------------------------------------------- mixer 'attention'
def head_slopes(H: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=F64)


def slope_attention(h, w, p, c, eps):
    T = h.shape[0]
    H, G, d, dv = int(c["heads"]), int(c["kv_heads"]), int(c["dim"]), int(c["vdim"])
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    q, k = head_norm(q, w[p + "q.norm"], eps), head_norm(k, w[p + "k.norm"], eps)
    o = masked_attention(q, k, v, float(c["scale"]), slopes=head_slopes(H))
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------------------- the rest of a layer
def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ------------------------------------------------------------------------------- the model
def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], return_layers: bool = False):
    """Logits [T, vocab] in 64-bit for one whole sequence (and the stream after every layer run)."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w["embed"][tok]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer['weights_of'] if layer.get('weights_of') is not None else i}."
        hm = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "parallel":
            m = parallel_mixer(hm, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "attention":
            m = slope_attention(hm, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        if layer.get("mlp"):
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward kind {layer['mlp']['kind']!r}")
            m = m + dense_ff(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        x = x + m
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
