"""Typed configuration of the Fuginex decoder, read from its config.json.

A Fuginex model is a list of layers.  A layer norms the stream twice (two weights, the same rows) and adds the
mixer of the one and the dense gated feed-forward (silu) of the other to the stream in one sum; a layer may have
no feed-forward.  Two kinds of layer: ``parallel`` runs two mixers on the same input and adds them with constant
weights -- *left*, a grouped-query attention over a sliding window whose values are its keys as projected, with
biases, normed q and k heads, a rotation of part of each head with ramp-scaled frequencies and one more term of
score 0 in the softmax's denominator; *right*, a gated delta rule with short filters, a decay per head and key
channel from a low-rank projection and a low-rank output gate -- and ``attention`` has one causal grouped-query
attention with biases, normed heads, no rotation, a slope per head times the distance taken off the scores, and a
sigmoid gate per head.  A layer with ``weights_of: j`` has no tensors: it runs with layer j's and keeps a cache
and state of its own.

config.json keys (every size and every constant that differs between models is read from here; the two low-rank
sizes of a delta rule are the checkpoint's, or ``decay_rank`` / ``gate_rank`` where a config names them):

    architecture            "Fuginex"
    vocab, width
    norm.eps
    layers[i].type          "parallel" | "attention"
    layers[i].weights_of    (absent: the layer has tensors ``l<i>.*``)
    layers[i].mixer         parallel: left {heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims, scaling
                            {factor, original, fast, slow}}}, right {heads, kv_heads, dim, vdim, conv}, left_scale,
                            right_scale;  attention: heads, kv_heads, dim, vdim, scale
    layers[i].mlp           null, or {kind: "dense", ff}

Tensor names: ``embed``, ``final.norm``, ``head``; layer i's start with ``l<i>.``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional, Tuple

from .specs import (ConfigError, DeltaRuleSpec, GatedMLPNames, GatedMLPSpec, HeadAttentionSpec, LayerSpec, MixerBranch,
                    ModelSpec, NormSpec, ParallelMixerSpec, RampScaling, RotarySpec, RunEntry)

ARCHITECTURE = "Fuginex"
MAX_POSITIONS = 1 << 24          # the design sets no limit of its own; positions are 32-bit integers
SLOPE_EXPONENT = 8.0             # head h of H takes 2^(-8 (h + 1) / H) times the distance off its scores

MLP_NAMES = GatedMLPNames(gate="mlp.gate", up="mlp.up", down="mlp.down")


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where}: required key '{key}' is missing")
    return d[key]


def _pos_int(d, key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or int(v) != v or int(v) <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return int(v)


def _heads(d, where):
    h, g = _pos_int(d, "heads", where), _pos_int(d, "kv_heads", where)
    if h % g:
        raise ConfigError(f"config.json: {where}: heads={h} is no multiple of kv_heads={g}")
    return h, g


@dataclass(frozen=True)
class WindowAttentionConfig:
    """The left mixer of a ``parallel`` layer."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]                       # None: every earlier key is seen
    rot_base: Optional[float]                   # None: no rotation
    rot_dims: int
    rot_scaling: Optional[Tuple[float, float, float, float]]    # factor, original, fast, slow

    @classmethod
    def from_dict(cls, d, where):
        h, g = _heads(d, where)
        rot = d.get("rot")
        base, dims, scaling = None, 0, None
        if rot:
            base, dims = float(_need(rot, "base", where + ".rot")), _pos_int(rot, "dims", where + ".rot")
            sc = rot.get("scaling")
            if sc:
                scaling = tuple(float(_need(sc, k, where + ".rot.scaling")) for k in ("factor", "original", "fast", "slow"))
        mask = d.get("mask")
        c = cls(heads=h, kv_heads=g, dim=_pos_int(d, "dim", where), vdim=_pos_int(d, "vdim", where),
                scale=float(_need(d, "scale", where)), window=None if not mask else _pos_int(mask, "size", where + ".mask"),
                rot_base=base, rot_dims=dims, rot_scaling=scaling)
        if c.vdim != c.dim:
            raise ConfigError(f"config.json: {where}: values are the keys as projected, so vdim={c.vdim} must equal dim={c.dim}")
        if c.rot_dims % 2 or c.rot_dims > c.dim:
            raise ConfigError(f"config.json: {where}.rot.dims={c.rot_dims} must be even and at most dim={c.dim}")
        if c.rot_base is not None and c.rot_base <= 1.0:
            raise ConfigError(f"config.json: {where}.rot.base must be above 1")
        if scaling is not None and (scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0):
            raise ConfigError(f"config.json: {where}.rot.scaling={scaling} cannot be applied")
        return c


@dataclass(frozen=True)
class DeltaRuleConfig:
    """The right mixer of a ``parallel`` layer."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int]
    gate_rank: Optional[int]

    @classmethod
    def from_dict(cls, d, where):
        h, g = _heads(d, where)
        c = cls(heads=h, kv_heads=g, dim=_pos_int(d, "dim", where), vdim=_pos_int(d, "vdim", where),
                conv=int(d.get("conv") or 1),
                decay_rank=None if d.get("decay_rank") is None else _pos_int(d, "decay_rank", where),
                gate_rank=None if d.get("gate_rank") is None else _pos_int(d, "gate_rank", where))
        if c.conv < 1:
            raise ConfigError(f"config.json: {where}.conv={c.conv} must be at least 1")
        return c


@dataclass(frozen=True)
class SlopeAttentionConfig:
    """The mixer of an ``attention`` layer."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float

    @classmethod
    def from_dict(cls, d, where):
        h, g = _heads(d, where)
        return cls(heads=h, kv_heads=g, dim=_pos_int(d, "dim", where), vdim=_pos_int(d, "vdim", where),
                   scale=float(_need(d, "scale", where)))


@dataclass(frozen=True)
class FuginexLayer:
    type: str
    weights_of: Optional[int]                   # the layer whose tensors this one runs with; None: its own
    left: Optional[WindowAttentionConfig] = None
    right: Optional[DeltaRuleConfig] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    attention: Optional[SlopeAttentionConfig] = None
    ff: Optional[int] = None                    # None: the layer has no feed-forward


@dataclass(frozen=True)
class FuginexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[FuginexLayer, ...]
    raw: dict = None                            # config.json as read (written back unchanged)
    architecture: str = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, d: dict) -> "FuginexConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != ARCHITECTURE:
            raise ConfigError(f"config.json: architecture={name!r}, expected {ARCHITECTURE!r}")
        raw_layers = _need(d, "layers", "config")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(L, "type", where)
            m = _need(L, "mixer", where)
            mlp = L.get("mlp")
            if mlp is not None and _need(mlp, "kind", where + ".mlp") != "dense":
                raise ConfigError(f"config.json: {where}.mlp.kind={mlp['kind']!r}; the design has 'dense'")
            ff = None if mlp is None else _pos_int(mlp, "ff", where + ".mlp")
            of = L.get("weights_of")
            if of is not None:
                if isinstance(of, bool) or int(of) != of or not 0 <= int(of) < len(raw_layers) or int(of) == i:
                    raise ConfigError(f"config.json: {where}.weights_of={of!r} names no other layer")
                other = raw_layers[int(of)]
                for key in ("type", "mixer", "mlp"):
                    if other.get(key) != L.get(key):
                        raise ConfigError(f"config.json: {where} runs with layer {of}'s tensors, but its '{key}' differs")
                of = int(of)
            if kind == "parallel":
                layers.append(FuginexLayer(
                    type=kind, weights_of=of,
                    left=WindowAttentionConfig.from_dict(_need(m, "left", where + ".mixer"), where + ".mixer.left"),
                    right=DeltaRuleConfig.from_dict(_need(m, "right", where + ".mixer"), where + ".mixer.right"),
                    left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0)), ff=ff))
            elif kind == "attention":
                layers.append(FuginexLayer(type=kind, weights_of=of, ff=ff,
                                           attention=SlopeAttentionConfig.from_dict(m, where + ".mixer")))
            else:
                raise ConfigError(f"config.json: {where}.type={kind!r}; the design has 'parallel' and 'attention'")
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        cfg = cls(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"),
                  norm_eps=float(_need(_need(d, "norm", "config"), "eps", "norm")),
                  layers=tuple(layers), raw=copy.deepcopy(d))
        if not cfg.norm_eps >= 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        for i in range(len(layers)):
            cfg.owner(i)                        # (a chain of weights_of that comes back to itself is refused here)
        return cfg

    def owner(self, i: int) -> int:
        """The layer whose tensors layer ``i`` runs with (itself, unless ``weights_of`` leads elsewhere)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of leads back to itself")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    # ----------------------------------------------------------------- write
    def to_dict(self) -> dict:
        d = copy.deepcopy(self.raw)
        d.setdefault("architecture", ARCHITECTURE)
        return d

    # ------------------------------------------------------------ translation
    def _mixer_spec(self, L: FuginexLayer):
        W, eps = self.width, self.norm_eps
        if L.type == "attention":
            a = L.attention
            return HeadAttentionSpec(hidden=W, n_heads=a.heads, n_kv_heads=a.kv_heads, key_dim=a.dim, value_dim=a.vdim,
                                     softmax_scale=a.scale, eps=eps, slope_exponent=SLOPE_EXPONENT, head_gate=True,
                                     bias_in=True)
        l, r = L.left, L.right
        rot = None
        if l.rot_base is not None and l.rot_dims:
            rot = RotarySpec(theta=l.rot_base, dim=l.rot_dims, max_positions=MAX_POSITIONS, variant="half_partial",
                             scaling=None if l.rot_scaling is None else RampScaling(*l.rot_scaling))
        left = HeadAttentionSpec(hidden=W, n_heads=l.heads, n_kv_heads=l.kv_heads, key_dim=l.dim, value_dim=l.vdim,
                                 softmax_scale=l.scale, eps=eps, position=rot, window=l.window, unit_sink=True,
                                 values_from_keys=True, bias_in=True, bias_out=True)
        right = DeltaRuleSpec(hidden=W, heads=r.heads, kv_heads=r.kv_heads, key_dim=r.dim, value_dim=r.vdim,
                              conv_taps=r.conv, norm_eps=eps, decay_rank=r.decay_rank, gate_rank=r.gate_rank)
        return ParallelMixerSpec(hidden=W, prefix="", branches=(
            MixerBranch(left, "left.", L.left_scale), MixerBranch(right, "right.", L.right_scale)))

    def to_model_spec(self) -> ModelSpec:
        eps, W = self.norm_eps, self.width
        own = [i for i, L in enumerate(self.layers) if L.weights_of is None]       # layers with tensors, in file order
        at = {i: n for n, i in enumerate(own)}
        specs = []
        for i in own:
            L = self.layers[i]
            ff = None if L.ff is None else GatedMLPSpec(hidden=W, intermediate=L.ff, names=MLP_NAMES, activation="silu")
            specs.append(LayerSpec(
                prefix=f"l{i}.", mixer=_prefixed(self._mixer_spec(L)), feed_forward=ff,
                mixer_norm=NormSpec(size=W, eps=eps, weight="norm1"),
                feed_forward_norm=None if ff is None else NormSpec(size=W, eps=eps, weight="norm2"),
                mixer_norm_prefix="", feed_forward_norm_prefix="", kind="parallel_residual"))
        # every layer of the file is a stop with a cache entry (and state) of its own, run with its owner's tensors
        schedule = tuple(RunEntry(layer=at[self.owner(i)], cache=i) for i in range(len(self.layers)))
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden=W, layers=tuple(specs), schedule=schedule,
            final_norm=NormSpec(size=W, eps=eps, weight="norm"), tie_embeddings=False,
            max_positions=MAX_POSITIONS, embed_name="embed", final_norm_prefix="final.", head_name="head")


def _prefixed(mixer):
    """A mixer's tensors lie under ``mix.`` behind the layer's prefix: a parallel mixer carries that prefix itself, a
    single mixer through its names."""
    import dataclasses
    if isinstance(mixer, ParallelMixerSpec):
        return dataclasses.replace(mixer, prefix="mix.")
    nm = mixer.names
    return dataclasses.replace(mixer, names=dataclasses.replace(
        nm, q="mix." + nm.q, k="mix." + nm.k, v="mix." + nm.v, o="mix." + nm.o, q_norm="mix." + nm.q_norm,
        k_norm="mix." + nm.k_norm, gate="mix." + nm.gate))
