"""Typed configuration of the Pununex decoder, read from its config.json.

A Pununex model is a token embedding with a hashed bigram row added, a list of layers, a final layer norm and an
untied head.  A layer's sublayers read the stream itself; a layer norm (weight and bias) sits BEHIND each sublayer and
its result, times a learned row, is added to the stream.  Two kinds of layer: ``delta`` has a gated delta rule with one
decay per head and a silu gate of full rank; ``parallel`` runs two mixers on the same input and adds them with constant
weights -- *left*, a grouped-query attention without rotation whose q and k heads are normed, whose scores are capped
by a tanh, which sees a sliding window plus the sequence's first tokens and has a learned sink per head in the
softmax's denominator; *right*, a gated delta rule with a decay per head and key channel from a low-rank projection and a
low-rank sigmoid gate.  A layer's feed-forward is absent, dense (``down(relu(gate x) * up x)``) or a mixture of experts
(softmax router, choice by corrected scores inside the best groups of neighbours, identity experts, a shared expert).

config.json keys (every size and every constant that differs between models is read from here; the low-rank sizes of
a ``parallel`` layer's delta rule are the checkpoint's):

    architecture            "Pununex"
    vocab, width
    norm.eps
    embedding.bigram        {buckets, mul_prev, mul_cur}   (absent: a plain lookup)
    layers[i].type          "delta" | "parallel"
    layers[i].mixer         delta: heads, kv_heads, dim, vdim, conv;  parallel: left {heads, kv_heads, dim, vdim, scale,
                            softcap, mask {size, keep_first}}, right {heads, kv_heads, dim, vdim, conv}, left_scale,
                            right_scale
    layers[i].mlp           null, {kind: "dense", ff}, or {kind: "moe", expert {ff}, router {experts, top, identity,
                            scale, groups {count, keep}}, shared {ff}}

Tensor names: ``embed``, ``bigram``, ``final.norm`` (+ ``.b``), ``head``; layer i's start with ``l<i>.``: ``norm1``,
``norm2`` (+ ``.b``), ``ls1``, ``ls2``, ``mix.*``, ``mlp.*``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional, Tuple

from .specs import (BigramHashSpec, ConfigError, DeltaRuleNames, DeltaRuleSpec, GatedMLPNames, GatedMLPSpec,
                    HeadAttentionNames, HeadAttentionSpec, LayerNormSpec, MixerBranch, ModelSpec, ParallelMixerSpec,
                    PostNormLayerSpec, RoutedExpertsSpec, default_schedule)

ARCHITECTURE = "Pununex"
MAX_POSITIONS = 1 << 24          # the design sets no limit of its own; positions are 32-bit integers


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where}: required key '{key}' is missing")
    return d[key]


def _int(d, key: str, where: str, least: int = 1) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or int(v) != v or int(v) < least:
        raise ConfigError(f"config.json: {where}.{key} must be an integer of at least {least}, got {v!r}")
    return int(v)


def _heads(d, where):
    h, g = _int(d, "heads", where), _int(d, "kv_heads", where)
    if h % g:
        raise ConfigError(f"config.json: {where}: heads={h} is no multiple of kv_heads={g}")
    return h, g


@dataclass(frozen=True)
class CappedAttentionConfig:
    """The left mixer of a ``parallel`` layer."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]                    # None: scores are not capped
    window: Optional[int]                       # None: every earlier key is seen
    keep_first: int                             # the sequence's first keys that stay seen behind the window

    @classmethod
    def from_dict(cls, d, where):
        h, g = _heads(d, where)
        mask = d.get("mask") or {}
        cap = d.get("softcap")
        c = cls(heads=h, kv_heads=g, dim=_int(d, "dim", where), vdim=_int(d, "vdim", where),
                scale=float(_need(d, "scale", where)), softcap=None if not cap else float(cap),
                window=None if not mask.get("size") else _int(mask, "size", where + ".mask"),
                keep_first=0 if not mask.get("keep_first") else _int(mask, "keep_first", where + ".mask", 0))
        if c.softcap is not None and not c.softcap > 0:
            raise ConfigError(f"config.json: {where}.softcap={c.softcap} must be positive")
        return c


@dataclass(frozen=True)
class DeltaConfig:
    """A gated delta rule: a ``delta`` layer's mixer, or the right mixer of a ``parallel`` layer."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, d, where):
        h, g = _heads(d, where)
        return cls(heads=h, kv_heads=g, dim=_int(d, "dim", where), vdim=_int(d, "vdim", where),
                   conv=1 if not d.get("conv") else _int(d, "conv", where))


@dataclass(frozen=True)
class RouterConfig:
    experts: int
    top: int
    identity: int
    scale: float
    groups: int
    keep: int

    @classmethod
    def from_dict(cls, d, where):
        g = d.get("groups") or {}
        count = 1 if not g.get("count") else _int(g, "count", where + ".groups")
        c = cls(experts=_int(d, "experts", where, 0), top=_int(d, "top", where),
                identity=0 if not d.get("identity") else _int(d, "identity", where, 0),
                scale=float(d.get("scale", 1.0)), groups=count,
                keep=count if not g.get("keep") else _int(g, "keep", where + ".groups"))
        total = c.experts + c.identity
        if total < 1 or c.top > total:
            raise ConfigError(f"config.json: {where}: {c.top} of {total} experts cannot be chosen")
        if total % c.groups or c.keep > c.groups or c.top > c.keep * (total // c.groups):
            raise ConfigError(f"config.json: {where}: {total} experts in {c.groups} groups of which {c.keep} are kept, "
                              f"{c.top} per token")
        return c


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                                   # "dense" | "moe"
    ff: int                                     # dense: its inner size; moe: an expert's
    router: Optional[RouterConfig] = None
    shared_ff: Optional[int] = None

    @classmethod
    def from_dict(cls, d, where):
        kind = _need(d, "kind", where)
        if kind == "dense":
            return cls(kind=kind, ff=_int(d, "ff", where))
        if kind == "moe":
            shared = d.get("shared")
            return cls(kind=kind, ff=_int(_need(d, "expert", where), "ff", where + ".expert"),
                       router=RouterConfig.from_dict(_need(d, "router", where), where + ".router"),
                       shared_ff=None if not shared else _int(shared, "ff", where + ".shared"))
        raise ConfigError(f"config.json: {where}.kind={kind!r}; the design has 'dense' and 'moe'")


@dataclass(frozen=True)
class PununexLayer:
    type: str
    delta: Optional[DeltaConfig] = None
    left: Optional[CappedAttentionConfig] = None
    right: Optional[DeltaConfig] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: Optional[FeedForwardConfig] = None


@dataclass(frozen=True)
class BigramConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class PununexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[PununexLayer, ...]
    bigram: Optional[BigramConfig] = None
    raw: dict = None                            # config.json as read (written back unchanged)
    architecture: str = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, d: dict) -> "PununexConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != ARCHITECTURE:
            raise ConfigError(f"config.json: architecture={name!r}, expected {ARCHITECTURE!r}")
        layers = []
        for i, L in enumerate(_need(d, "layers", "config")):
            where = f"layers[{i}]"
            kind = _need(L, "type", where)
            m = _need(L, "mixer", where)
            mlp = None if L.get("mlp") is None else FeedForwardConfig.from_dict(L["mlp"], where + ".mlp")
            if kind == "delta":
                layers.append(PununexLayer(type=kind, delta=DeltaConfig.from_dict(m, where + ".mixer"), mlp=mlp))
            elif kind == "parallel":
                layers.append(PununexLayer(
                    type=kind, mlp=mlp,
                    left=CappedAttentionConfig.from_dict(_need(m, "left", where + ".mixer"), where + ".mixer.left"),
                    right=DeltaConfig.from_dict(_need(m, "right", where + ".mixer"), where + ".mixer.right"),
                    left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0))))
            else:
                raise ConfigError(f"config.json: {where}.type={kind!r}; the design has 'delta' and 'parallel'")
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        bg = (d.get("embedding") or {}).get("bigram")
        bigram = None
        if bg:
            bigram = BigramConfig(buckets=_int(bg, "buckets", "embedding.bigram"), mul_prev=_int(bg, "mul_prev", "embedding.bigram", 0),
                                  mul_cur=_int(bg, "mul_cur", "embedding.bigram", 0))
        cfg = cls(vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"),
                  norm_eps=float(_need(_need(d, "norm", "config"), "eps", "norm")),
                  layers=tuple(layers), bigram=bigram, raw=copy.deepcopy(d))
        if not cfg.norm_eps >= 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        return cfg

    # ----------------------------------------------------------------- write
    def to_dict(self) -> dict:
        d = copy.deepcopy(self.raw)
        d.setdefault("architecture", ARCHITECTURE)
        return d

    # ------------------------------------------------------------ translation
    def _delta_spec(self, c: DeltaConfig, names: DeltaRuleNames, per_head: bool) -> DeltaRuleSpec:
        return DeltaRuleSpec(hidden=self.width, heads=c.heads, kv_heads=c.kv_heads, key_dim=c.dim, value_dim=c.vdim,
                             conv_taps=c.conv, norm_eps=self.norm_eps, names=names,
                             decay="head" if per_head else "channel", gate="silu" if per_head else "sigmoid_low_rank")

    def _mixer_spec(self, L: PununexLayer):
        W, eps = self.width, self.norm_eps
        if L.type == "delta":
            nm = DeltaRuleNames()
            pre = {f: "mix." + getattr(nm, f) for f in ("q", "k", "v", "beta", "a_log", "decay", "dt_bias", "gate", "norm", "o")}
            return self._delta_spec(L.delta, DeltaRuleNames(**pre), per_head=True)
        l = L.left
        left = HeadAttentionSpec(hidden=W, n_heads=l.heads, n_kv_heads=l.kv_heads, key_dim=l.dim, value_dim=l.vdim,
                                 softmax_scale=l.scale, eps=eps, window=l.window, keep_first=l.keep_first if l.window else 0,
                                 softcap=l.softcap, sink=True, names=HeadAttentionNames())
        right = self._delta_spec(L.right, DeltaRuleNames(), per_head=False)
        return ParallelMixerSpec(hidden=W, prefix="mix.", branches=(
            MixerBranch(left, "left.", L.left_scale), MixerBranch(right, "right.", L.right_scale)))

    def _ff_spec(self, c: Optional[FeedForwardConfig]):
        if c is None:
            return None
        W = self.width
        if c.kind == "dense":
            return GatedMLPSpec(hidden=W, intermediate=c.ff, activation="relu",
                                names=GatedMLPNames(gate="mlp.gate", up="mlp.up", down="mlp.down"))
        r = c.router
        shared = None
        if c.shared_ff:
            shared = GatedMLPSpec(hidden=W, intermediate=c.shared_ff, activation="silu",
                                  names=GatedMLPNames(gate="mlp.shared.gate", up="mlp.shared.up", down="mlp.shared.down"))
        return RoutedExpertsSpec(hidden=W, intermediate=c.ff, n_experts=r.experts, top=r.top, n_identity=r.identity,
                                 groups=r.groups, groups_keep=r.keep, scale=r.scale, activation="silu", shared=shared,
                                 router="mlp.router", correction="mlp.correction", expert="mlp.e{}.")

    def to_model_spec(self) -> ModelSpec:
        eps, W = self.norm_eps, self.width
        specs = []
        for i, L in enumerate(self.layers):
            ff = self._ff_spec(L.mlp)
            specs.append(PostNormLayerSpec(
                prefix=f"l{i}.", mixer=self._mixer_spec(L), mixer_post_norm=LayerNormSpec(size=W, eps=eps, weight="norm1"),
                mixer_scale="ls1", feed_forward=ff,
                feed_forward_post_norm=None if ff is None else LayerNormSpec(size=W, eps=eps, weight="norm2"),
                feed_forward_scale=None if ff is None else "ls2"))
        embedding = None
        if self.bigram is not None:
            b = self.bigram
            embedding = BigramHashSpec(hidden=W, buckets=b.buckets, mul_prev=b.mul_prev, mul_cur=b.mul_cur, table="bigram")
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden=W, layers=tuple(specs),
            schedule=default_schedule(len(specs)), final_norm=LayerNormSpec(size=W, eps=eps, weight="norm"),
            tie_embeddings=False, max_positions=MAX_POSITIONS, embed_name="embed", final_norm_prefix="final.",
            head_name="head", embedding=embedding)
