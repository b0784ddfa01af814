"""Architecture-neutral descriptions of a model: what each layer is made of.

An architecture's typed configuration (for instance ``Qwen3Config``) is
translated once into a ``ModelSpec``.  Everything below the registry (parts,
cache, engine, weights) works from these specs only, so no part knows which
model it is in, and another architecture is another translation.

A spec carries every size and constant its part needs.  The ``kind`` field of
a spec is the key under which the implementing class is registered
(``idempotent_llm_b200.parts.registry``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A configuration that cannot be built (bad value, missing key)."""


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding.

    Angles are ``position * theta ** (-2 j / dim)`` for ``j < dim / 2``, tiled
    twice (not interleaved); pairs are ``(d, d + dim / 2)``
    (reference: src/detllm/ops/rope.py:25-35, 47-55).  ``variant`` names how the
    rotation sits in a head, which the mixer's kernels must have:
    ``"half_whole_head"`` (``dim`` = the head size, pairs half a head apart),
    ``"half_partial"`` (the first ``dim`` dims of a head, pairs ``dim / 2`` apart) and
    ``"interleaved"`` (neighbours ``(2 j, 2 j + 1)`` turned by angle ``j``) are built, each by
    the mixers that name it; any other is refused by name.  ``scaling`` rescales the
    frequencies (``WavelengthScaling`` or ``RampScaling``).
    """

    theta: float
    dim: int
    max_positions: int
    variant: str = "half_whole_head"
    kind: str = "rotary"
    scaling: Optional["WavelengthScaling"] = None


@dataclass(frozen=True)
class WavelengthScaling:
    """Frequencies rescaled by wavelength ``l = 2 pi / f`` against a trained length ``original``: waves shorter
    than ``original / high`` are kept, waves longer than ``original / low`` are divided by ``factor``, and
    between the two the frequency is ``(1 - s) f / factor + s f`` with ``s = (original / l - low) /
    (high - low)``."""

    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class RampScaling:
    """Frequencies slowed down along a ramp over the index j (a stretch of the trained length ``original`` by
    ``factor``).  With ``at(n) = dim * ln(original / (2 pi n)) / (2 ln theta)`` the index whose wave makes ``n`` turns
    over the trained length, ``lo = max(floor(at(fast)), 0)``, ``hi = min(ceil(at(slow)), dim - 1)`` and ``s_j =
    clamp((j - lo) / max(hi - lo, 0.001), 0, 1)``, the frequency is ``s_j f_j / factor + (1 - s_j) f_j``; cos and sin
    are multiplied by ``0.1 ln(factor) + 1``."""

    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class DyTNormSpec:
    """A norm without statistics: ``tanh(alpha x) * w + b`` element by element, ``alpha`` one learned number.  The
    tensors are ``prefix + weight``, that name plus ``alpha_suffix`` and plus ``bias_suffix``."""

    size: int
    weight: str = "weight"
    alpha_suffix: str = ".alpha"
    bias_suffix: str = ".b"
    kind: str = "dyt"


@dataclass(frozen=True)
class NormSpec:
    """Root-mean-square norm over the last axis, weight applied afterwards.
    ``weight``: the tensor's name behind the prefix the block gives the norm."""

    size: int
    eps: float
    weight: str = "weight"
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class LayerNormSpec:
    """Layer norm over the last axis: ``(x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b``.  The weight is ``prefix +
    weight``, the bias that name plus ``bias_suffix``."""

    size: int
    eps: float
    weight: str = "weight"
    bias_suffix: str = ".b"
    kind: str = "layernorm"


@dataclass(frozen=True)
class AttentionNames:
    """Checkpoint names of an attention layer's tensors, behind the layer's prefix.  An architecture's
    configuration sets them; the part has none of its own."""

    q: str
    k: str
    v: str
    o: str
    q_norm: str
    k_norm: str


@dataclass(frozen=True)
class GatedMLPNames:
    """Checkpoint names of a gated feed-forward's matrices, behind the layer's prefix."""

    gate: str
    up: str
    down: str


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention (a *mixer*).

    ``head_dim`` is free of ``hidden / n_heads``.  ``qk_norm`` applies an
    RMS norm over ``head_dim`` with one weight shared by all heads to q and k
    before the position encoding (reference: src/detllm/model.py:200-216).
    ``window`` of W lets a query at position p see keys p-W+1 .. p; ``None``
    means all keys.  ``kv_from_other`` marks a layer that owns no k/v
    projection and reads the cache another layer wrote.
    """

    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    softmax_scale: float
    qk_norm: bool
    qk_norm_eps: float
    position: Optional[RotarySpec]
    names: AttentionNames
    window: Optional[int] = None
    kv_from_other: bool = False
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: ``down(act(gate(x)) * up(x))``
    (reference: src/detllm/model.py:415-427, src/detllm/ops/di_swiglu.py:43-45)."""

    hidden: int
    intermediate: int
    names: GatedMLPNames
    activation: str = "silu"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class LatentAttentionNames:
    """Checkpoint names of a latent attention's tensors, behind the mixer's prefix."""

    q: str = "q"
    down: str = "dkv"
    down_norm: str = "dkv.norm"
    up_k: str = "uk"
    up_v: str = "uv"
    o: str = "o"
    sink: str = "sink"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are made from one latent vector per token (a *mixer*).

    A head's query has ``plain_dim`` unrotated dims followed by ``rot_dim`` rotated ones.  The down projection
    gives ``kv_rank + rot_dim`` numbers per token: the first ``kv_rank``, divided by their root mean square (``eps``
    inside the root) and multiplied by a weight, are the latent ``c``; the last ``rot_dim``, rotated, are a key part
    all heads share.  Head h's unrotated key is ``Uk_h c`` and its value ``Uv_h c`` (``value_dim`` numbers); the score
    is ``(q_plain . k_plain + q_rot . k_rot) * softmax_scale``.  ``position`` (variant ``"interleaved"``) turns the
    first ``position.dim`` of the rotated dims.  ``sink``: one learned score per head joins the softmax's
    denominator with no key and no value.  Only ``c`` and the rotated key part are kept per token."""

    hidden: int
    n_heads: int
    plain_dim: int
    rot_dim: int
    value_dim: int
    kv_rank: int
    softmax_scale: float
    eps: float
    position: Optional[RotarySpec] = None
    sink: bool = False
    names: LatentAttentionNames = LatentAttentionNames()
    kind: str = "latent_attention"


@dataclass(frozen=True)
class DenseMLPNames:
    up: str = "up"
    down: str = "down"


@dataclass(frozen=True)
class DenseMLPSpec:
    """Feed-forward without a gate: ``down(act(up(x)))``; ``activation`` ``"relu2"`` is the square of relu."""

    hidden: int
    intermediate: int
    activation: str = "relu2"
    names: DenseMLPNames = DenseMLPNames()
    kind: str = "dense_mlp"


@dataclass(frozen=True)
class TableExpertsSpec:
    """``n_experts`` small gated feed-forwards ``down_e(act(gate_e x) * up_e x)`` of which a token uses ``top``, named by
    a table ``[vocab_size, top]`` of integers indexed by the token's id (no learned router), each with weight
    ``1 / top``.  Expert e's tensors are ``prefix + expert.format(e) + gate / up / down``."""

    hidden: int
    intermediate: int
    n_experts: int
    top: int
    vocab_size: int
    activation: str = "silu"
    table: str = "table"
    expert: str = "e{}."
    names: GatedMLPNames = GatedMLPNames(gate="gate", up="up", down="down")
    kind: str = "table_experts"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """``n_experts`` small gated feed-forwards ``down_e(act(gate_e x) * up_e x)`` and ``n_identity`` experts that hand
    their input on, of which a token uses ``top``, named by a learned router.  With ``z = W_r x`` over all ``n_experts +
    n_identity`` outputs (32-bit): ``s = softmax(z)``; experts are CHOSEN by ``s + correction`` (a learned row), the
    ``top`` largest among the experts of the ``groups_keep`` best of ``groups`` equal groups of neighbours (a group's
    score: its largest choice score); the WEIGHTS are the chosen experts' ``s`` over their sum (+ 1e-20), times
    ``scale``.  ``shared``: a gated feed-forward of the same form that every token runs, added to the sum.  Expert e's
    tensors are ``prefix + expert.format(e) + gate / up / down``; identity experts are the router's last outputs and
    have no tensors."""

    hidden: int
    intermediate: int
    n_experts: int
    top: int
    n_identity: int = 0
    groups: int = 1
    groups_keep: int = 1
    scale: float = 1.0
    activation: str = "silu"
    shared: Optional["GatedMLPSpec"] = None
    router: str = "router"
    correction: str = "correction"
    expert: str = "e{}."
    names: GatedMLPNames = GatedMLPNames(gate="gate", up="up", down="down")
    kind: str = "routed_experts"


@dataclass(frozen=True)
class SinkAttentionNames:
    """Checkpoint names of a gated attention with short filters and a sink, behind the mixer's prefix; a filter's
    tensor is its projection's name plus ``conv``."""

    q: str = "q"
    k: str = "k"
    v: str = "v"
    o: str = "o"
    gate: str = "g"
    sink: str = "sink"
    conv: str = ".conv"


@dataclass(frozen=True)
class SinkAttentionSpec:
    """Causal grouped-query attention (a *mixer*) with, each optional: a short causal filter over time on
    every channel of q, k and v (``conv_taps`` > 1) directly behind the projections; a rotation of the first
    ``position.dim`` dims of each q and k head (variant ``"half_partial"``: dim i with dim i + dim / 2, the rest
    untouched); one learned score per head that joins the softmax's denominator with no key and no value
    (``sink``); the merged heads times ``sigmoid(gate projection of the mixer's input)`` before the output
    projection (``gate``).  Keys have ``key_dim`` and values ``value_dim`` elements per head."""

    hidden: int
    n_heads: int
    n_kv_heads: int
    key_dim: int
    value_dim: int
    softmax_scale: float
    conv_taps: int = 1
    position: Optional[RotarySpec] = None
    sink: bool = True
    gate: bool = True
    names: SinkAttentionNames = SinkAttentionNames()
    kind: str = "sink_attention"


@dataclass(frozen=True)
class SSDNames:
    """Checkpoint names of a state-space mixer, behind the mixer's prefix."""

    w_in: str = "in"
    conv: str = "conv"
    conv_bias: str = "conv.b"
    dt_bias: str = "dt_bias"
    a_log: str = "A_log"
    d: str = "D"
    norm: str = "norm"
    o: str = "o"


@dataclass(frozen=True)
class SSDSpec:
    """Selective state-space mixer with a scalar decay per head (the state-space duality form).  The input
    projection's rows are ``[z: inner | x: inner | B: groups * state | C: groups * state | dt: heads]`` with
    ``inner = heads * head_dim``; x, B and C pass a causal filter of ``conv_taps`` taps with bias and silu;
    ``dt = softplus(dt + dt_bias)``; per head ``S <- exp(-exp(A_log) dt) S + dt B x^T``, ``y = S^T C + D x``;
    ``y * silu(z)`` is normed in ``norm_groups`` equal parts (each by its own root mean square), times a
    weight; then the output projection."""

    hidden: int
    heads: int
    head_dim: int
    state: int
    groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    names: SSDNames = SSDNames()
    kind: str = "ssd"


@dataclass(frozen=True)
class HeadAttentionNames:
    """Checkpoint names of a normed attention's tensors, behind the mixer's prefix; a projection's bias is its
    name plus ``bias``."""

    q: str = "q"
    k: str = "k"
    v: str = "v"
    o: str = "o"
    q_norm: str = "q.norm"
    k_norm: str = "k.norm"
    gate: str = "g"
    bias: str = ".b"
    sink: str = "sink"


@dataclass(frozen=True)
class HeadAttentionSpec:
    """Causal grouped-query attention (a *mixer*) whose q and k heads are normed (RMS over the head, one weight
    for all heads, ``eps``) before an optional rotation of the first ``position.dim`` dims of each head (variant
    ``"half_partial"``).  Each of the following is an option: biases on the input projections (``bias_in``) and on
    the output projection (``bias_out``); ``values_from_keys``: there is no value projection, a token's value is its
    key as projected (with bias, before norm and rotation); ``window`` of W: a query at p sees keys p - W + 1 .. p;
    ``unit_sink``: the softmax's denominator has one more term of score 0 and no value; ``sink``: that term's score is a
    learned number per head instead (tensor ``names.sink`` [heads]; it is neither scaled nor capped); ``keep_first`` of F
    (with a window): a query also sees the sequence's first F keys, however far back; ``softcap`` c: a score becomes
    ``c tanh(score / c)`` after the scale; ``slope_exponent`` c: head h of H takes ``2^(-c (h + 1) / H)`` times the
    distance to a key off its score; ``head_gate``: a head's output times ``sigmoid`` of one number per head projected
    from the mixer's input."""

    hidden: int
    n_heads: int
    n_kv_heads: int
    key_dim: int
    value_dim: int
    softmax_scale: float
    eps: float
    qk_norm: bool = True
    position: Optional[RotarySpec] = None
    window: Optional[int] = None
    unit_sink: bool = False
    slope_exponent: Optional[float] = None
    head_gate: bool = False
    values_from_keys: bool = False
    bias_in: bool = False
    bias_out: bool = False
    sink: bool = False
    keep_first: int = 0
    softcap: Optional[float] = None
    names: HeadAttentionNames = HeadAttentionNames()
    kind: str = "head_attention"


@dataclass(frozen=True)
class DeltaRuleNames:
    """Checkpoint names of a gated delta rule's tensors, behind the mixer's prefix; a filter's tensor is its
    projection's name plus ``conv``."""

    q: str = "q"
    k: str = "k"
    v: str = "v"
    conv: str = ".conv"
    beta: str = "b"
    a_log: str = "A_log"
    decay_down: str = "a1"
    decay_up: str = "a2"
    dt_bias: str = "dt_bias"
    gate_down: str = "g1"
    gate_up: str = "g2"
    decay: str = "a"
    gate: str = "g"
    norm: str = "norm"
    o: str = "o"


@dataclass(frozen=True)
class DeltaRuleSpec:
    """Gated delta rule (a recurrent *mixer*): per head a state ``S [key_dim, value_dim]``, per token ``S <- diag(g)
    S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``.  q, k (``kv_heads`` heads of ``key_dim``) and v (``heads`` of
    ``value_dim``) pass a causal filter of ``conv_taps`` taps per channel and silu; q and k become unit vectors per head
    (``x / sqrt(sum x^2 + 1e-6)``), q also times ``key_dim ** -0.5``; ``beta = sigmoid(W_b h)`` per head; ``g =
    exp(-exp(A_log_h) softplus(W_a2 W_a1 h + dt_bias))`` per head and key channel; the read-out is divided by its
    root mean square over ``value_dim`` (``norm_eps``), times a weight ``[value_dim]``, times ``sigmoid(W_g2 W_g1
    h)``.  ``decay_rank`` / ``gate_rank`` are the inner sizes of the two low-rank projections; None: whatever the
    checkpoint's tensors have (random weights then take ``key_dim // 2`` rounded up to 8).

    ``decay`` ``"head"`` instead of ``"channel"``: one decay per head, ``g = exp(-exp(A_log_h) softplus(W_a h + dt_bias_h))``
    with a full matrix ``names.decay`` [heads, hidden] and ``dt_bias`` [heads].  ``gate`` ``"silu"`` instead of
    ``"sigmoid_low_rank"``: the read-out times ``silu(W_g h)`` with a full matrix ``names.gate`` [heads * value_dim,
    hidden]."""

    hidden: int
    heads: int
    kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None
    decay: str = "channel"
    gate: str = "sigmoid_low_rank"
    names: DeltaRuleNames = DeltaRuleNames()
    kind: str = "gated_delta"


@dataclass(frozen=True)
class MixerBranch:
    """One of the mixers of a ``ParallelMixerSpec``: its spec, the prefix of its tensors behind the parallel
    mixer's own, and the constant its output is multiplied with."""

    mixer: object
    prefix: str
    scale: float = 1.0


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side that read the same input; the result is the sum of their outputs, each times
    its constant.  At most one branch keeps keys and values; any may keep per-sequence state."""

    hidden: int
    branches: Tuple[MixerBranch, ...]
    prefix: str = ""
    kind: str = "parallel"


@dataclass(frozen=True)
class TokenSideSpec:
    """A per-layer input that depends on the token itself: ``g = act(gate h) * e`` with ``e`` the columns
    ``[col0, col0 + dim)`` of the token's row of a second embedding table shared by all layers; ``y = proj g``;
    ``h += y / sqrt(mean(y^2) + eps) * norm``."""

    hidden: int
    dim: int
    col0: int
    vocab_size: int
    table_width: int
    eps: float
    table: str                      # the shared table's checkpoint name (no layer prefix)
    gate: str = "side.gate"
    proj: str = "side.proj"
    norm: str = "side.norm"
    activation: str = "gelu_tanh"
    kind: str = "token_side"


@dataclass(frozen=True)
class SandwichLayerSpec:
    """A layer that norms every sublayer's input AND output: ``h += post(mixer(pre(h)))``, then, if it has a
    feed-forward, ``h += post(ff(pre(h)))``, then, if it has one, the token side input.  The four norms'
    tensors are ``prefix + <NormSpec.weight>``."""

    prefix: str
    mixer: object
    mixer_norm: NormSpec
    mixer_post_norm: NormSpec
    feed_forward: Optional[object] = None
    feed_forward_norm: Optional[NormSpec] = None
    feed_forward_post_norm: Optional[NormSpec] = None
    token_side: Optional[TokenSideSpec] = None
    kind: str = "sandwich"


@dataclass(frozen=True)
class PostNormLayerSpec:
    """A layer whose sublayers read the stream itself and whose norms sit BEHIND them: ``h += s1 * N1(mixer(h))``,
    then, if it has a feed-forward, ``h += s2 * N2(ff(h))``.  ``mixer_scale`` / ``feed_forward_scale`` name learned rows
    ``[hidden]`` (None: no scale).  The norms' tensors are ``prefix + <spec.weight>``."""

    prefix: str
    mixer: object
    mixer_post_norm: object
    feed_forward: Optional[object] = None
    feed_forward_post_norm: Optional[object] = None
    mixer_scale: Optional[str] = None
    feed_forward_scale: Optional[str] = None
    kind: str = "postnorm"


@dataclass(frozen=True)
class BigramHashSpec:
    """A token embedding with a hashed bigram row added: ``E[token_t] + B[(mul_prev * token_(t-1) + mul_cur * token_t)
    mod buckets]``, and ``B[buckets]`` (the table's last row) for a sequence's first token.  A sequence's last token is
    part of its state between steps."""

    hidden: int
    buckets: int
    mul_prev: int
    mul_cur: int
    table: str = "bigram"
    kind: str = "bigram_hash"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which block arrangement, and the parts inside it.

    ``prefix`` is the weight-name prefix of the layer (``model.layers.3.``);
    ``mixer_norm_prefix`` / ``feed_forward_norm_prefix`` follow it for the two norms'
    tensors.  ``mixer`` and ``feed_forward`` are specs of any registered kind.
    """

    prefix: str
    mixer: object
    feed_forward: object                # None: the layer has no feed-forward (then no second norm either)
    mixer_norm: object
    feed_forward_norm: object
    mixer_norm_prefix: str
    feed_forward_norm_prefix: str
    kind: str = "prenorm"           # "parallel_residual": h += mixer(norm1(h)) + feed_forward(norm2(h)), both norms of the same h


@dataclass(frozen=True)
class RunEntry:
    """One stop in the order in which layers run.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named twice).
    ``cache`` names the cache entry the mixer uses; entries that share a
    number share keys and values.  ``writes_cache`` is False for a mixer that
    only reads what an earlier entry wrote.  ``mix_in``: before this stop the
    stream is replaced by ``M [stream ; embedding output]`` with the model's
    ``ModelSpec.mix_in_name`` matrix ``[hidden, 2 hidden]`` (the opening of a
    pass over layers that run several times).
    """

    layer: int
    cache: int
    writes_cache: bool = True
    mix_in: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[RunEntry, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    max_positions: int
    embed_name: str                     # checkpoint names: set by the architecture's configuration
    final_norm_prefix: str
    head_name: str
    stop_token_ids: Tuple[int, ...] = ()
    init_std: float = 0.02
    embed_scale: float = 1.0            # the embedding row is multiplied with this constant
    mix_in_name: Optional[str] = None   # the matrix of the schedule's `mix_in` stops
    logit_scale: float = 1.0            # logits are multiplied with this constant, then
    logit_softcap: Optional[float] = None   # capped: cap * tanh(logits / cap)
    embedding: Optional[object] = None      # a registered kind of token embedding (``BigramHashSpec``); None: a plain lookup
    extra: dict = field(default_factory=dict, compare=False)

    def __post_init__(self):
        n = len(self.layers)
        seen_writer = set()
        for e in self.schedule:
            if not 0 <= e.layer < n:
                raise ConfigError(f"schedule names layer {e.layer}, model has {n}")
            if e.writes_cache:
                if e.cache in seen_writer:
                    raise ConfigError(f"cache entry {e.cache} is written by two schedule entries")
                seen_writer.add(e.cache)
            elif e.cache not in seen_writer:
                raise ConfigError(f"schedule entry reads cache {e.cache} before anything wrote it")
            if e.mix_in and not self.mix_in_name:
                raise ConfigError("a schedule entry mixes the embedding in, but the model names no matrix for it")


def default_schedule(n_layers: int) -> Tuple[RunEntry, ...]:
    """Every layer once, in order, each with a cache entry of its own."""
    return tuple(RunEntry(layer=i, cache=i) for i in range(n_layers))
