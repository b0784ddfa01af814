"""The Pununex decoder on the GPU against the plain implementation (``plain_pununex.py``): every mechanism alone,
then whole models through the engine: prompts, token-by-token decoding, portions, unequal batches, slots and pages
used again, marked keys far away, at page borders, at a window's edges and among the kept first tokens, first tokens,
long decoding, drawn configurations, greedy generation, and the trace replay program."""

import os

import pytest
import torch

import helpers
import plain_pununex as plain
from idempotent_llm_b200 import api
from idempotent_llm_b200.cache import SequenceCache
from idempotent_llm_b200.config import BigramHashSpec, DeltaRuleSpec, GatedMLPSpec, HeadAttentionSpec, RoutedExpertsSpec
from idempotent_llm_b200.config.specs import GatedMLPNames
from idempotent_llm_b200.engine.batch import context_from_packed, pack_step_host
from idempotent_llm_b200.parts import EMBEDDINGS, FEED_FORWARDS, MIXERS, Runtime
from idempotent_llm_b200.weights import random_weights

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# against the 64-bit plain implementation, relative to the largest value: 32-bit sums of a few hundred terms; bfloat16
# rounds activations (8 bits of mantissa) a handful of times per layer
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
F64 = torch.float64


def _close(got, want, dtype):
    if dtype == "float32":
        return helpers.rel_err(got, want) < TOL[dtype]
    g, w = got.detach().double().cpu(), want.detach().double().cpu()
    rms = float((g - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt())
    return rms < TOL[dtype] and helpers.rel_err(got, want) < 0.25


def _close_rows(got, want, dtype):
    """For a routed feed-forward alone in bfloat16: a token whose two best choice scores lie within the rounding of
    the router's input may take another expert than the 64-bit witness, so a row in thirty may be off; every other row
    is held to the type's tolerance.  32-bit is held as ever."""
    if dtype == "float32":
        return _close(got, want, dtype)
    g, w = got.detach().double().cpu(), want.detach().double().cpu()
    rows = ((g - w).pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt())
    return int((rows > TOL[dtype]).sum()) <= max(1, rows.numel() // 30) and float(rows.median()) < TOL[dtype] / 2


def _rt(dtype):
    from idempotent_llm_b200.kernels import Kernels
    dev = torch.device("cuda:0")
    return Runtime(device=dev, dtype=DT[dtype], kernels=Kernels(DT[dtype], dev))


def _ctx(slots, starts, lens, tokens=None):
    toks = tokens if tokens is not None else [[0] * L for L in lens]
    packed, n, q_lens = pack_step_host(slots, starts, toks)
    return context_from_packed(packed.cuda(), n, slots, q_lens, starts, host_tokens=toks)


def _w64(w):
    return {k: (v.double().cpu() if v.is_floating_point() else v.cpu()) for k, v in w.items()}


def _cuts(T, sizes):
    out, lo, i = [], 0, 0
    while lo < T:
        n = sizes[min(i, len(sizes) - 1)]
        out.append((lo, min(T, lo + n)))
        lo, i = lo + n, i + 1
    return out


# ----------------------------------------------------------------------------------- the attention, alone
def _head_spec(**kw):
    base = dict(hidden=40, n_heads=6, n_kv_heads=2, key_dim=24, value_dim=16, softmax_scale=0.3, eps=1e-5, sink=True)
    base.update(kw)
    return HeadAttentionSpec(**base)


def _plain_left(x, w, s, p):
    c = dict(heads=s.n_heads, kv_heads=s.n_kv_heads, dim=s.key_dim, vdim=s.value_dim, scale=s.softmax_scale, softcap=s.softcap,
             mask=dict(size=s.window, keep_first=s.keep_first) if s.window else None)
    if not s.sink:
        w = {k: v for k, v in w.items() if k != p + "sink"}
    return plain.window_attention(x, w, p, c, s.eps)


HEAD_VARIANTS = {
    # the design's left mixer: a cap, a window with kept tokens, a learned sink, values narrower than keys
    "capped_window": lambda: _head_spec(window=37, keep_first=4, softcap=3.0),
    # kept tokens that fill a block of 32 keys, more than one, and a whole page and one; windows around them
    "keep_32": lambda: _head_spec(window=9, keep_first=32, softcap=8.0, n_kv_heads=1),
    "keep_33": lambda: _head_spec(window=64, keep_first=33, softcap=None),
    "keep_65": lambda: _head_spec(window=5, keep_first=65, softcap=50.0, value_dim=40),
    # a window of one key: a token sees itself, the kept ones and the sink
    "window_1": lambda: _head_spec(window=1, keep_first=2, softcap=2.0),
    # more kept tokens than the sequence ever has; no kept tokens; no window at all (kept tokens mean nothing then)
    "keep_all": lambda: _head_spec(window=20, keep_first=10000, softcap=5.0),
    "keep_none": lambda: _head_spec(window=20, keep_first=0, softcap=5.0),
    "no_window": lambda: _head_spec(window=None, keep_first=0, softcap=1.5, n_heads=3, n_kv_heads=3, key_dim=10, value_dim=12),
    # no sink: the cap and the kept tokens alone
    "no_sink": lambda: _head_spec(window=30, keep_first=3, softcap=4.0, sink=False),
    # head sizes the tensor cores have
    "capped_64": lambda: _head_spec(n_heads=4, n_kv_heads=2, key_dim=64, value_dim=64, softmax_scale=0.15, window=100, keep_first=7,
                                    softcap=25.0),
    "capped_128_long": lambda: _head_spec(n_heads=2, n_kv_heads=1, key_dim=128, value_dim=128, softmax_scale=0.09, window=700,
                                          keep_first=70, softcap=30.0),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", sorted(HEAD_VARIANTS))
def test_capped_attention_alone_prompt_then_single_tokens(dtype, variant):
    spec = HEAD_VARIANTS[variant]()
    rt = _rt(dtype)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "M."), 5, 0.25, dtype=DT[dtype], device="cuda")
    for n in ("M.q.norm", "M.k.norm"):                                # sharper scores than random weights give: the cap bites
        w[n] = (w[n].float() * 2.0).to(DT[dtype])
    part = cls(spec, w, "M.", rt)
    T, pre = (1300, 1290) if variant.endswith("long") else (150, 131)
    cache = SequenceCache({0: cls.cache_need(spec)}, 64 * 24, DT[dtype], "cuda:0", max_seqs=2)
    slot = cache.alloc_slot()
    x = (torch.randn(T, spec.hidden, generator=torch.Generator().manual_seed(3)) * 1.5).to(DT[dtype])
    ref = _plain_left(x.double(), _w64(w), spec, "M.")
    outs = []
    for lo, hi in [(0, 70), (70, pre)] + [(i, i + 1) for i in range(pre, T)]:
        cache.reserve([(slot, hi)]); cache.flush()
        ctx = _ctx([slot], [lo], [hi - lo])
        outs.append(part.forward(x[lo:hi].contiguous().cuda(), ctx, cache.view(0), cache.state_of(0), True).sum(0))
        cache.set_length(slot, hi)
    assert helpers.rel_err(torch.cat(outs), ref) < TOL[dtype]


TC_SHAPES = {
    # (head size, q-heads, kv-heads, window, kept tokens, cap): kept tokens inside the window's first key block, in
    # blocks of their own far before it, more than a key block of them, more than a run of key blocks of them
    "w600_k5_h64_g8": (64, 8, 1, 600, 5, 20.0),
    "w1100_k70_h128_g2": (128, 4, 2, 1100, 70, 30.0),
    "w65_k64_h64_g4": (64, 4, 1, 65, 64, None),
    "w100_k600_h64_g2": (64, 2, 1, 100, 600, 8.0),
    "w1_k1_h64_g1": (64, 1, 1, 1, 1, 5.0),
    "cap_only_h128_g1": (128, 2, 2, None, 0, 10.0),
}


@pytest.mark.parametrize("shape", sorted(TC_SHAPES))
def test_caps_and_kept_tokens_on_the_tensor_cores_against_the_general_kernel(shape):
    """bfloat16 with head sizes of 64 and 128 runs on the tensor cores; the general kernel is the witness.  Two unequal
    sequences in the same steps: a long prompt, a portion behind it, single tokens."""
    hd, H, G, window, keep, cap = TC_SHAPES[shape]
    spec = _head_spec(hidden=32, n_heads=H, n_kv_heads=G, key_dim=hd, value_dim=hd, softmax_scale=hd ** -0.5, window=window,
                      keep_first=keep, softcap=cap)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "M."), 9, 0.3, dtype=torch.bfloat16, device="cuda")
    w["M.q.norm"] = (w["M.q.norm"].float() * 2.5).to(torch.bfloat16)       # sharp scores: single keys carry weight
    lens = (2900, 1500)
    x = [(torch.randn(n, 32, generator=torch.Generator().manual_seed(3 + n)) * 1.5).to(torch.bfloat16).cuda() for n in lens]
    outs = {}
    for impl in ("generic", "tcgen05"):
        rt = _rt("bfloat16")
        rt.kernels.attention_impl = impl
        calls, inner = [], rt.kernels.attention_tc
        rt.kernels.attention_tc = lambda *a, _f=inner, **k: (calls.append(1), _f(*a, **k))[1]
        part = cls(spec, w, "M.", rt)
        cache = SequenceCache({0: cls.cache_need(spec)}, 64 * 80, torch.bfloat16, "cuda:0", max_seqs=2)
        slots = [cache.alloc_slot(), cache.alloc_slot()]
        got, at = [[], []], [0, 0]
        steps = [(2500, 1200), (380, 290)] + [(1, 1)] * 10 + [(10, 0)]
        for step in steps:
            live = [i for i in (0, 1) if step[i]]
            hi = [at[i] + step[i] for i in live]
            cache.reserve([(slots[i], h) for i, h in zip(live, hi)]); cache.flush()
            ctx = _ctx([slots[i] for i in live], [at[i] for i in live], [step[i] for i in live])
            y = part.forward(torch.cat([x[i][at[i]:h] for i, h in zip(live, hi)]), ctx, cache.view(0), None, True).sum(0)
            off = 0
            for i, h in zip(live, hi):
                got[i].append(y[off:off + step[i]]); off += step[i]
                cache.set_length(slots[i], h); at[i] = h
        assert rt.kernels.attention_tc_status() == 0 and (len(calls) == len(steps)) == (impl == "tcgen05")
        outs[impl] = [torch.cat(g) for g in got]
    for i in (0, 1):
        ref = _plain_left(x[i].double().cpu(), _w64(w), spec, "M.")
        assert helpers.rel_err(outs["generic"][i], ref) < TOL["bfloat16"]
        assert helpers.rel_err(outs["tcgen05"][i], ref) < TOL["bfloat16"]
        assert helpers.rel_err(outs["tcgen05"][i], outs["generic"][i]) < 2e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_learned_sink_takes_weight_without_a_value(dtype):
    """A sink far above every score leaves nothing of the values; one far below is as good as none; the cap does not
    touch it (a sink of 9 against scores capped at 2 still takes nearly all the weight)."""
    spec = _head_spec(window=None, softcap=2.0)
    rt = _rt(dtype)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "M."), 6, 0.25, dtype=DT[dtype], device="cuda")
    x = (torch.randn(40, spec.hidden, generator=torch.Generator().manual_seed(4)) * 1.5).to(DT[dtype])
    out = {}
    for name, value in (("high", 60.0), ("nine", 9.0), ("low", -60.0)):
        w["M.sink"] = torch.full_like(w["M.sink"], value)
        part = cls(spec, w, "M.", rt)
        cache = SequenceCache({0: cls.cache_need(spec)}, 128, DT[dtype], "cuda:0", max_seqs=1)
        slot = cache.alloc_slot()
        cache.reserve([(slot, 40)]); cache.flush()
        out[name] = part.forward(x.cuda(), _ctx([slot], [0], [40]), cache.view(0), None, True).sum(0)
        assert helpers.rel_err(out[name], _plain_left(x.double(), _w64(w), spec, "M.")) < TOL[dtype] or name == "high"
    import dataclasses
    none = dataclasses.replace(spec, sink=False)
    assert float(out["high"].abs().max()) < 1e-12 * float(out["low"].abs().max()) + 1e-20
    assert helpers.rel_err(out["low"], _plain_left(x.double(), _w64(w), none, "M.")) < TOL[dtype]
    assert float(out["nine"].abs().max()) < 0.05 * float(out["low"].abs().max())


# ----------------------------------------------------------------------------------- the delta rule, alone
def _delta_spec(**kw):
    base = dict(hidden=40, heads=4, kv_heads=2, key_dim=12, value_dim=20, conv_taps=3, norm_eps=1e-5, decay="head", gate="silu")
    base.update(kw)
    return DeltaRuleSpec(**base)


DELTA_VARIANTS = {
    "head_decay_silu": lambda: _delta_spec(),
    "one_head_one_tap": lambda: _delta_spec(heads=1, kv_heads=1, key_dim=8, value_dim=8, conv_taps=1),
    "wide": lambda: _delta_spec(heads=2, kv_heads=2, key_dim=64, value_dim=128, conv_taps=4),
    "keys_130": lambda: _delta_spec(heads=2, kv_heads=1, key_dim=130, value_dim=6, conv_taps=2),
    # the two choices are independent of each other
    "head_decay_low_rank_gate": lambda: _delta_spec(gate="sigmoid_low_rank", gate_rank=8),
    "channel_decay_silu": lambda: _delta_spec(decay="channel", decay_rank=16),
    "channel_decay_low_rank_gate": lambda: _delta_spec(decay="channel", gate="sigmoid_low_rank", decay_rank=8, gate_rank=16),
}


def _plain_delta(x, w, s, p):
    T = x.shape[0]
    c = dict(heads=s.heads, kv_heads=s.kv_heads, dim=s.key_dim, vdim=s.value_dim)
    q, k, v, beta = plain.delta_inputs(x, w, p, c)
    if s.decay == "head":
        g = torch.exp(-torch.exp(w[p + "A_log"]) * plain.softplus(x @ w[p + "a"].T + w[p + "dt_bias"]))[:, :, None].expand(T, s.heads, s.key_dim)
    else:
        dt = plain.softplus((x @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, s.heads, s.key_dim)
        g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * dt)
    o = plain.rms_norm(plain.delta_recurrence(q, k, v, beta, g), w[p + "norm"], s.norm_eps)
    if s.gate == "silu":
        o = o * plain.silu(x @ w[p + "g"].T).view(T, s.heads, s.value_dim)
    else:
        o = o * torch.sigmoid((x @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, s.heads, s.value_dim)
    return o.reshape(T, -1) @ w[p + "o"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", sorted(DELTA_VARIANTS))
def test_delta_rule_alone_in_portions(dtype, variant):
    spec = DELTA_VARIANTS[variant]()
    rt = _rt(dtype)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "M."), 7, 0.2, dtype=DT[dtype], device="cuda")
    part = cls(spec, w, "M.", rt)
    cache = SequenceCache({0: cls.cache_need(spec)}, 256, DT[dtype], "cuda:0", max_seqs=2)
    T = 120
    x = (torch.randn(T, spec.hidden, generator=torch.Generator().manual_seed(8)) * 1.2).to(DT[dtype])
    ref = _plain_delta(x.double(), _w64(w), spec, "M.")
    for sizes in ([T], [1], [2], [3, 1, 40, 2, 17]):
        slot = cache.alloc_slot()
        outs = []
        for lo, hi in _cuts(T, sizes):
            cache.reserve([(slot, hi)]); cache.flush()
            outs.append(part.forward(x[lo:hi].contiguous().cuda(), _ctx([slot], [lo], [hi - lo]), None, cache.state_of(0), True).sum(0))
            cache.set_length(slot, hi)
        cache.free_slot(slot)
        assert _close(torch.cat(outs), ref, dtype), f"portions of {sizes}"


# ----------------------------------------------------------------------------------- router and experts, alone
ROUTER_SHAPES = [
    # experts (identity experts among them), per token, groups, kept groups
    (18, 2, 3, 1), (7, 3, 1, 1), (64, 6, 8, 3), (3, 3, 1, 1), (12, 4, 4, 4), (40, 1, 5, 1), (96, 8, 3, 2), (2, 1, 2, 1),
]


@pytest.mark.parametrize("E,top,groups,keep", ROUTER_SHAPES)
@pytest.mark.parametrize("shift", [0.0, -3.0])
def test_the_router_kernel_against_plain(E, top, groups, keep, shift):
    """Choice by corrected scores inside the best groups, weights from the uncorrected ones.  With ``shift`` every
    choice score is negative: an expert that is shut out must count as minus infinity, not as zero."""
    K = _rt("float32").kernels
    g = torch.Generator().manual_seed(E * 7 + top)
    z = (torch.randn(300, E, generator=g) * 2.0).cuda()
    corr = (torch.randn(E, generator=g) * 0.1 + shift).cuda()
    chosen, weight = K.route(z, corr, top, groups, keep, 1.7)
    want_c, want_w = plain.route(z.double().cpu(), corr.double().cpu(), dict(top=top, scale=1.7, groups=dict(count=groups, keep=keep)))
    assert torch.equal(chosen.cpu().long(), want_c)
    assert helpers.rel_err(weight, want_w) < 1e-5


def _moe_spec(shared=40, **kw):
    base = dict(hidden=32, intermediate=24, n_experts=6, top=3, n_identity=2, groups=4, groups_keep=2, scale=1.5)
    base.update(kw)
    if shared:
        base["shared"] = GatedMLPSpec(hidden=base["hidden"], intermediate=shared, names=GatedMLPNames("shared.gate", "shared.up", "shared.down"))
    return RoutedExpertsSpec(**base)


MOE_VARIANTS = {
    "groups_identity_shared": lambda: _moe_spec(),
    "one_of_three": lambda: _moe_spec(n_experts=3, top=1, n_identity=0, groups=1, groups_keep=1, scale=1.0, shared=None),
    "off_borders": lambda: _moe_spec(hidden=20, intermediate=12, n_experts=5, n_identity=1, top=2, groups=3, groups_keep=3, shared=28),
    "many": lambda: _moe_spec(hidden=64, intermediate=32, n_experts=16, n_identity=0, top=2, groups=2, groups_keep=1, scale=2.5),
    "identity_only_beside_one": lambda: _moe_spec(n_experts=1, n_identity=3, top=2, groups=2, groups_keep=2, shared=None),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", sorted(MOE_VARIANTS))
def test_routed_experts_alone_in_steps_of_every_size(dtype, variant):
    """3 tokens (every pair streams its expert), 30 and 100 (expert by expert, or every expert over all tokens), 300
    (rows grouped by expert on the host), and 300 without the host's help (a captured step's way): the same sums."""
    spec = MOE_VARIANTS[variant]()
    rt = _rt(dtype)
    cls = FEED_FORWARDS.get(spec.kind)
    w = random_weights(cls.declare(spec, "F."), 11, 0.2, dtype=DT[dtype], device="cuda")
    w["F.router"] = (w["F.router"].float() * 6.0).to(DT[dtype])          # decisive choices: few calls close enough to round over
    part = cls(spec, w, "F.", rt)
    w64 = _w64(w)
    c = dict(kind="moe", expert=dict(ff=spec.intermediate), shared=dict(ff=1) if spec.shared else None,
             router=dict(experts=spec.n_experts, identity=spec.n_identity, top=spec.top, scale=spec.scale,
                         groups=dict(count=spec.groups, keep=spec.groups_keep)))
    for n, host in ((3, True), (30, True), (100, True), (300, True), (300, False)):
        x = (torch.randn(n, spec.hidden, generator=torch.Generator().manual_seed(n)) * 1.3).to(DT[dtype])
        ctx = _ctx([0], [0], [n])
        if not host:
            ctx.host_tokens = None
        got = part.forward(x.cuda(), ctx).sum(0)
        want = plain.routed_ff(x.double(), w64, "F.", c)
        assert _close_rows(got, want, dtype), f"{n} tokens, host {host}"
        if dtype == "float32":                                           # the choices themselves
            chosen, weight = part.route(x.cuda())
            want_c, want_w = plain.route(x.double() @ w64["F.router"].T, w64["F.correction"], c["router"])
            assert torch.equal(chosen.cpu().long(), want_c) and helpers.rel_err(weight, want_w) < 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,ff", [(32, 48), (20, 28), (256, 512)])
def test_dense_feed_forward_with_relu(dtype, hidden, ff):
    spec = GatedMLPSpec(hidden=hidden, intermediate=ff, activation="relu", names=GatedMLPNames("gate", "up", "down"))
    rt = _rt(dtype)
    cls = FEED_FORWARDS.get(spec.kind)
    w = random_weights(cls.declare(spec, "F."), 2, 0.2, dtype=DT[dtype], device="cuda")
    part = cls(spec, w, "F.", rt)
    for n in (1, 9, 200):
        x = (torch.randn(n, hidden, generator=torch.Generator().manual_seed(n))).to(DT[dtype])
        got = part.forward(x.cuda(), _ctx([0], [0], [n])).sum(0)
        assert _close(got, plain.gated_ff(x.double(), _w64(w), "F.", torch.relu), dtype)


# ----------------------------------------------------------------------------------- norms and embedding, alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [18, 20, 96, 1024, 1028, 2048, 4100])
def test_layer_norm_behind_a_sublayer_and_in_front_of_the_head(dtype, hidden):
    K = _rt(dtype).kernels
    g = torch.Generator().manual_seed(hidden)
    w, b, ls = (torch.randn(hidden, generator=g).cuda() for _ in range(3))
    for n in (3, 70):
        h0 = torch.randn(n, hidden, generator=g).cuda()
        y = (torch.randn(n, hidden, generator=g) * 3.0 + 40.0).cuda()     # a mean far above the spread
        h = h0.clone()
        x = K.post_layernorm(h, y, w, b, ls, 1e-5, cast=True)
        want = h0.double() + ls.double() * plain.layer_norm(y.double(), w.double(), b.double(), 1e-5)
        assert helpers.rel_err(h, want) < 1e-5 and helpers.rel_err(x, want) < (1e-5 if dtype == "float32" else 1e-2)
        h2 = h0.clone()
        K.post_layernorm(h2, y, w, b, None, 1e-5)
        assert helpers.rel_err(h2, h0.double() + plain.layer_norm(y.double(), w.double(), b.double(), 1e-5)) < 1e-5
        rows = torch.tensor([n - 1, 0], dtype=torch.int32).cuda()
        got = K.add_layernorm(y, None, w, b, 1e-5, rows=rows)
        assert helpers.rel_err(got, plain.layer_norm(y.double()[[n - 1, 0]], w.double(), b.double(), 1e-5)) < (1e-4 if dtype == "float32" else 1e-2)
    # a row's bits do not depend on how many rows the step holds
    y = torch.randn(70, hidden, generator=g).cuda()
    a, c = torch.zeros(70, hidden).cuda(), torch.zeros(3, hidden).cuda()
    K.post_layernorm(a, y, w, b, ls, 1e-5)
    K.post_layernorm(c, y[:3].contiguous(), w, b, ls, 1e-5)
    assert torch.equal(a[:3], c)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(53, 5, 11), (7, 1000003, 999983), (1, 3, 4), (300, 0, 1)])
def test_bigram_embedding_across_steps_and_slots(dtype, buckets, mul_prev, mul_cur):
    """Portions cut anywhere, two sequences in a step, a slot used again: the token before a step's first one is the
    sequence's own last token, and a new sequence starts from the table's last row."""
    V, W = 300, 24
    spec = BigramHashSpec(hidden=W, buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur)
    rt = _rt(dtype)
    cls = EMBEDDINGS.get(spec.kind)
    g = torch.Generator().manual_seed(1)
    w = {"embed": torch.randn(V, W, generator=g).to(DT[dtype]).cuda(), "bigram": torch.randn(buckets + 1, W, generator=g).to(DT[dtype]).cuda()}
    part = cls(spec, w, "", rt)
    cache = SequenceCache({-1: cls.cache_need(spec)}, 256, DT[dtype], "cuda:0", max_seqs=2)
    cfg = dict(embedding=dict(bigram=dict(buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur)))
    for trial in range(3):                                             # (slots come back and are taken again)
        seqs = [helpers.rand_ids(40, V, 10 + trial), helpers.rand_ids(23, V, 20 + trial)]
        slots = [cache.alloc_slot(), cache.alloc_slot()]
        at, got = [0, 0], [[], []]
        for step in [(1, 5), (2, 1), (30, 1), (1, 16), (6, 0)]:
            live = [i for i in (0, 1) if step[i]]
            toks = [seqs[i][at[i]:at[i] + step[i]] for i in live]
            h, pending = part.forward(w["embed"], _ctx([slots[i] for i in live], [at[i] for i in live], [step[i] for i in live], toks),
                                      cache.state_of(-1))
            assert helpers.rel_err(pending.x, h) < (1e-7 if dtype == "float32" else 1e-2)
            off = 0
            for i in live:
                got[i].append(h[off:off + step[i]]); off += step[i]; at[i] += step[i]
        for i in (0, 1):
            assert helpers.rel_err(torch.cat(got[i]), plain.embed(seqs[i], _w64(w), cfg)) < 1e-6
            cache.free_slot(slots[i])


# ----------------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def pununex_dirs(tmp_path_factory):
    made = {}

    def get(name, dtype="bfloat16", seed=1, sharp=1.0):
        key = (name, dtype, seed, sharp)
        if key not in made:
            d = str(tmp_path_factory.mktemp(f"pununex-{name}-{dtype}-{seed}"))

            def edit(n, t):            # sharper attention: single far keys carry real weight; decisive routers
                if sharp != 1.0 and n.endswith("q.norm"):
                    return (t.float() * sharp).to(t.dtype)
                if n.endswith("mlp.router"):
                    return (t.float() * 6.0).to(t.dtype)
                return t
            helpers.make_pununex_dir(helpers.PUNUNEX[name](), d, seed=seed, dtype=DT[dtype], edit=edit)
            made[key] = d
        return made[key]
    return get


class RouteTap:
    """Writes down, per routed layer and sequence, the experts the model gave each token and what its router read
    (steps called from Python only: a captured step's choices stay on the device).  In bfloat16 the stream a router
    reads is a few parts in a thousand off the 64-bit one, so a choice may fall another way than in 64-bit, and what
    the token and those behind it then compute is another function.  So the 64-bit witness is given the model's choices
    (``plain.forward(routes=...)``: weights, experts and everything else stay its own), and the choices themselves are
    held against the plain router run on the very rows the model's router read: there they must be the same but for
    ties.  32-bit models are compared with nothing handed over."""

    def __init__(self, lm):
        self.seen, self.layout = {}, None
        for li, b in enumerate(lm.model.blocks):
            ff = getattr(b, "feed_forward", None)
            if ff is not None and hasattr(ff, "route"):
                ff.route = self._wrap(ff.route, li)
        inner = lm.engine.step

        def step(entries, want=None):
            self.layout = [(int(s), len(t)) for s, t in entries]
            return inner(entries, want)
        lm.engine.step = step

    def _wrap(self, inner, li):
        def route(x):
            chosen, weight = inner(x)
            rows, xs, off = chosen.cpu(), x.double().cpu(), 0
            for slot, n in self.layout:
                self.seen.setdefault(slot, {}).setdefault(li, []).append((rows[off:off + n], xs[off:off + n]))
                off += n
            return chosen, weight
        return route

    def routes(self, slot, cfg=None, w=None):
        """{layer: [T, top]} of a sequence, checked against the plain router on the same inputs."""
        out = {}
        for li, parts in self.seen.pop(slot, {}).items():
            chosen, x = torch.cat([p[0] for p in parts]).long(), torch.cat([p[1] for p in parts])
            out[li] = chosen
            if cfg is not None:
                r, p = cfg["layers"][li]["mlp"]["router"], f"l{li}.mlp."
                z = x @ w[p + "router"].T
                own, _ = plain.route(z, w[p + "correction"], r)
                margin = plain.route_margin(z, w[p + "correction"], r)
                off = [t for t in range(x.shape[0]) if sorted(own[t].tolist()) != sorted(chosen[t].tolist())]
                assert all(float(margin[t]) < 2e-3 for t in off), f"layer {li}: tokens {off[:5]} were given other experts than their scores name"
        return out


def _load(d, dtype, **kw):
    """The model and, in bfloat16, the tap on its routers (with steps called from Python)."""
    if dtype == "bfloat16":
        lm = api.load(d, dtype=dtype, use_graph=False, **kw)
        return lm, RouteTap(lm)
    return api.load(d, dtype=dtype, **kw), None


def _close_model(got, want, dtype):
    """Whole models.  32-bit: as everywhere.  bfloat16: row by row.  A layer of this design divides a sublayer's output
    by that output's own spread, and the delta rule divides keys and queries by their own lengths, so a token whose
    vector happens to be short against its rounding is blown up: the 64-bit implementation itself, its input moved by
    2^-9, moves such a row's output by a tenth or more and the typical row's by a few thousandths.  So the worst row in
    twenty is left out of the root mean square, which is held to the type's tolerance, and no row may be lost."""
    if dtype == "float32":
        return _close(got, want, dtype)
    g, w = got.detach().double().cpu(), want.detach().double().cpu()
    rows = (g - w).pow(2).mean(-1) / w.pow(2).mean()
    kept = rows.sort().values[:rows.numel() - max(2, rows.numel() // 20)] if rows.numel() > 4 else rows
    return float(kept.mean().sqrt()) < TOL[dtype] and float(rows.max().sqrt()) < 1.0


def _plain_logits(model_dir, tokens, tap=None, slot=None, layers=None):
    cfg, w = plain.load(model_dir)
    if tap is None:
        return plain.forward(cfg, w, tokens, layers)
    flips = []
    out = plain.forward(cfg, w, tokens, layers, routes=tap.routes(slot, cfg, w), flips=flips)
    assert len(flips) <= max(3, len(tokens) // 4), f"{len(flips)} choices of {len(tokens)} tokens fell another way than in 64-bit"
    return out


def _step_all(lm, slot, tokens, lo, hi):
    return lm.engine.step([(slot, tokens[lo:hi])], [list(range(hi - lo))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "T"])
def test_whole_prompt_and_every_layer_against_plain(pununex_dirs, name, dtype):
    d = pununex_dirs(name, dtype)
    lm, tap = _load(d, dtype, max_tokens=512)
    toks = helpers.rand_ids(150, lm.spec.vocab_size, 5)
    seen = []

    def recording(inner):
        def forward(h, *a, **k):
            out = inner(h, *a, **k)
            seen.append(out[0].clone())                  # (what a post-norm layer hands on adds nothing)
            return out
        return forward
    for b in lm.model.blocks:
        b.forward = recording(b.forward)
    s = lm.engine.open()
    got = _step_all(lm, s, toks, 0, len(toks))
    layers = []
    want = _plain_logits(d, toks, tap, s, layers)
    assert len(seen) == len(layers)
    for i, h in enumerate(seen):
        assert _close_model(h, layers[i], dtype), f"stream after layer {i}"
    assert _close_model(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "T"])
def test_token_by_token_from_the_first_token_equals_the_prompt(pununex_dirs, name, dtype):
    d = pununex_dirs(name, dtype)
    lm, tap = _load(d, dtype, max_tokens=512)
    toks = helpers.rand_ids(110, lm.spec.vocab_size, 9)
    s = lm.engine.open()
    whole = _step_all(lm, s, toks, 0, len(toks))
    assert _close_model(whole, _plain_logits(d, toks, tap, s), dtype)
    lm.engine.close(s)
    s = lm.engine.open()
    one = torch.cat([_step_all(lm, s, toks, i, i + 1) for i in range(len(toks))])
    assert _close_model(one, _plain_logits(d, toks, tap, s), dtype)
    if dtype == "float32":
        assert helpers.rel_err(one, whole) < TOL[dtype] / 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [[2], [3, 2, 64, 1, 2], [63, 2, 1, 1, 64], [64, 65], [1, 128, 2]])
def test_portions_of_several_sizes(pununex_dirs, dtype, sizes):
    d = pununex_dirs("A", dtype, sharp=2.0)
    lm, tap = _load(d, dtype, max_tokens=512)
    toks = helpers.rand_ids(40 if sizes == [2] else 200, lm.spec.vocab_size, 21)
    s = lm.engine.open()
    got = torch.cat([_step_all(lm, s, toks, lo, hi) for lo, hi in _cuts(len(toks), sizes)])
    assert _close_model(got, _plain_logits(d, toks, tap, s), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "T"])
def test_unequal_batch_against_each_alone_with_slots_and_pages_used_again(pununex_dirs, name, dtype):
    """Three requests of unlike lengths start in one step and decode together, the short ones leaving early; then
    the slots and pages they gave back serve other requests, whose state (the recurrences', the filters', the
    embedding's last token) must start from nothing."""
    d = pununex_dirs(name, dtype, sharp=2.0)
    lm, tap = _load(d, dtype, max_tokens=64 * 6, max_seqs=3)
    V = lm.spec.vocab_size
    rounds = [[helpers.rand_ids(n, V, 30 + n) for n in (1, 67, 130)], [helpers.rand_ids(n, V, 50 + n) for n in (129, 3, 64)]]
    extra = [12, 5, 9]
    for reqs in rounds:
        full = [r + helpers.rand_ids(e, V, len(r)) for r, e in zip(reqs, extra)]
        slots = [lm.engine.open() for _ in reqs]
        got = [[] for _ in reqs]
        lg = lm.engine.step([(s, r) for s, r in zip(slots, reqs)], [list(range(len(r))) for r in reqs])
        off = 0
        for i, r in enumerate(reqs):
            got[i].append(lg[off:off + len(r)]); off += len(r)
        for step in range(max(extra)):
            live = [i for i in range(len(reqs)) if step < extra[i]]
            lg = lm.engine.step([(slots[i], [full[i][len(reqs[i]) + step]]) for i in live])
            for row, i in enumerate(live):
                got[i].append(lg[row:row + 1])
            for i in range(len(reqs)):
                if step == extra[i] - 1:
                    lm.engine.close(slots[i])
        for i in range(len(reqs)):
            assert _close_model(torch.cat(got[i]), _plain_logits(d, full[i], tap, slots[i]), dtype), f"request {i}"
    assert lm.engine.cache.pages_held() == 0


def _marked_model(tmp, dtype, window=None, keep_first=0, softcap=None):
    """A one-layer model whose first attention head looks for ONE key.  The stream's first coordinate is -1 for every
    token but token 1 (+1) (the bigram table is zero); the head's query is minus that coordinate and its key plus it,
    so that after the head norms (a query weight of 3) a query of any other token scores +24 on the marked key and
    -24 on every other (capped: +-cap tanh(24 / cap)).  The sink (score 0) therefore holds the weight whenever the
    marked key is out of sight; the delta rule beside the attention is turned down; no feed-forward."""
    layer = helpers.pununex_parallel(heads=2, kv_heads=1, dim=8, vdim=8, scale=1.0, softcap=softcap, window=window,
                                     keep_first=keep_first, r_heads=1, r_kv_heads=1, r_dim=8, r_vdim=8, conv=2, left_scale=1.0,
                                     right_scale=0.05, mlp=None)
    cfg = helpers.pununex_config([layer], vocab=16, width=16, bigram=(5, 1, 2))
    p = "l0.mix.left."

    def edit(n, t):
        if n == "embed":
            t = t.float(); t[:, 0] = -1.0; t[1, 0] = 1.0; return t.to(DT[dtype])
        if n in (p + "q", p + "k"):
            t = torch.zeros_like(t.float()); t[0, 0] = -1.0 if n.endswith("q") else 1.0; return t.to(DT[dtype])
        if n in ("bigram", p + "sink"):
            return torch.zeros_like(t)
        if n == p + "k.norm":
            return torch.ones_like(t)
        if n == p + "q.norm":
            return torch.full_like(t, 3.0)
        return t
    return helpers.make_pununex_dir(cfg, tmp, seed=3, dtype=DT[dtype], edit=edit)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("where", [0, 63, 64, 65, 127, 128, 300])
def test_one_far_key_among_hundreds_in_prompts_and_in_decoding(tmp_path, dtype, where):
    """The marked token sits at a page's first or last place, or far back; every later query finds it (no window), in a
    prompt, across portions and when decoding alone.  Without the mark the logits differ, so a lost key shows."""
    d = _marked_model(str(tmp_path), dtype, softcap=30.0)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    T = 330
    toks = [2 + (i % 13) for i in range(T)]
    toks[where] = 1
    want = _plain_logits(d, toks)
    lost = list(toks); lost[where] = 2
    assert helpers.rel_err(_plain_logits(d, lost)[-1:], want[-1:]) > 0.05        # the key matters to the last query
    s = lm.engine.open()
    portions = _cuts(T, [where + 1, 2, 250])[:3]               # up to the mark, two tokens, up to 250, the rest alone
    got = torch.cat([_step_all(lm, s, toks, lo, hi) for lo, hi in portions]
                    + [_step_all(lm, s, toks, i, i + 1) for i in range(portions[-1][1], T)])
    assert _close(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,where", [(1, 5), (7, 0), (64, 0), (64, 63), (65, 30), (100, 64), (129, 1)])
def test_a_marked_key_just_inside_and_just_outside_the_window(tmp_path, dtype, window, where):
    """The query ``window - 1`` places behind the marked key is the last that sees it; the next one's weight is with
    the sink.  As a prompt, cut into portions at the edge, and decoded token by token across it."""
    d = _marked_model(str(tmp_path), dtype, window=window)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    inside, outside = where + window - 1, where + window
    T = outside + 6
    toks = [2 + (i % 13) for i in range(T)]
    toks[where] = 1
    want = _plain_logits(d, toks)
    if window > 1:                                            # (a window of one key: a token sees itself alone)
        lost = list(toks); lost[where] = 2
        miss = _plain_logits(d, lost)
        assert helpers.rel_err(miss[inside:inside + 1], want[inside:inside + 1]) > 0.05
        assert helpers.rel_err(want[outside:outside + 1], want[inside:inside + 1]) > 0.05
    schedules = [[(0, T)], _cuts(T, [inside, 1, 1, 2]), _cuts(T, [outside, 2]),
                 [(0, max(1, inside - 3))] + [(i, i + 1) for i in range(max(1, inside - 3), T)]]
    for cuts in schedules:
        s = lm.engine.open()
        got = torch.cat([_step_all(lm, s, toks, lo, hi) for lo, hi in cuts])
        lm.engine.close(s)
        assert _close(got, want, dtype), f"cuts {cuts[:4]}"
        assert _close(got[inside:outside + 1], want[inside:outside + 1], dtype), f"edge, cuts {cuts[:4]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,keep", [(5, 1), (5, 3), (20, 32), (7, 33), (64, 64), (65, 65), (3, 70), (40, 130)])
def test_the_last_kept_token_and_the_first_that_is_not(tmp_path, dtype, window, keep):
    """A marked key at place ``keep - 1`` stays seen however far the window has moved on; at place ``keep`` it is lost
    as soon as the window has passed it.  Kept tokens below, at and above a block of 32 keys and a page; as a prompt,
    in portions cut behind the kept tokens and at the window's edge, and decoded one by one."""
    d = _marked_model(str(tmp_path), dtype, window=window, keep_first=keep, softcap=40.0)
    lm = api.load(d, dtype=dtype, max_tokens=1024)
    T = keep + window + 80
    for where in (keep - 1, keep):
        toks = [2 + (i % 13) for i in range(T)]
        toks[where] = 1
        want = _plain_logits(d, toks)
        lost = list(toks); lost[where] = 2
        miss = _plain_logits(d, lost)
        far = helpers.rel_err(miss[-1:], want[-1:])
        assert far > 0.05 if where < keep else far < 1e-9          # the last query sees the one and not the other
        edge = where + window                                       # the first query whose window has passed the mark
        schedules = [[(0, T)], _cuts(T, [keep, 1, window, 2]), _cuts(T, [edge, 1, 1, 40]),
                     [(0, keep + 1)] + [(i, i + 1) for i in range(keep + 1, T)]]
        for cuts in schedules:
            s = lm.engine.open()
            got = torch.cat([_step_all(lm, s, toks, lo, hi) for lo, hi in cuts])
            lm.engine.close(s)
            assert _close(got, want, dtype), f"mark at {where}, cuts {cuts[:4]}"
            assert _close(got[edge - 1:edge + 2], want[edge - 1:edge + 2], dtype), f"mark at {where}, edge, cuts {cuts[:4]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_sequence(pununex_dirs, dtype):
    """Sequences of one, two and three tokens (fewer than a filter's taps; the first token's bigram row), alone and as
    a batch, after the slot held a longer request."""
    d = pununex_dirs("T", dtype)
    lm, tap = _load(d, dtype, max_tokens=256, max_seqs=3)
    V = lm.spec.vocab_size
    s = lm.engine.open()
    lm.engine.step([(s, helpers.rand_ids(90, V, 1))])
    lm.engine.close(s)
    if tap is not None:
        tap.routes(s)
    reqs = [helpers.rand_ids(n, V, 70 + n) for n in (1, 2, 3)]
    slots = [lm.engine.open() for _ in reqs]
    lg = lm.engine.step(list(zip(slots, reqs)), [list(range(len(r))) for r in reqs])
    off = 0
    for r, s in zip(reqs, slots):
        assert _close_model(lg[off:off + len(r)], _plain_logits(d, r, tap, s), dtype)
        off += len(r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,graph", [("A", True), ("A", False), ("T", True)])
def test_long_decoding_of_a_batch(pununex_dirs, name, dtype, graph):
    """200 single-token steps of two sequences (captured graphs or not): state, filters, last tokens and pages carry
    on, and the window passes over decoded tokens while the kept ones stay.  In bfloat16 the steps called from Python
    are held against the plain implementation and the captured ones against those."""
    d = pununex_dirs(name, dtype)
    V = helpers.PUNUNEX[name]()["vocab"]
    full = [helpers.rand_ids(40 + 200, V, 3), helpers.rand_ids(3 + 200, V, 4)]
    starts = [40, 3]

    def run(lm):
        slots = [lm.engine.open(), lm.engine.open()]
        lm.engine.step([(s, f[:n]) for s, f, n in zip(slots, full, starts)])
        rows = [[], []]
        for k in range(200):
            last = lm.engine.step([(s, [f[n + k]]) for s, f, n in zip(slots, full, starts)])
            if k >= 170:
                rows[0].append(last[0:1]); rows[1].append(last[1:2])
        return slots, [torch.cat(r) for r in rows]
    if dtype == "float32":
        lm = api.load(d, dtype=dtype, max_tokens=1024, max_seqs=2, use_graph=graph)
        _, rows = run(lm)
        for row, f in enumerate(full):
            assert _close_model(rows[row], _plain_logits(d, f)[-30:], dtype)
        return
    lm, tap = _load(d, dtype, max_tokens=1024, max_seqs=2)
    slots, rows = run(lm)
    for row, f in enumerate(full):
        assert _close_model(rows[row], _plain_logits(d, f, tap, slots[row])[-30:], dtype)
    if graph:
        _, captured = run(api.load(d, dtype=dtype, max_tokens=1024, max_seqs=2, use_graph=True))
        for row in (0, 1):
            assert helpers.rel_err(captured[row], rows[row]) < 1e-5       # the same kernels on the same numbers


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_drawn_configurations_in_a_batch_and_decoding(tmp_path, seed):
    """Configurations drawn at random (sizes, head counts, windows, kept tokens, caps, filters, layer order, routers):
    a prompt of 200 tokens beside a short one, then six single tokens each, in both types."""
    cfg = helpers.pununex_random_config(seed)
    d = helpers.make_pununex_dir(cfg, str(tmp_path), seed=seed, std=0.08,
                                 edit=lambda n, t: (t.float() * 12.0).to(t.dtype) if n.endswith("mlp.router") else t)
    V = cfg["vocab"]
    a, b = helpers.rand_ids(206, V, seed), helpers.rand_ids(9, V, seed + 100)
    for dtype in ("float32", "bfloat16"):
        lm, tap = _load(d, dtype, max_tokens=512)
        sa, sb = lm.engine.open(), lm.engine.open()
        g = lm.engine.step([(sa, a[:200]), (sb, b[:3])], [list(range(200)), [0, 1, 2]])
        ga, gb = [g[:200]], [g[200:]]
        for k in range(6):
            g = lm.engine.step([(sa, [a[200 + k]]), (sb, [b[3 + k]])])
            ga.append(g[0:1]); gb.append(g[1:2])
        assert _close_model(torch.cat(ga), _plain_logits(d, a, tap, sa), dtype), f"{dtype}: {cfg}"
        assert _close_model(torch.cat(gb), _plain_logits(d, b, tap, sb), dtype), f"{dtype}: {cfg}"
        del lm


def test_greedy_generation_through_the_entry_point(pununex_dirs):
    """``LM.generate`` (scheduler, batching, sampling, captured steps) against greedy decoding with the plain
    implementation, in 32-bit, where a choice of experts cannot fall another way; and bfloat16 generates what its own
    steps called one by one would."""
    d = pununex_dirs("A", "float32")
    lm = api.load(d, dtype="float32", max_tokens=256)
    V = lm.spec.vocab_size
    prompts = [helpers.rand_ids(n, V, 80 + n) for n in (5, 1, 19)]
    toks, _ = lm.generate(prompts, max_new=40)                 # (more new tokens than the windows hold)
    cfg, w = plain.load(d)
    for p, row in zip(prompts, toks.tolist()):
        seq = list(p)
        for t in row:
            lg = plain.forward(cfg, w, seq)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > 1e-3:                # a near tie may fall either way
                assert t == int(lg.argmax())
            seq.append(t)
    d = pununex_dirs("A", "bfloat16")
    lm = api.load(d, dtype="bfloat16", max_tokens=256)
    toks, _ = lm.generate(prompts, max_new=40)
    eager = api.load(d, dtype="bfloat16", max_tokens=256, use_graph=False)
    for p, row in zip(prompts, toks.tolist()):
        s = eager.engine.open()
        lg = eager.engine.step([(s, p)])
        for t in row:
            top2 = torch.topk(lg[0], 2).values
            if float(top2[0] - top2[1]) > 0.05:
                assert t == int(lg[0].argmax())
            lg = eager.engine.step([(s, [t])])


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("T", "bfloat16")])
def test_the_device_side_decode_loop_gives_the_tokens_generation_gives(pununex_dirs, name, dtype):
    """``Engine.decode_session`` (model, greedy pick and feedback in one captured graph): the embedding's bigram row is
    hashed from a token that was chosen on the device one replay earlier and never seen by the host."""
    d = pununex_dirs(name, dtype)
    lm = api.load(d, dtype=dtype, max_tokens=64 * 24, max_seqs=8)
    eng = lm.engine
    prompts = [helpers.rand_ids(n, lm.spec.vocab_size, 500 + n) for n in (5, 61, 30)]
    steps = 70
    toks, _ = lm.generate(prompts, steps)
    assert eng.cache.slots.n_held == 0 and eng.cache.pages_held() == 0
    slots = [eng.open() for _ in prompts]
    first = eng.sample(eng.step(list(zip(slots, prompts))), 0.0, 0, list(range(len(prompts))), [0] * len(prompts))
    assert first == toks[:, 0].tolist()
    sess = eng.decode_session(slots, first, steps - 1)
    sess.run(steps - 1)
    got = sess.tokens()
    sess.finish()
    assert torch.equal(got.T.long(), toks[:, 1:].long()), "the device-side loop chose other tokens than generation"
    if dtype == "float32":                                     # and the sequences go on from where the session left them
        more = eng.step([(s, [int(t)]) for s, t in zip(slots, got[-1])])
        whole = torch.stack([_plain_logits(d, list(p) + toks[i].tolist())[-1] for i, p in enumerate(prompts)])
        assert helpers.rel_err(more, whole) < TOL[dtype]
    for s in slots:
        eng.close(s)


def test_sampling_with_a_temperature_is_the_same_in_any_batch(pununex_dirs):
    """Tokens drawn at temperature 0.8 for a request alone and beside two others: the same (the draw is keyed by seed,
    request and step; the logits do not depend on the batch beyond rounding, which no draw here rests on)."""
    d = pununex_dirs("A", "float32")
    lm = api.load(d, dtype="float32", max_tokens=512)
    V = lm.spec.vocab_size
    prompts = [helpers.rand_ids(n, V, 90 + n) for n in (7, 2, 33)]
    together = lm.generate_requests(prompts, 12, temperature=0.8, seed=5)
    alone = lm.generate_requests(prompts[:1], 12, temperature=0.8, seed=5)
    assert together[0].tokens == alone[0].tokens and len(set(together[0].tokens)) > 3


def test_the_command_line_replays_a_trace(pununex_dirs, tmp_path):
    """``bin/trace_run`` on a Pununex folder: whole, decoded and batched give the plain implementation's logits."""
    import json
    import subprocess
    import sys
    import numpy as np
    d = pununex_dirs("A", "float32")
    V = helpers.PUNUNEX["A"]()["vocab"]
    a, b = helpers.rand_ids(70, V, 1), helpers.rand_ids(9, V, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for k in range(4):
        steps.append({"step": k + 1, "entries": [{"id": "a", "tokens": [a[66 + k]], "want": [0]}, {"id": "b", "tokens": [b[5 + k]], "want": [0] if k == 3 else []}],
                      "end": ["a", "b"] if k == 3 else []})
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]})
    p = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                        "--out", str(tmp_path), "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(6)]
    read = lambda i: torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), f"{i}.f32"), dtype="<f4").reshape(-1, V).copy())
    wa, wb = _plain_logits(d, a), _plain_logits(d, b)
    assert helpers.rel_err(read(0), torch.stack([wa[0], wa[65], wb[4]])) < TOL["float32"]
    assert helpers.rel_err(read(4), torch.stack([wa[69], wb[8]])) < TOL["float32"]
    assert helpers.rel_err(read(5), wb[8:9]) < TOL["float32"]
    assert helpers.rel_err(read(5), read(4)[1:2]) < 1e-5
