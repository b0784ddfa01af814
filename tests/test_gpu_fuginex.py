"""The Fuginex decoder on the GPU against the plain implementation (``plain_fuginex.py``): every mechanism alone,
then whole models through the engine: prompts, token-by-token decoding, portions, unequal batches, slots and pages
used again, marked keys far away, at page borders and at a window's edges, first tokens, long decoding, drawn
configurations, greedy generation, and the trace replay program."""

import os

import pytest
import torch

import helpers
import plain_fuginex as plain
from idempotent_llm_b200 import api
from idempotent_llm_b200.cache import SequenceCache
from idempotent_llm_b200.config import (DeltaRuleSpec, HeadAttentionSpec, MixerBranch, ParallelMixerSpec, RampScaling,
                                        RotarySpec)
from idempotent_llm_b200.engine.batch import context_from_packed, pack_step_host
from idempotent_llm_b200.parts import MIXERS, Runtime
from idempotent_llm_b200.weights import random_weights

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# against the 64-bit plain implementation, relative to the largest value (see test_gpu_lunulix.py for the reasoning)
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
F64 = torch.float64


def _close(got, want, dtype):
    if dtype == "float32":
        return helpers.rel_err(got, want) < TOL[dtype]
    g, w = got.detach().double().cpu(), want.detach().double().cpu()
    rms = float((g - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt())
    return rms < TOL[dtype] and helpers.rel_err(got, want) < 0.25


def _rt(dtype):
    from idempotent_llm_b200.kernels import Kernels
    dev = torch.device("cuda:0")
    return Runtime(device=dev, dtype=DT[dtype], kernels=Kernels(DT[dtype], dev))


def _ctx(slots, starts, lens):
    packed, n, q_lens = pack_step_host(slots, starts, [[0] * L for L in lens])
    return context_from_packed(packed.cuda(), n, slots, q_lens, starts)


def _w64(w):
    return {k: v.double().cpu() for k, v in w.items()}


def _cuts(T, sizes):
    out, lo, i = [], 0, 0
    while lo < T:
        n = sizes[min(i, len(sizes) - 1)]
        out.append((lo, min(T, lo + n)))
        lo, i = lo + n, i + 1
    return out


# ----------------------------------------------------------------------------------- the attention, alone
def _head_spec(**kw):
    base = dict(hidden=40, n_heads=6, n_kv_heads=2, key_dim=24, value_dim=24, softmax_scale=0.3, eps=1e-5)
    base.update(kw)
    return HeadAttentionSpec(**base)


def _plain_head_attention(x, w, s, p):
    """The options of a normed attention one by one, from the plain pieces."""
    T = x.shape[0]
    H, G, d, dv = s.n_heads, s.n_kv_heads, s.key_dim, s.value_dim
    bias = (lambda n: w[p + n + ".b"]) if s.bias_in else (lambda n: 0.0)
    q = (x @ w[p + "q"].T + bias("q")).view(T, H, d)
    k = (x @ w[p + "k"].T + bias("k")).view(T, G, d)
    v = k if s.values_from_keys else (x @ w[p + "v"].T + bias("v")).view(T, G, dv)
    q, k = plain.head_norm(q, w[p + "q.norm"], s.eps), plain.head_norm(k, w[p + "k.norm"], s.eps)
    if s.position is not None:
        rot = dict(base=s.position.theta, dims=s.position.dim)
        sc = s.position.scaling
        if sc is not None:
            rot["scaling"] = dict(factor=sc.factor, original=sc.original, fast=sc.fast, slow=sc.slow)
        f, mag = plain.ramp_frequencies(rot)
        q, k = plain.rotate(q, torch.arange(T), f, mag), plain.rotate(k, torch.arange(T), f, mag)
    slopes = None
    if s.slope_exponent is not None:
        slopes = torch.tensor([2.0 ** (-s.slope_exponent * (h + 1) / H) for h in range(H)], dtype=F64)
    o = plain.masked_attention(q, k, v, s.softmax_scale, window=s.window, unit_sink=s.unit_sink, slopes=slopes)
    if s.head_gate:
        o = o * torch.sigmoid(x @ w[p + "g"].T)[:, :, None]
    o = o.reshape(T, H * dv) @ w[p + "o"].T
    return o + w[p + "o.b"] if s.bias_out else o


HEAD_VARIANTS = {
    # the windowed side of a parallel layer: keys as values, sink, biases, part of the head turned on a ramp
    "windowed": lambda: _head_spec(window=37, unit_sink=True, values_from_keys=True, bias_in=True, bias_out=True,
                                   position=RotarySpec(3e4, 16, 1 << 20, variant="half_partial",
                                                       scaling=RampScaling(4.0, 64.0, 8.0, 1.0))),
    # a window of one page and one key, the whole head turned, no scaling, one kv head
    "window_65": lambda: _head_spec(window=65, unit_sink=True, values_from_keys=True, bias_in=True, bias_out=True, n_kv_heads=1,
                                    position=RotarySpec(1e4, 24, 1 << 20, variant="half_partial")),
    # the attention layer: slopes, a gate per head, values of another size, input biases only
    "slopes": lambda: _head_spec(value_dim=40, slope_exponent=8.0, head_gate=True, bias_in=True),
    # nothing: ordinary softmax attention behind normed heads
    "bare": lambda: _head_spec(n_heads=3, n_kv_heads=3, key_dim=10, value_dim=12),
    # every option at once
    "all": lambda: _head_spec(window=50, unit_sink=True, slope_exponent=4.0, head_gate=True, bias_in=True, bias_out=True,
                              value_dim=8, position=RotarySpec(5e5, 8, 1 << 20, variant="half_partial",
                                                               scaling=RampScaling(2.0, 32.0, 4.0, 4.0))),
    # head sizes the tensor cores have
    "windowed_64": lambda: _head_spec(n_heads=4, n_kv_heads=1, key_dim=64, value_dim=64, softmax_scale=0.15, window=100,
                                      unit_sink=True, values_from_keys=True, bias_in=True, bias_out=True,
                                      position=RotarySpec(3e4, 32, 1 << 20, variant="half_partial")),
    "slopes_128": lambda: _head_spec(n_heads=4, n_kv_heads=2, key_dim=128, value_dim=128, softmax_scale=0.09,
                                     slope_exponent=8.0, head_gate=True, bias_in=True),
    "windowed_128_long": lambda: _head_spec(n_heads=2, n_kv_heads=1, key_dim=128, value_dim=128, softmax_scale=0.09,
                                            window=700, unit_sink=True, values_from_keys=True, bias_in=True, bias_out=True),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", sorted(HEAD_VARIANTS))
def test_normed_attention_alone_prompt_then_single_tokens(dtype, variant):
    spec = HEAD_VARIANTS[variant]()
    rt = _rt(dtype)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "M."), 5, 0.25, dtype=DT[dtype], device="cuda")
    for n in ("M.q.norm", "M.k.norm"):                                # sharper scores than random weights give
        w[n] = (w[n].float() * 1.5).to(DT[dtype])
    part = cls(spec, w, "M.", rt)
    need = cls.cache_need(spec)
    assert need.key_row() == (spec.n_kv_heads, spec.key_dim) and need.value_row() == (spec.n_kv_heads, spec.value_dim)
    T, pre = (1300, 1290) if variant.endswith("long") else (150, 131)
    cache = SequenceCache({0: need}, 64 * 24, DT[dtype], "cuda:0", max_seqs=2)
    slot = cache.alloc_slot()
    x = (torch.randn(T, spec.hidden, generator=torch.Generator().manual_seed(3)) * 1.5).to(DT[dtype])
    ref = _plain_head_attention(x.double(), _w64(w), spec, "M.")
    outs = []
    for lo, hi in [(0, 70), (70, pre)] + [(i, i + 1) for i in range(pre, T)]:
        cache.reserve([(slot, hi)]); cache.flush()
        ctx = _ctx([slot], [lo], [hi - lo])
        outs.append(part.forward(x[lo:hi].contiguous().cuda(), ctx, cache.view(0), cache.state_of(0), True).sum(0))
        cache.set_length(slot, hi)
    assert helpers.rel_err(torch.cat(outs), ref) < TOL[dtype]


TC_SHAPES = {
    # (head size, q-heads, kv-heads, window, slopes): tiles of 16, 64 and 128 tokens; windows below a page, across many
    # runs of key blocks, and wider than the sequence
    "w600_h64_g8": (64, 8, 1, 600, False),
    "w1100_h128_g2": (128, 4, 2, 1100, False),
    "slopes_h128_g1": (128, 2, 2, None, True),
    "w65_slopes_h64_g4": (64, 4, 1, 65, True),
    "w9000_h64_g2": (64, 2, 1, 9000, False),
    "w1_h64_g1": (64, 1, 1, 1, False),
}


@pytest.mark.parametrize("shape", sorted(TC_SHAPES))
def test_windows_and_slopes_on_the_tensor_cores_against_the_general_kernel(shape):
    """bfloat16 with head sizes of 64 and 128 runs on the tensor cores; the general kernel is the witness.  Two unequal
    sequences in the same steps: a long prompt (tiles shared by several blocks, runs of key blocks before the window
    left out), a portion, single tokens (a block per run), with and without the kernel's other ways through scratch."""
    hd, H, G, window, slopes = TC_SHAPES[shape]
    spec = _head_spec(hidden=32, n_heads=H, n_kv_heads=G, key_dim=hd, value_dim=hd, softmax_scale=hd ** -0.5, window=window,
                      unit_sink=window is not None, slope_exponent=6.0 if slopes else None, head_gate=slopes)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "M."), 9, 0.3, dtype=torch.bfloat16, device="cuda")
    w["M.q.norm"] = (w["M.q.norm"].float() * 2.5).to(torch.bfloat16)       # sharp scores: single keys carry weight
    lens = (2900, 1500)
    x = [(torch.randn(n, 32, generator=torch.Generator().manual_seed(3 + n)) * 1.5).to(torch.bfloat16).cuda() for n in lens]
    outs = {}
    for impl, scratch in (("generic", None), ("tcgen05", None), ("tcgen05", True), ("tcgen05", False)):
        rt = _rt("bfloat16")
        rt.kernels.attention_impl = impl
        if scratch is not None:                          # every run a block of its own / no tile shared
            plan = rt.kernels.attention_tc_plan
            rt.kernels.attention_tc_plan = (lambda *a, _p=plan, **k: _p(*a[:4], through_scratch=True)) if scratch else \
                (lambda *a, _p=plan, **k: _p(*a[:4], share=False))
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
        outs[(impl, scratch)] = [torch.cat(g) for g in got]
    want = outs[("generic", None)]
    for key, got in outs.items():
        for i in (0, 1):
            assert helpers.rel_err(got[i], want[i]) < 2e-2, f"{key}, sequence {i}"


def test_the_unit_sink_takes_weight_without_a_value():
    """Scores far below 0 leave the weight with the sink and the output at the output bias; scores far above 0 make it
    ordinary softmax attention."""
    rt = _rt("float32")
    x = torch.randn(9, 16, generator=torch.Generator().manual_seed(1))
    for scale, sink_wins in ((-60.0, True), (60.0, False)):
        spec = _head_spec(hidden=16, n_heads=2, n_kv_heads=1, key_dim=8, value_dim=8, unit_sink=True, softmax_scale=scale,
                          values_from_keys=True, bias_out=True)
        cls = MIXERS.get(spec.kind)
        w = random_weights(cls.declare(spec, "M."), 7, 0.3, dtype=torch.float32, device="cuda")
        w["M.k"] = w["M.q"][:8].clone()                                    # q . k > 0 for head 0 of every token with itself
        w["M.q"] = torch.cat([w["M.k"], w["M.k"]])
        w["M.q.norm"] = w["M.k.norm"] = torch.ones(8, device="cuda")
        part = cls(spec, w, "M.", rt)
        cache = SequenceCache({0: cls.cache_need(spec)}, 64, torch.float32, "cuda:0", max_seqs=1)
        slot = cache.alloc_slot()
        cache.reserve([(slot, 1)]); cache.flush()
        got = part.forward(x[:1].contiguous().cuda(), _ctx([slot], [0], [1]), cache.view(0), None, True).sum(0).cpu()
        v = (x[:1].double() @ w["M.k"].double().cpu().T)                   # one key: itself, its value the key as projected
        want = torch.cat([v, v], dim=1) @ w["M.o"].double().cpu().T * (0.0 if sink_wins else 1.0) + w["M.o.b"].double().cpu()
        assert helpers.rel_err(got, want) < 1e-5


# ----------------------------------------------------------------------------------- the delta rule, alone
def _delta_spec(**kw):
    base = dict(hidden=40, heads=4, kv_heads=2, key_dim=12, value_dim=20, conv_taps=3, norm_eps=1e-5, decay_rank=8, gate_rank=16)
    base.update(kw)
    return DeltaRuleSpec(**base)


def _plain_delta_cfg(s):
    return dict(heads=s.heads, kv_heads=s.kv_heads, dim=s.key_dim, vdim=s.value_dim, conv=s.conv_taps)


DELTA_VARIANTS = {
    "grouped": lambda: _delta_spec(),
    "odd": lambda: _delta_spec(heads=3, kv_heads=3, key_dim=10, value_dim=6, conv_taps=2, decay_rank=5, gate_rank=3),
    "one_tap_one_head": lambda: _delta_spec(heads=1, kv_heads=1, key_dim=8, value_dim=8, conv_taps=1, decay_rank=None, gate_rank=None),
    "wide": lambda: _delta_spec(heads=2, kv_heads=1, key_dim=128, value_dim=64, conv_taps=4, decay_rank=16, gate_rank=24),
    "wider": lambda: _delta_spec(heads=2, kv_heads=2, key_dim=72, value_dim=136, conv_taps=4),
    "widest_keys": lambda: _delta_spec(heads=1, kv_heads=1, key_dim=200, value_dim=24, conv_taps=2),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", sorted(DELTA_VARIANTS))
def test_delta_rule_alone_in_portions(dtype, variant):
    """Portions of 1, 2, 7, 40 and more tokens carry filters and state on; a second slot was taken first, so the state
    is not the first region."""
    spec = DELTA_VARIANTS[variant]()
    rt = _rt(dtype)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "R."), 11, 0.2, dtype=DT[dtype], device="cuda")
    w["R.A_log"] = torch.linspace(-3.0, 0.5, spec.heads, device="cuda").to(DT[dtype])     # slow and fast decays
    part = cls(spec, w, "R.", rt)
    need = cls.cache_need(spec)
    ch = 2 * spec.kv_heads * spec.key_dim + spec.heads * spec.value_dim
    assert need.kind == "none" and need.state_shape == ((spec.conv_taps - 1) * ch + spec.heads * spec.key_dim * spec.value_dim,)
    cache = SequenceCache({0: need}, 64 * 4, DT[dtype], "cuda:0", max_seqs=3)
    cache.alloc_slot()
    slot = cache.alloc_slot()
    T = 420
    x = (torch.randn(T, spec.hidden, generator=torch.Generator().manual_seed(4)) * 1.2).to(DT[dtype])
    ref = plain.delta_mixer(x.double(), _w64(w), "R.", _plain_delta_cfg(spec), spec.norm_eps)
    outs = []
    for lo, hi in _cuts(T, [1, 2, 1, 7, 40, 1, 129, 1, 200, 2, 1]):
        ctx = _ctx([slot], [lo], [hi - lo])
        outs.append(part.forward(x[lo:hi].contiguous().cuda(), ctx, None, cache.state_of(0), True).sum(0))
    assert helpers.rel_err(torch.cat(outs), ref) < TOL[dtype]


def test_the_delta_rule_overwrites_what_a_key_held():
    """The recurrence's kernel alone on hand-made inputs: with beta = 1 and no decay, writing a second value at the same
    unit key replaces the first; a decay of 1/2 halves what an orthogonal key held; the read-out sees the token's own
    write."""
    K = _rt("float32").kernels
    dk, dv = 4, 3
    # columns of c: q [dk] | k [dk] | v [dv]
    e0, e1 = [1.0, 0, 0, 0], [0, 1.0, 0, 0]
    rows = [e0 + e0 + [2.0, 3.0, 4.0],            # write (e0, a), read e0 -> a
            e0 + e1 + [5.0, 6.0, 7.0],            # write (e1, b), read e0 -> a / 2 (decayed once)
            e0 + e0 + [1.0, 1.0, 1.0],            # overwrite e0, read e0 -> (1, 1, 1)
            e1 + e0 + [9.0, 9.0, 9.0]]            # overwrite e0 again, read e1 -> b / 4
    c = torch.tensor(rows, device="cuda")
    g = torch.tensor([[1.0] * dk] + [[0.5] * dk] * 3, device="cuda")
    beta = torch.ones(4, 1, device="cuda")
    state = torch.zeros(2, dk * dv, device="cuda")
    y = K.delta_scan(c, 0, dk, 2 * dk, g, 0, beta, state, _ctx([1], [0], [4]), 1, 1, dk, dv).cpu()
    want = torch.tensor([[2.0, 3.0, 4.0], [1.0, 1.5, 2.0], [1.0, 1.0, 1.0], [1.25, 1.5, 1.75]])
    assert (y - want).abs().max() < 1e-6 and float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("T", [67, 16, 33])
@pytest.mark.parametrize("dk,dv,H,Hk", [(4, 3, 1, 1), (10, 20, 2, 1), (32, 16, 2, 2), (64, 40, 4, 2), (128, 64, 2, 1), (136, 8, 1, 1)])
def test_long_and_short_portions_walk_the_recurrence_to_the_same_numbers(dk, dv, H, Hk, T):
    """Portions of at most four tokens are walked token by token from global memory; longer ones run sixteen tokens
    at a time (keys of up to 128: the sums against the state as products, the corrections from a triangular system)
    or are walked through shared memory (wider keys: the same bits as the short walk).  One portion and portions of
    at most four give the same read-outs and state, and both agree with the recurrence written out.  Some decays are
    so strong that their product over a chunk underflows; some are exactly 1."""
    K = _rt("float32").kernels
    gen = torch.Generator().manual_seed(dk * 131 + dv)
    qk = Hk * dk
    c = torch.randn(T, 2 * qk + H * dv, generator=gen)
    c[:, :2 * qk] = torch.nn.functional.normalize(c[:, :2 * qk].reshape(T, 2 * Hk, dk), dim=-1).reshape(T, -1)
    g = torch.rand(T, H * dk, generator=gen) * 0.5 + 0.5
    g[:, 0] = 1e-6
    g[:, 1] = 1.0
    g[T // 2, :] = 1e-4
    beta = torch.rand(T, H, generator=gen)
    cd, gd, bd = c.cuda(), g.cuda(), beta.cuda()
    got = []
    for sizes in ([T], [4, 3, 1, 2]):
        state = torch.zeros(2, H * dk * dv, device="cuda")
        ys = []
        for lo, hi in _cuts(T, sizes):
            ys.append(K.delta_scan(cd[lo:hi].contiguous(), 0, qk, 2 * qk, gd[lo:hi].contiguous(), 0, bd[lo:hi].contiguous(),
                                   state, _ctx([1], [lo], [hi - lo]), H, Hk, dk, dv))
        got.append((torch.cat(ys).cpu(), state[1].cpu().clone()))
        assert float(state[0].abs().max()) == 0.0
    if dk > 128:
        assert torch.equal(got[0][0], got[1][0]) and torch.equal(got[0][1], got[1][1])
    assert helpers.rel_err(got[0][0], got[1][0]) < 1e-5 and helpers.rel_err(got[0][1], got[1][1]) < 1e-5
    S = torch.zeros(H, dk, dv, dtype=torch.float64)
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            q, k = (c[t, o + (h // (H // Hk)) * dk:][:dk].double() for o in (0, qk))
            v = c[t, 2 * qk + h * dv:][:dv].double()
            S[h] = g[t, h * dk:(h + 1) * dk].double()[:, None] * S[h]
            S[h] = S[h] + torch.outer(k, float(beta[t, h]) * (v - S[h].T @ k))
            want[t, h] = S[h].T @ q
    assert helpers.rel_err(got[0][0].reshape(T, H, dv), want) < 1e-5
    assert helpers.rel_err(got[0][1].reshape(H, dv, dk).transpose(1, 2), S) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parallel_mixer_is_the_weighted_sum_of_its_branches(dtype):
    left = HEAD_VARIANTS["windowed"]()
    right = _delta_spec()
    spec = ParallelMixerSpec(hidden=40, prefix="mix.", branches=(MixerBranch(left, "left.", 0.8), MixerBranch(right, "right.", 1.7)))
    rt = _rt(dtype)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "l0."), 13, 0.25, dtype=DT[dtype], device="cuda")
    part = cls(spec, w, "l0.", rt)
    need = cls.cache_need(spec)
    assert need.kind == "full" and need.state_shape == (2 * (24 + 24 + 80) + 4 * 12 * 20,)
    cache = SequenceCache({0: need}, 64 * 4, DT[dtype], "cuda:0", max_seqs=2)
    slot = cache.alloc_slot()
    T = 90
    x = (torch.randn(T, 40, generator=torch.Generator().manual_seed(8)) * 1.2).to(DT[dtype])
    w64 = _w64(w)
    ref = (0.8 * _plain_head_attention(x.double(), w64, left, "l0.mix.left.")
           + 1.7 * plain.delta_mixer(x.double(), w64, "l0.mix.right.", _plain_delta_cfg(right), 1e-5))
    outs = []
    for lo, hi in _cuts(T, [33, 1, 1, 2, 50, 1]):
        cache.reserve([(slot, hi)]); cache.flush()
        ctx = _ctx([slot], [lo], [hi - lo])
        outs.append(part.forward(x[lo:hi].contiguous().cuda(), ctx, cache.view(0), cache.state_of(0), True).sum(0))
        cache.set_length(slot, hi)
    assert helpers.rel_err(torch.cat(outs), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [18, 20, 96, 1028, 2048, 4096, 4100])
def test_two_norms_of_one_row_in_one_pass(dtype, hidden):
    K = _rt(dtype).kernels
    g = torch.Generator().manual_seed(2)
    h0, d = torch.randn(7, hidden, generator=g), torch.randn(2, 7, hidden, generator=g)
    w1, w2, post = torch.rand(hidden, generator=g) + 0.5, torch.rand(hidden, generator=g) + 0.5, torch.randn(hidden, generator=g)
    for delta, second, bias in ((d, True, True), (None, True, False), (d[:1], False, True)):
        h = h0.clone().cuda()
        x1, x2 = K.add_rmsnorm2(h, None if delta is None else delta.contiguous().cuda(), w1.cuda(), w2.cuda() if second else None,
                                1e-3, post=post.cuda() if bias else None)
        s = h0.double() + (0 if delta is None else delta.double().sum(0))
        tol = 1e-6 if dtype == "float32" else 5e-3
        assert helpers.rel_err(x1, plain.rms_norm(s, w1.double(), 1e-3)) < tol
        assert (x2 is None) if not second else helpers.rel_err(x2, plain.rms_norm(s, w2.double(), 1e-3)) < tol
        assert (h.cpu().double() - (s + (post.double() if bias else 0))).abs().max() < 1e-5


# ------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def fuginex_dirs(tmp_path_factory):
    made = {}

    def get(name, dtype="bfloat16", seed=1, sharp=1.0):
        key = (name, dtype, seed, sharp)
        if key not in made:
            d = str(tmp_path_factory.mktemp(f"fuginex-{name}-{dtype}-{seed}"))

            def edit(n, t):            # sharper attention: single far keys carry real weight
                return (t.float() * sharp).to(t.dtype) if (sharp != 1.0 and n.endswith("q.norm")) else t
            helpers.make_fuginex_dir(helpers.FUGINEX[name](), d, seed=seed, dtype=DT[dtype], edit=edit)
            made[key] = d
        return made[key]
    return get


def _plain_logits(model_dir, tokens):
    cfg, w = helpers.read_model_dir(model_dir)
    return plain.forward(cfg, w, tokens)


def _step_all(lm, slot, tokens, lo, hi):
    return lm.engine.step([(slot, tokens[lo:hi])], [list(range(hi - lo))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "T"])
def test_whole_prompt_and_every_layer_against_plain(fuginex_dirs, name, dtype):
    d = fuginex_dirs(name, dtype)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    cfg, w = helpers.read_model_dir(d)
    toks = helpers.rand_ids(150, cfg["vocab"], 5)
    want, layers = plain.forward(cfg, w, toks, return_layers=True)
    seen = []

    def recording(inner):
        def forward(h, *a, **k):
            out = inner(h, *a, **k)
            after = out[0].clone()
            if out[1] is not None:                   # what the layer's products still owe the stream
                after += out[1].sum(0)
            seen.append(after)
            return out
        return forward
    for b in lm.model.blocks:
        b.forward = recording(b.forward)
    s = lm.engine.open()
    got = _step_all(lm, s, toks, 0, len(toks))
    assert _close(got, want, dtype)
    assert len(seen) == len(cfg["layers"])           # a layer that runs with another's tensors is a run of its own
    for i, h in enumerate(seen):
        assert _close(h, layers[i], dtype), f"stream after layer {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "T"])
def test_token_by_token_from_the_first_token_equals_the_prompt(fuginex_dirs, name, dtype):
    d = fuginex_dirs(name, dtype)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    toks = helpers.rand_ids(110, lm.spec.vocab_size, 9)
    want = _plain_logits(d, toks)
    s = lm.engine.open()
    whole = _step_all(lm, s, toks, 0, len(toks))
    lm.engine.close(s)
    s = lm.engine.open()
    one = torch.cat([_step_all(lm, s, toks, i, i + 1) for i in range(len(toks))])
    assert _close(one, want, dtype) and _close(whole, want, dtype)
    assert helpers.rel_err(one, whole) < (1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [[2], [3, 2, 64, 1, 2], [63, 2, 1, 1, 64], [64, 65], [1, 128, 2]])
def test_portions_of_several_sizes(fuginex_dirs, dtype, sizes):
    d = fuginex_dirs("A", dtype, sharp=2.0)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    toks = helpers.rand_ids(40 if sizes == [2] else 200, lm.spec.vocab_size, 21)
    want = _plain_logits(d, toks)
    s = lm.engine.open()
    got = torch.cat([_step_all(lm, s, toks, lo, hi) for lo, hi in _cuts(len(toks), sizes)])
    assert _close(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "T"])
def test_unequal_batch_against_each_alone_with_slots_and_pages_used_again(fuginex_dirs, name, dtype):
    """Three requests of unlike lengths start in one step and decode together, the short ones leaving early; then
    the slots and pages they gave back serve other requests, whose state must start from nothing."""
    d = fuginex_dirs(name, dtype, sharp=2.0)
    lm = api.load(d, dtype=dtype, max_tokens=64 * 6, max_seqs=3)
    V = lm.spec.vocab_size
    rounds = [[helpers.rand_ids(n, V, 30 + n) for n in (1, 67, 130)], [helpers.rand_ids(n, V, 50 + n) for n in (129, 3, 64)]]
    extra = [12, 5, 9]
    for reqs in rounds:
        full = [r + helpers.rand_ids(e, V, len(r)) for r, e in zip(reqs, extra)]
        want = [_plain_logits(d, f) for f in full]
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
            assert _close(torch.cat(got[i]), want[i], dtype), f"request {i}"
    assert lm.engine.cache.pages_held() == 0


def _marked_model(tmp, dtype, kind, window=None):
    """A one-layer model whose first attention head looks for ONE key.  The embedding's first coordinate is -1 for every
    token but token 1 (+1); the head's query is minus that coordinate and its key plus it, so that after the head norms
    (a query weight of 3) a query of any other token scores +24 on the marked key and -24 on every other.  In a
    ``parallel`` layer the sink (score 0) therefore holds the weight whenever the marked key is out of sight, and the
    value of a key is its first coordinate; the delta rule beside it is turned down."""
    if kind == "parallel":
        layer = helpers.fuginex_parallel(heads=2, kv_heads=1, dim=8, scale=1.0, window=window, rot_dims=0, r_heads=1,
                                         r_kv_heads=1, r_dim=8, r_vdim=8, conv=2, ranks=(8, 8), left_scale=1.0,
                                         right_scale=0.05, ff=None)
        p = "l0.mix.left."
    else:
        layer = helpers.fuginex_attention(heads=2, kv_heads=1, dim=8, vdim=8, scale=1.0, ff=None)
        p = "l0.mix."
    cfg = helpers.fuginex_config([layer], vocab=16, width=16)

    def edit(n, t):
        if n == "embed":
            t = t.float(); t[:, 0] = -1.0; t[1, 0] = 1.0; return t.to(DT[dtype])
        if n in (p + "q", p + "k"):
            t = torch.zeros_like(t.float()); t[0, 0] = -1.0 if n.endswith("q") else 1.0; return t.to(DT[dtype])
        if n in (p + "q.b", p + "k.b"):
            return torch.zeros_like(t)
        if n in ("l0.norm1", p + "k.norm"):
            return torch.ones_like(t)
        if n == p + "q.norm":
            return torch.full_like(t, 3.0)
        return t
    return helpers.make_fuginex_dir(cfg, tmp, seed=3, dtype=DT[dtype], edit=edit)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["parallel", "attention"])
@pytest.mark.parametrize("where", [0, 63, 64, 65, 127, 128, 300])
def test_one_far_key_among_hundreds_in_prompts_and_in_decoding(tmp_path, dtype, kind, where):
    """The marked token sits at a page's first or last place, or far back; every later query finds it (no window; in
    the attention layer the slope times the distance is taken off and the key still stands out), in a prompt, across
    portions and when decoding alone.  Without the mark the logits differ, so a lost key shows."""
    d = _marked_model(str(tmp_path), dtype, kind)
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
    d = _marked_model(str(tmp_path), dtype, "parallel", window=window)
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
def test_the_first_tokens_of_a_sequence(fuginex_dirs, dtype):
    """Sequences of one, two and three tokens (fewer than a filter's taps), alone and as a batch, after the slot
    held a longer request."""
    d = fuginex_dirs("T", dtype)
    lm = api.load(d, dtype=dtype, max_tokens=256, max_seqs=3)
    V = lm.spec.vocab_size
    s = lm.engine.open()
    lm.engine.step([(s, helpers.rand_ids(90, V, 1))])
    lm.engine.close(s)
    reqs = [helpers.rand_ids(n, V, 70 + n) for n in (1, 2, 3)]
    slots = [lm.engine.open() for _ in reqs]
    lg = lm.engine.step(list(zip(slots, reqs)), [list(range(len(r))) for r in reqs])
    off = 0
    for r in reqs:
        assert _close(lg[off:off + len(r)], _plain_logits(d, r), dtype)
        off += len(r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,graph", [("A", True), ("A", False), ("T", True)])
def test_long_decoding_of_a_batch(fuginex_dirs, name, dtype, graph):
    """200 single-token steps of two sequences (captured graphs or not): state, filters and pages carry on, and the
    window passes over decoded tokens."""
    d = fuginex_dirs(name, dtype)
    lm = api.load(d, dtype=dtype, max_tokens=1024, max_seqs=2, use_graph=graph)
    V = lm.spec.vocab_size
    full = [helpers.rand_ids(40 + 200, V, 3), helpers.rand_ids(3 + 200, V, 4)]
    starts = [40, 3]
    slots = [lm.engine.open(), lm.engine.open()]
    lm.engine.step([(s, f[:n]) for s, f, n in zip(slots, full, starts)])
    last = None
    for k in range(200):
        last = lm.engine.step([(s, [f[n + k]]) for s, f, n in zip(slots, full, starts)])
    for row, f in enumerate(full):
        assert _close(last[row:row + 1], _plain_logits(d, f)[-1:], dtype)


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_drawn_configurations_in_a_batch_and_decoding(tmp_path, seed):
    """Configurations drawn at random (sizes, head counts, windows, rotations, filters, layer order and borrowed tensors):
    a prompt of 200 tokens beside a short one, then six single tokens each, in both types."""
    cfg = helpers.fuginex_random_config(seed)
    d = helpers.make_fuginex_dir(cfg, str(tmp_path), seed=seed, std=0.08)
    V = cfg["vocab"]
    a, b = helpers.rand_ids(206, V, seed), helpers.rand_ids(9, V, seed + 100)
    want_a, want_b = _plain_logits(d, a), _plain_logits(d, b)
    for dtype in ("float32", "bfloat16"):
        lm = api.load(d, dtype=dtype, max_tokens=512)
        sa, sb = lm.engine.open(), lm.engine.open()
        g = lm.engine.step([(sa, a[:200]), (sb, b[:3])], [list(range(200)), [0, 1, 2]])
        ga, gb = [g[:200]], [g[200:]]
        for k in range(6):
            g = lm.engine.step([(sa, [a[200 + k]]), (sb, [b[3 + k]])])
            ga.append(g[0:1]); gb.append(g[1:2])
        assert _close(torch.cat(ga), want_a, dtype) and _close(torch.cat(gb), want_b, dtype), f"{dtype}: {cfg}"
        del lm


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(fuginex_dirs, dtype):
    """``LM.generate`` (scheduler, batching, sampling) against greedy decoding with the plain implementation."""
    d = fuginex_dirs("A", dtype)
    lm = api.load(d, dtype=dtype, max_tokens=256)
    V = lm.spec.vocab_size
    prompts = [helpers.rand_ids(n, V, 80 + n) for n in (5, 1, 19)]
    toks, _ = lm.generate(prompts, max_new=24)                 # (more new tokens than the window holds)
    cfg, w = helpers.read_model_dir(d)
    for p, row in zip(prompts, toks.tolist()):
        seq = list(p)
        for t in row:
            lg = plain.forward(cfg, w, seq)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > (1e-3 if dtype == "float32" else 0.1):      # a near tie may fall either way
                assert t == int(lg.argmax())
            seq.append(t)


def test_the_command_line_replays_a_trace(fuginex_dirs, tmp_path):
    """``bin/trace_run`` on a Fuginex folder: whole, decoded and batched give the plain implementation's logits."""
    import json
    import subprocess
    import sys
    import numpy as np
    d = fuginex_dirs("A", "float32")
    V = helpers.FUGINEX["A"]()["vocab"]
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
