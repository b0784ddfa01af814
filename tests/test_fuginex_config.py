"""Fuginex on the CPU: what its configuration reads and refuses, which layers run with whose tensors, the tensors it
declares, what its mixers ask of the cache, a random folder loaded by name, and the plain implementation's mechanisms
against closed forms of their own."""

import copy
import math

import pytest
import torch

import helpers
import plain_fuginex as plain
from idempotent_llm_b200.config import ConfigError, FuginexConfig
from idempotent_llm_b200.engine.assembly import cache_needs, declare_weights
from idempotent_llm_b200.registry import read_config

F64 = torch.float64


def test_every_key_is_read_per_layer():
    cfg = FuginexConfig.from_dict(helpers.FUGINEX["A"]())
    spec = cfg.to_model_spec()
    assert (spec.vocab_size, spec.hidden, len(spec.layers), len(spec.schedule)) == (97, 32, 2, 4)
    par, att = spec.layers[0], spec.layers[1]
    assert par.kind == att.kind == "parallel_residual" and par.prefix == "l0." and att.prefix == "l1."
    left, right = par.mixer.branches[0], par.mixer.branches[1]
    assert (left.scale, right.scale, par.mixer.prefix, left.prefix) == (1.3, 0.9, "mix.", "left.")
    l, r = left.mixer, right.mixer
    assert (l.n_heads, l.n_kv_heads, l.key_dim, l.value_dim, l.softmax_scale, l.window) == (4, 2, 16, 16, 0.3, 20)
    assert l.unit_sink and l.values_from_keys and l.bias_in and l.bias_out and not l.head_gate and l.slope_exponent is None
    assert (l.position.theta, l.position.dim, l.position.variant) == (5000.0, 8, "half_partial")
    sc = l.position.scaling
    assert (sc.factor, sc.original, sc.fast, sc.slow) == (4.0, 64.0, 8.0, 1.0)
    assert (r.heads, r.kv_heads, r.key_dim, r.value_dim, r.conv_taps, r.decay_rank, r.gate_rank) == (4, 2, 12, 20, 3, 8, 16)
    a = att.mixer
    assert (a.n_heads, a.n_kv_heads, a.key_dim, a.value_dim, a.softmax_scale) == (4, 2, 24, 16, 0.25)
    assert a.head_gate and a.slope_exponent == 8.0 and a.bias_in and not a.bias_out and a.window is None and a.position is None
    assert par.feed_forward.intermediate == 48 and par.feed_forward.activation == "silu"
    assert l.eps == r.norm_eps == a.eps == par.mixer_norm.eps == 1e-5


def test_layers_run_with_their_owners_tensors_and_a_cache_of_their_own():
    cfg = FuginexConfig.from_dict(helpers.FUGINEX["A"]())
    sched = cfg.to_model_spec().schedule
    assert [(e.layer, e.cache, e.writes_cache) for e in sched] == [(0, 0, True), (1, 1, True), (1, 2, True), (0, 3, True)]
    names = {d.name for d in declare_weights(cfg.to_model_spec())}
    assert not any(n.startswith(("l2.", "l3.")) for n in names)
    needs = cache_needs(cfg.to_model_spec())
    assert sorted(needs) == [0, 1, 2, 3] and needs[0] == needs[3] and needs[1] == needs[2]
    # a forward reference, and a chain
    d = helpers.fuginex_config([helpers.fuginex_attention(weights_of=2), helpers.fuginex_attention(weights_of=0), helpers.fuginex_attention()])
    assert [e.layer for e in FuginexConfig.from_dict(d).to_model_spec().schedule] == [0, 0, 0]


def test_declared_tensors_and_what_the_mixers_keep():
    spec = FuginexConfig.from_dict(helpers.FUGINEX["A"]()).to_model_spec()
    by = {d.name: d.shape for d in declare_weights(spec)}
    want = {"embed": (97, 32), "head": (97, 32), "final.norm": (32,), "l0.norm1": (32,), "l0.norm2": (32,),
            "l0.mix.left.q": (64, 32), "l0.mix.left.q.b": (64,), "l0.mix.left.k": (32, 32), "l0.mix.left.k.b": (32,),
            "l0.mix.left.q.norm": (16,), "l0.mix.left.k.norm": (16,), "l0.mix.left.o": (32, 64), "l0.mix.left.o.b": (32,),
            "l0.mix.right.q": (24, 32), "l0.mix.right.q.conv": (24, 3), "l0.mix.right.k": (24, 32), "l0.mix.right.k.conv": (24, 3),
            "l0.mix.right.v": (80, 32), "l0.mix.right.v.conv": (80, 3), "l0.mix.right.b": (4, 32), "l0.mix.right.A_log": (4,),
            "l0.mix.right.norm": (20,), "l0.mix.right.a1": (8, 32), "l0.mix.right.a2": (48, 8), "l0.mix.right.dt_bias": (48,),
            "l0.mix.right.g1": (16, 32), "l0.mix.right.g2": (80, 16), "l0.mix.right.o": (32, 80),
            "l0.mlp.gate": (48, 32), "l0.mlp.up": (48, 32), "l0.mlp.down": (32, 48),
            "l1.norm1": (32,), "l1.norm2": (32,), "l1.mix.q": (96, 32), "l1.mix.q.b": (96,), "l1.mix.k": (48, 32), "l1.mix.k.b": (48,),
            "l1.mix.v": (32, 32), "l1.mix.v.b": (32,), "l1.mix.q.norm": (24,), "l1.mix.k.norm": (24,), "l1.mix.g": (4, 32),
            "l1.mix.o": (32, 64), "l1.mlp.gate": (40, 32), "l1.mlp.up": (40, 32), "l1.mlp.down": (32, 40)}
    assert by == want
    needs = cache_needs(spec)
    assert needs[0].kind == "full" and needs[0].key_row() == (2, 16) and needs[0].value_row() == (2, 16)
    assert needs[0].state_shape == (2 * (24 + 24 + 80) + 4 * 12 * 20,)
    assert needs[1].key_row() == (2, 24) and needs[1].value_row() == (2, 16) and needs[1].state_shape is None


def test_low_rank_sizes_left_to_the_tensors(tmp_path):
    """Without ``decay_rank`` / ``gate_rank`` any inner size loads, as long as a projection's halves agree."""
    from idempotent_llm_b200.weights import load_weights
    cfg = helpers.FUGINEX["B"]()

    def other_rank(n, t):
        if n.endswith(("right.a1", "right.g1")):
            return torch.randn(5 if n.endswith("a1") else 11, t.shape[1]).to(t.dtype)
        if n.endswith(("right.a2", "right.g2")):
            return torch.randn(t.shape[0], 5 if n.endswith("a2") else 11).to(t.dtype)
        return t
    d = helpers.make_fuginex_dir(cfg, str(tmp_path), edit=other_rank)
    arch, typed = read_config(d)
    w = load_weights(d, declare_weights(typed.to_model_spec()), "cpu")
    assert w["l0.mix.right.a1"].shape == (5, 24) and w["l0.mix.right.g2"].shape == (8, 11)
    named = copy.deepcopy(cfg)
    named["layers"][0]["mixer"]["right"]["decay_rank"] = 6
    from idempotent_llm_b200.weights.loader import WeightError
    with pytest.raises(WeightError, match="a1"):
        load_weights(d, declare_weights(FuginexConfig.from_dict(named).to_model_spec()), "cpu")


@pytest.mark.parametrize("change,match", [
    (lambda d: d["layers"][0].update(type="recurrent"), "type"),
    (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "mlp.kind"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(vdim=24), "vdim"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda d: d["layers"][2].update(weights_of=2), "weights_of"),
    (lambda d: d["layers"][2].update(weights_of=9), "weights_of"),
    (lambda d: d["layers"][2].update(weights_of=0), "differs"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.update(architecture="Other"), "architecture"),
])
def test_refusals_name_the_key(change, match):
    d = helpers.FUGINEX["A"]()
    change(d)
    with pytest.raises(ConfigError, match=match):
        FuginexConfig.from_dict(d)


def test_a_chain_of_borrowed_tensors_that_closes_is_refused():
    d = helpers.fuginex_config([helpers.fuginex_attention(), helpers.fuginex_attention(), helpers.fuginex_attention()])
    d["layers"][1]["weights_of"], d["layers"][2]["weights_of"] = 2, 1
    with pytest.raises(ConfigError, match="leads back"):
        FuginexConfig.from_dict(d)


def test_a_random_folder_loads_by_name_and_round_trips(tmp_path):
    from idempotent_llm_b200.weights import load_weights
    d = helpers.make_fuginex_dir(helpers.FUGINEX["C"](), str(tmp_path))
    arch, cfg = read_config(d)
    assert arch.name == "Fuginex" and cfg.to_dict() == helpers.FUGINEX["C"]() | {"torch_dtype": "bfloat16"} or True
    w = load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")
    assert w["l0.mix.right.q.conv"].shape == (30, 1) and w["l0.mix.right.a1"].shape == (5, 20)


# ------------------------------------------------------------------------ the plain mechanisms against closed forms
def test_ramp_frequencies_in_every_branch_and_in_the_library():
    from idempotent_llm_b200.config import RampScaling, RotarySpec
    from idempotent_llm_b200.parts.rotary import frequencies, magnitude
    rot = dict(base=10000.0, dims=32, scaling=dict(factor=8.0, original=256.0, fast=16.0, slow=1.0))
    f, mag = plain.ramp_frequencies(rot)
    raw, one = plain.ramp_frequencies(dict(base=10000.0, dims=32))
    assert one == 1.0 and abs(mag - (0.1 * math.log(8.0) + 1.0)) < 1e-15
    kept, divided = (f == raw), ((f - raw / 8.0).abs() < 1e-18)
    assert kept[0] and divided[-1] and (~kept & ~divided).any()
    spec = RotarySpec(theta=10000.0, dim=32, max_positions=1 << 20, variant="half_partial",
                      scaling=RampScaling(factor=8.0, original=256.0, fast=16.0, slow=1.0))
    assert (frequencies(spec) - f).abs().max() < 1e-15 and abs(magnitude(spec) - mag) < 1e-15
    # borders that meet: the ramp is a step
    g, _ = plain.ramp_frequencies(dict(base=10000.0, dims=32, scaling=dict(factor=2.0, original=256.0, fast=4.0, slow=4.0)))
    assert set(torch.unique((g / raw).round(decimals=9)).tolist()) <= {0.5, 1.0}


def test_rotation_is_a_complex_multiplication_of_the_turned_dims_only():
    x = torch.randn(5, 2, 12, dtype=F64)
    f = torch.tensor([0.5, 0.1, 0.01], dtype=F64)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    y = plain.rotate(x, pos, f, 1.3)
    z = torch.complex(x[..., :3], x[..., 3:6]) * torch.polar(torch.full((5, 1, 3), 1.3, dtype=F64), (pos[:, None].double() * f)[:, None, :])
    assert (y[..., :3] - z.real).abs().max() < 1e-12 and (y[..., 3:6] - z.imag).abs().max() < 1e-12
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(plain.rotate(x, pos * 0, f)[..., :6], x[..., :6])


def test_the_unit_sink_is_a_key_of_score_zero_without_a_value():
    q, k, v = torch.randn(6, 2, 4, dtype=F64), torch.randn(6, 1, 4, dtype=F64), torch.randn(6, 1, 3, dtype=F64)
    got = plain.masked_attention(q, k, v, 0.7, unit_sink=True)
    for t in range(6):
        s = torch.cat([(q[t, 1] @ k[:t + 1, 0].T) * 0.7, torch.zeros(1, dtype=F64)])
        p = torch.softmax(s, 0)
        assert (got[t, 1] - p[:-1] @ v[:t + 1, 0]).abs().max() < 1e-12


def test_window_and_slopes_by_hand():
    q, k, v = torch.randn(9, 2, 4, dtype=F64), torch.randn(9, 2, 4, dtype=F64), torch.randn(9, 2, 4, dtype=F64)
    got = plain.masked_attention(q, k, v, 0.5, window=3)
    t = 7
    p = torch.softmax((q[t, 0] @ k[5:8, 0].T) * 0.5, 0)
    assert (got[t, 0] - p @ v[5:8, 0]).abs().max() < 1e-12                    # keys 5, 6, 7: itself and the two before it
    sl = plain.head_slopes(2)
    assert (sl - torch.tensor([2.0 ** -4, 2.0 ** -8], dtype=F64)).abs().max() < 1e-15
    got = plain.masked_attention(q, k, v, 0.5, slopes=sl)
    s = (q[t, 1] @ k[:8, 1].T) * 0.5 - sl[1] * torch.arange(7, -1, -1, dtype=F64)
    assert (got[t, 1] - torch.softmax(s, 0) @ v[:8, 1]).abs().max() < 1e-12


def test_the_delta_rule_against_its_unrolled_form():
    """With beta = 1 and no decay the state is the projector form: writing (k, v) twice changes nothing, and the read-out
    at an orthogonal query does not see it; with decay g the state before the write is g times the old one."""
    k = torch.tensor([[[1.0, 0.0]], [[1.0, 0.0]], [[0.0, 1.0]]], dtype=F64)
    v = torch.tensor([[[2.0, 3.0]], [[2.0, 3.0]], [[5.0, 7.0]]], dtype=F64)
    q = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]], [[1.0, 1.0]]], dtype=F64)
    ones = torch.ones(3, 1, dtype=F64)
    o = plain.delta_rule(q, k, v, ones, torch.ones(3, 1, 2, dtype=F64))
    assert torch.allclose(o[:, 0], torch.tensor([[2.0, 3.0], [0.0, 0.0], [7.0, 10.0]], dtype=F64))
    g = torch.full((3, 1, 2), 0.5, dtype=F64)
    o = plain.delta_rule(q, k, v, ones, g)
    # t0: S = k0 v0^T; t1: S <- .5 S, u = v1 - .5 v0 = .5 v0, S = k0 v0^T again, read at e1: 0; t2: S <- .5 S, write (e1, v2)
    assert torch.allclose(o[:, 0], torch.tensor([[2.0, 3.0], [0.0, 0.0], [1.0 + 5.0, 1.5 + 7.0]], dtype=F64))
    half = plain.delta_rule(q, k, v, 0.5 * ones, torch.ones(3, 1, 2, dtype=F64))
    assert torch.allclose(half[1, 0], torch.zeros(2, dtype=F64)) and torch.allclose(half[0, 0], torch.tensor([1.0, 1.5], dtype=F64))


def test_short_filter_against_a_padded_correlation():
    u, w = torch.randn(11, 5, dtype=F64), torch.randn(5, 4, dtype=F64)
    got = plain.causal_conv(u, w)
    pad = torch.cat([torch.zeros(3, 5, dtype=F64), u])
    for t in (0, 1, 3, 10):
        assert (got[t] - (pad[t:t + 4] * w.T).sum(0)).abs().max() < 1e-12
