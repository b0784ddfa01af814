"""Pununex on the CPU: its configuration (every key read per layer, absent options, refusals by key), the tensors
it declares, what its parts ask of the cache, a random folder loaded by name, and the plain implementation's
mechanisms against closed forms of their own."""

import math

import pytest
import torch

import helpers
import plain_pununex as plain
from idempotent_llm_b200.config import (BigramHashSpec, ConfigError, DeltaRuleSpec, GatedMLPSpec, HeadAttentionSpec,
                                        LayerNormSpec, ParallelMixerSpec, PostNormLayerSpec, PununexConfig, RoutedExpertsSpec)
from idempotent_llm_b200.engine.assembly import EMBEDDING_CACHE_ID, cache_needs, declare_weights
from idempotent_llm_b200.registry import read_config, registered_architectures

F64 = torch.float64


# ----------------------------------------------------------------------------------- configuration
def test_every_key_is_read_per_layer():
    cfg = PununexConfig.from_dict(helpers.PUNUNEX["A"]())
    spec = cfg.to_model_spec()
    assert "Pununex" in registered_architectures()
    assert isinstance(spec.embedding, BigramHashSpec) and (spec.embedding.buckets, spec.embedding.mul_prev, spec.embedding.mul_cur) == (53, 5, 11)
    assert isinstance(spec.final_norm, LayerNormSpec) and not spec.tie_embeddings
    kinds = [type(L.mixer) for L in spec.layers]
    assert kinds == [DeltaRuleSpec, ParallelMixerSpec, ParallelMixerSpec, DeltaRuleSpec]
    assert all(isinstance(L, PostNormLayerSpec) and L.mixer_scale == "ls1" for L in spec.layers)
    d0 = spec.layers[0].mixer
    assert (d0.heads, d0.kv_heads, d0.key_dim, d0.value_dim, d0.conv_taps, d0.decay, d0.gate) == (4, 2, 16, 24, 3, "head", "silu")
    left, right = (b.mixer for b in spec.layers[1].mixer.branches)
    assert isinstance(left, HeadAttentionSpec) and (left.n_heads, left.n_kv_heads, left.key_dim, left.value_dim) == (4, 2, 24, 16)
    assert (left.softmax_scale, left.softcap, left.window, left.keep_first, left.sink, left.unit_sink, left.position) == (0.25, 10.0, 20, 3, True, False, None)
    assert (right.decay, right.gate, right.key_dim, right.value_dim, right.conv_taps) == ("channel", "sigmoid_low_rank", 12, 20, 4)
    assert [b.scale for b in spec.layers[1].mixer.branches] == [1.3, 0.6]
    assert (spec.layers[2].mixer.branches[0].mixer.window, spec.layers[2].mixer.branches[0].mixer.keep_first) == (33, 1)
    ff0, ff1 = spec.layers[0].feed_forward, spec.layers[1].feed_forward
    assert isinstance(ff0, GatedMLPSpec) and ff0.activation == "relu" and ff0.intermediate == 48
    assert isinstance(ff1, RoutedExpertsSpec)
    assert (ff1.n_experts, ff1.n_identity, ff1.top, ff1.groups, ff1.groups_keep, ff1.scale, ff1.intermediate) == (6, 2, 3, 4, 2, 1.5, 24)
    assert ff1.shared.intermediate == 40 and ff1.shared.activation == "silu" and ff1.activation == "silu"


def test_absent_options():
    spec = PununexConfig.from_dict(helpers.PUNUNEX["B"]()).to_model_spec()
    assert spec.embedding is None
    left = spec.layers[0].mixer.branches[0].mixer
    assert left.softcap is None and left.window is None and left.keep_first == 0
    ff = spec.layers[0].feed_forward
    assert (ff.n_identity, ff.groups, ff.groups_keep, ff.top, ff.shared) == (0, 1, 1, 1, None)
    assert spec.layers[1].feed_forward is None and spec.layers[1].feed_forward_post_norm is None
    names = {d.name for d in declare_weights(spec)}
    assert "bigram" not in names and "l1.norm2" not in names and "l1.ls2" not in names and "l1.ls1" in names
    assert EMBEDDING_CACHE_ID not in cache_needs(spec)


def test_declared_tensors_and_state():
    spec = PununexConfig.from_dict(helpers.PUNUNEX["A"]()).to_model_spec()
    decl = {d.name: d for d in declare_weights(spec)}
    assert decl["bigram"].shape == (54, 32) and decl["final.norm.b"].shape == (32,) and decl["head"].shape == (97, 32)
    for n, shape in {"l0.mix.q": (32, 32), "l0.mix.v.conv": (96, 3), "l0.mix.a": (4, 32), "l0.mix.dt_bias": (4,), "l0.mix.g": (96, 32),
                     "l0.mix.o": (32, 96), "l0.mlp.gate": (48, 32), "l0.ls2": (32,), "l0.norm1.b": (32,),
                     "l1.mix.left.q": (96, 32), "l1.mix.left.k": (48, 32), "l1.mix.left.v": (32, 32), "l1.mix.left.q.norm": (24,),
                     "l1.mix.left.sink": (4,), "l1.mix.left.o": (32, 64), "l1.mix.right.dt_bias": (24,), "l1.mix.right.a2": (24, -1),
                     "l1.mix.right.g2": (40, -1), "l1.mlp.router": (8, 32), "l1.mlp.correction": (8,), "l1.mlp.e5.down": (32, 24),
                     "l1.mlp.shared.up": (40, 32)}.items():
        assert decl[n].shape == shape, n
    assert "l1.mlp.e6.gate" not in decl and "l0.mix.a1" not in decl and "l1.mix.right.a" not in decl
    needs = cache_needs(spec)
    assert needs[EMBEDDING_CACHE_ID].state_shape == (1,) and needs[EMBEDDING_CACHE_ID].state_dtype == torch.int32
    assert needs[0].kind == "none" and needs[0].state_shape == (2 * (32 + 32 + 96) + 4 * 16 * 24,)
    assert needs[1].kind == "full" and needs[1].key_row() == (2, 24) and needs[1].value_row() == (2, 16)
    assert needs[1].state_shape == (3 * (12 + 12 + 40) + 2 * 12 * 20,)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("dim"), "dim"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(softcap=-1.0), "softcap"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "chosen"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=1), "groups"),      # three experts from one group of two
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["embedding"]["bigram"].pop("buckets"), "buckets"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "empty"),
])
def test_refusals_by_key(edit, word):
    cfg = helpers.PUNUNEX["A"]()
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        PununexConfig.from_dict(cfg)
    assert word in str(e.value)


def test_random_folder_round_trip(tmp_path):
    from idempotent_llm_b200.weights import load_weights
    cfg = helpers.PUNUNEX["C"]()
    d = helpers.make_pununex_dir(cfg, str(tmp_path), seed=4)
    arch, typed = read_config(d)
    assert arch.name == "Pununex" and typed.to_dict()["layers"] == cfg["layers"]
    w = load_weights(d, declare_weights(typed.to_model_spec()), "cpu")
    assert w["l0.mix.right.a1"].shape[1] == 20 and w["l0.mix.right.a2"].shape[1] == w["l0.mix.right.a1"].shape[0]
    c2, w2 = plain.load(d)
    assert c2 == typed.to_dict() or c2["layers"] == cfg["layers"]
    assert torch.equal(w2["head"], w["head"].double())


# ----------------------------------------------------------------------------------- plain mechanisms, by hand
def test_bigram_rows_by_hand():
    assert plain.bigram_rows([4, 9, 2], 10, 3, 7) == [10, (4 * 3 + 9 * 7) % 10, (9 * 3 + 2 * 7) % 10]
    assert plain.bigram_rows([5], 7, 1, 1) == [7]
    big = plain.bigram_rows([2 ** 20, 2 ** 20 + 1], 2003, 1000003, 999983)
    assert big[1] == (2 ** 20 * 1000003 + (2 ** 20 + 1) * 999983) % 2003


def test_layer_norm_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=F64)
    w, b = torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=F64), torch.tensor([0.0, 1.0, 0.0, -1.0], dtype=F64)
    var = (4 + 1 + 0 + 9) / 4
    want = (x - 3.0) / math.sqrt(var + 0.5) * w + b
    assert torch.allclose(plain.layer_norm(x, w, b, 0.5), want, atol=1e-14)


def test_seen_mask_window_and_kept_tokens():
    m = plain.seen_mask(12, 3, 2)
    assert m[11].tolist() == [True, True] + [False] * 7 + [True] * 3
    assert m[3].tolist() == [True, True, True, True] + [False] * 8          # 0 and 1 kept, 1..3 in the window
    assert m[4].tolist() == [True, True, True, True, True] + [False] * 7 and not plain.seen_mask(12, 3, 0)[4, 1]
    assert plain.seen_mask(5, None, 0).tolist() == torch.tril(torch.ones(5, 5)).bool().tolist()


def test_the_sink_is_a_key_without_a_value_and_the_cap_bounds_scores():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(9, 2, 4, generator=g, dtype=F64) * 3 for _ in range(3))
    sink = torch.tensor([0.7, -1.1], dtype=F64)
    got = plain.capped_sink_attention(q, k, v, 0.9, 2.5, 4, 1, sink)
    for h in range(2):
        for t in range(9):
            js = [j for j in range(t + 1) if t - j < 4 or j < 1]
            s = torch.stack([2.5 * torch.tanh(0.9 * (q[t, h] @ k[j, h]) / 2.5) for j in js] + [sink[h]])
            assert float(s[:-1].abs().max()) <= 2.5
            a = torch.softmax(s, 0)
            want = sum(a[i] * v[j, h] for i, j in enumerate(js))              # the sink's share goes nowhere
            assert torch.allclose(got[t, h], want, atol=1e-12)


def test_delta_recurrence_against_its_unrolled_form():
    g = torch.Generator().manual_seed(2)
    T, dk, dv = 6, 3, 2
    q, k = torch.randn(T, 1, dk, generator=g, dtype=F64), torch.randn(T, 1, dk, generator=g, dtype=F64)
    v, beta = torch.randn(T, 2, dv, generator=g, dtype=F64), torch.rand(T, 2, generator=g, dtype=F64)
    dec = torch.rand(T, 2, dk, generator=g, dtype=F64)
    got = plain.delta_recurrence(q, k, v, beta, dec)
    for h in range(2):
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            # S_t = (I - beta k k^T) diag(g) S_(t-1) + beta k v^T
            S = (torch.eye(dk, dtype=F64) - beta[t, h] * torch.outer(k[t, 0], k[t, 0])) @ (dec[t, h][:, None] * S) \
                + beta[t, h] * torch.outer(k[t, 0], v[t, h])
            assert torch.allclose(got[t, h], S.T @ q[t, 0], atol=1e-12)


def test_route_by_hand():
    # four groups of two; choice scores are softmax + correction; groups 1 and 3 are the best two
    z = torch.log(torch.tensor([[0.05, 0.05, 0.30, 0.10, 0.05, 0.05, 0.25, 0.15]], dtype=F64))
    corr = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.19, 0.0, 0.0, 0.0], dtype=F64)     # expert 4 would be third, but its group loses
    r = dict(top=3, scale=2.0, groups=dict(count=4, keep=2))
    chosen, weights = plain.route(z, corr, r)
    assert chosen.tolist() == [[2, 6, 7]]
    s = torch.tensor([0.30, 0.25, 0.15], dtype=F64)
    assert torch.allclose(weights[0], s / s.sum() * 2.0, atol=1e-12)          # weights from the scores WITHOUT the correction
    # shut-out experts count as minus infinity, not as zero: with negative choice scores the kept group still wins
    corr = torch.full((8,), -5.0, dtype=F64)
    chosen, _ = plain.route(z, corr, dict(top=2, scale=1.0, groups=dict(count=4, keep=1)))
    assert chosen.tolist() == [[2, 3]]
    # no groups: the plain top
    chosen, _ = plain.route(z, torch.zeros(8, dtype=F64), dict(top=2, scale=1.0))
    assert chosen.tolist() == [[2, 6]]


def test_identity_experts_and_the_shared_expert():
    g = torch.Generator().manual_seed(3)
    W, E = 6, 3
    c = dict(kind="moe", expert=dict(ff=4), router=dict(experts=E, identity=1, top=2, scale=1.0), shared=dict(ff=5))
    w = {"router": torch.randn(E + 1, W, generator=g, dtype=F64), "correction": torch.zeros(E + 1, dtype=F64)}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (torch.randn(*s, generator=g, dtype=F64) for s in ((4, W), (4, W), (W, 4)))
    w["shared.gate"], w["shared.up"], w["shared.down"] = (torch.randn(*s, generator=g, dtype=F64) for s in ((5, W), (5, W), (W, 5)))
    w["router"][E] += 50.0 * torch.ones(W, dtype=F64)                          # the identity expert wins wherever sum(h) > 0
    h = torch.rand(4, W, generator=g, dtype=F64) + 0.1
    out = plain.routed_ff(h, w, "", c)
    chosen, weights = plain.route(h @ w["router"].T, w["correction"], c["router"])
    for t in range(4):
        assert chosen[t, 0] == E
        other = int(chosen[t, 1])
        want = weights[t, 0] * h[t] + weights[t, 1] * plain.gated_ff(h[t:t + 1], w, f"e{other}.", plain.silu)[0] \
            + plain.gated_ff(h[t:t + 1], w, "shared.", plain.silu)[0]
        assert torch.allclose(out[t], want, atol=1e-12)
