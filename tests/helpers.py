"""Small configurations and utilities of the tests."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", attention_bias=False, hidden_act="silu")

# Tiny configurations that differ in every size and option: head counts and groups, sizes that
# are no power of two, layers, vocabulary, eps, theta, tied or not, window.
TINY = {
    # BASELINE "Tiny Qwen3 A"
    "A": dict(_BASE, num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=2048, eos_token_id=255, initializer_range=0.02),
    # BASELINE "Tiny Qwen3 B", plus a window of 80 keys on layers >= 1
    "B": dict(_BASE, num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=3,
              head_dim=32, intermediate_size=224, vocab_size=320, rope_theta=1000000.0, rms_norm_eps=1e-5,
              tie_word_embeddings=False, max_position_embeddings=4096, eos_token_id=[318, 319],
              initializer_range=0.05, use_sliding_window=True, sliding_window=80, max_window_layers=1),
    # head_dim 128 (the benchmark's head size), group of 4, odd vocabulary and widths
    "C": dict(_BASE, num_hidden_layers=2, hidden_size=160, num_attention_heads=8, num_key_value_heads=2,
              head_dim=128, intermediate_size=288, vocab_size=1000, rope_theta=500000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=8192, eos_token_id=999, initializer_range=0.04),
    # head_dim 48 (a multiple of 16 that is no power of two), no grouping, prime-ish sizes
    "D": dict(_BASE, num_hidden_layers=1, hidden_size=80, num_attention_heads=5, num_key_value_heads=5,
              head_dim=48, intermediate_size=136, vocab_size=131, rope_theta=20000.0, rms_norm_eps=1e-4,
              tie_word_embeddings=False, max_position_embeddings=1024, initializer_range=0.05),
}


def make_model_dir(cfg: dict, out_dir: str, seed: int = 1, dtype=torch.bfloat16, sharp: float = 1.0) -> str:
    """A model folder with seeded random weights.  ``sharp`` > 1 scales every q_norm weight, which
    sharpens attention so that single far keys carry real weight (random weights alone give
    near-uniform attention, which hides a dropped or misplaced key)."""
    from idempotent_llm_b200.config import Qwen3Config
    from idempotent_llm_b200.weights import write_random_model, write_safetensors, SafetensorsFile
    write_random_model(Qwen3Config.from_dict(cfg), out_dir, seed=seed, dtype=dtype)
    if sharp != 1.0:
        path = os.path.join(out_dir, "model.safetensors")
        f = SafetensorsFile(path)
        tensors = []
        for n in f.names():
            t = f.get(n).clone()
            if n.endswith("q_norm.weight"):
                t = (t.float() * sharp).to(t.dtype)
            tensors.append((n, t))
        del f
        write_safetensors(path, tensors)
    return out_dir


def rand_ids(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


# Tolerances against the 64-bit plain implementation, fixed before any measurement:
# 32-bit arithmetic with sums of a few hundred terms; bfloat16 rounds activations (8 bits of
# mantissa) a handful of times per layer.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def run_trace(model_dir: str, dtype: str, steps: list, out_dir: str, max_tokens: int, timeout: int = 600,
              extra=()):
    """Run bin/trace_run on a list of step records; returns {step: tensor [wanted, vocab]}."""
    import numpy as np
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    inp = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype",
                        dtype, "--out", out_dir, "--max-tokens", str(max_tokens), *extra],
                       input=inp, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, f"trace_run failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}"
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [l.split()[1] for l in done] == [str(s["step"]) for s in steps], p.stdout[-2000:]
    out = {}
    for s in steps:
        n = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if n:
            out[s["step"]] = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(n, vocab).copy())
        else:
            assert not os.path.exists(path)
    return out


# ------------------------------------------------------------------------------------- Lunulix
def lunulix_layer(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, lconv=3, rot_dims=8, rot_base=5000.0,
                  scaling=(4.0, 1.0, 4.0, 64), r_heads=3, r_vdim=8, state=12, groups=1, rconv=4, norm_groups=2,
                  left_scale=0.7, right_scale=1.3, ff=40):
    """One layer of a Lunulix config.json; every size and constant is an argument."""
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if lconv:
        left["conv"] = lconv
    if rot_dims:
        left["rot"] = dict(base=rot_base, dims=rot_dims)
        if scaling:
            left["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    right = dict(heads=r_heads, vdim=r_vdim, state=state, groups=groups, conv=rconv, norm_groups=norm_groups)
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale),
                mlp=None if not ff else dict(kind="dense", ff=ff))


def lunulix_config(layers, vocab=97, width=32, emb_scale=3.0, eps=1e-5, side_dim=8):
    d = dict(architecture="Lunulix", vocab=vocab, width=width, embedding=dict(scale=emb_scale), norm=dict(eps=eps),
             layers=list(layers))
    if side_dim:
        d["token_side"] = dict(dim=side_dim)
    return d


# Small Lunulix models that differ from one another in every size and option.
LUNULIX = {
    # two unlike layers: grouped heads with key and value rows of different widths, a partial rotation with scaled
    # frequencies, filters of 3 and 4 taps; then a layer without feed-forward, whole-head rotation without scaling,
    # other filters, one norm part, state size no multiple of 4
    "P": lambda: lunulix_config([
        lunulix_layer(),
        lunulix_layer(heads=2, kv_heads=2, dim=24, vdim=16, scale=0.2, lconv=2, rot_dims=24, scaling=None, r_heads=4,
                      r_vdim=12, state=10, groups=2, rconv=3, norm_groups=1, left_scale=1.0, right_scale=0.5, ff=None)]),
    # no token side input, no embedding scale, no filter and no rotation on the attention side, one kv-head,
    # norm parts that cut through heads (3 heads of 8 in 4 parts of 6)
    "Q": lambda: lunulix_config([
        lunulix_layer(heads=3, kv_heads=1, dim=8, vdim=8, lconv=0, rot_dims=0, r_heads=3, r_vdim=8, state=16, groups=3,
                      rconv=2, norm_groups=4, ff=24)], vocab=50, width=24, emb_scale=1.0, side_dim=0),
    # widths that are no multiple of 8 (bfloat16 rows off the 16-byte borders): products with padded operands, keys
    # read element by element, the feed-forward's activation as a kernel of its own
    "S": lambda: lunulix_config([
        lunulix_layer(heads=3, kv_heads=1, dim=12, vdim=10, scale=0.3, rot_dims=6, r_heads=2, r_vdim=6, state=6, groups=1,
                      rconv=3, norm_groups=3, ff=28)] * 2, vocab=33, width=20, emb_scale=2.0, side_dim=4),
    # head sizes the tensor-core attention has (64), three layers, width 64
    "R": lambda: lunulix_config([lunulix_layer(heads=6, kv_heads=2, dim=64, vdim=64, scale=0.11, rot_dims=48,
                                               r_heads=2, r_vdim=32, state=32, groups=1, ff=96)] * 3,
                                vocab=211, width=64, emb_scale=8.0, side_dim=24),
}


def lunulix_random_config(seed: int) -> dict:
    """A Lunulix configuration drawn from sizes a model of the design may have: one to three unlike layers, grouped
    and ungrouped heads, key and value widths that differ or not (64 and 128 among them: the tensor-core attention),
    rotation of none, part or all of a head with or without scaling, filters of 0 to 4 taps, state sizes of 16 to 256,
    norm parts, layers without feed-forward, with or without the token side input."""
    import random
    r = random.Random(seed)

    def layer():
        kv = r.choice([1, 2, 4]); heads = kv * r.choice([1, 2, 3, 4])
        dim = r.choice([32, 48, 64, 64, 128, 96]); vdim = r.choice([dim, dim, 32, 64, 80])
        rot = r.choice([0, dim // 2, dim, 16])
        scaling = r.choice([None, (8.0, 1.0, 4.0, 2048), (2.0, 0.5, 8.0, 512), (32.0, 1.0, 4.0, 64)])
        r_heads = r.choice([2, 4, 6, 8]); groups = r.choice([g for g in (1, 2, r_heads) if r_heads % g == 0])
        r_vdim = r.choice([16, 32, 48, 64, 128]); state = r.choice([16, 32, 48, 64, 128, 256])
        parts = r.choice([g for g in (1, 2, 4, r_heads, 8) if (r_heads * r_vdim) % g == 0])
        return lunulix_layer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=r.choice([dim ** -0.5, 0.1, 0.05]),
                             lconv=r.choice([0, 2, 3, 4]), rot_dims=rot, rot_base=r.choice([1e4, 2.5e5, 1e6]),
                             scaling=scaling if rot else None, r_heads=r_heads, r_vdim=r_vdim, state=state, groups=groups,
                             rconv=r.choice([2, 3, 4]), norm_groups=parts, left_scale=r.choice([1.0, 0.6, 0.3]),
                             right_scale=r.choice([1.0, 0.9, 1.5]), ff=r.choice([None, 64, 160, 256]))
    width = r.choice([64, 96, 128, 256, 320])
    return lunulix_config([layer() for _ in range(r.choice([1, 2, 3]))], vocab=r.choice([128, 500, 1000]), width=width,
                          emb_scale=r.choice([1.0, 4.0, 16.0]), eps=r.choice([1e-5, 1e-6]), side_dim=r.choice([0, 8, 16, 32]))


def make_lunulix_dir(cfg: dict, out_dir: str, seed: int = 1, dtype=torch.bfloat16, std: float = 0.15, edit=None) -> str:
    """A Lunulix model folder with seeded random weights; ``edit(name, tensor) -> tensor`` may change them."""
    from idempotent_llm_b200.config import LunulixConfig
    from idempotent_llm_b200.weights import write_random_model, write_safetensors, SafetensorsFile
    write_random_model(LunulixConfig.from_dict(cfg), out_dir, seed=seed, dtype=dtype, std=std)
    if edit is not None:
        path = os.path.join(out_dir, "model.safetensors")
        f = SafetensorsFile(path)
        tensors = [(n, edit(n, f.get(n).clone())) for n in f.names()]
        del f
        write_safetensors(path, tensors)
    return out_dir


def read_lunulix(model_dir: str):
    """(config dict, tensors by name) read without the package (for the plain implementation)."""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(model_dir, "model.safetensors"))


# ------------------------------------------------------------------------------------- Panodra
def panodra_layer(sink=False, heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.2, rot_base=3e4, scaling=None,
                  mlp="dense", ff=72, experts=5, top=3):
    """One layer of a Panodra config.json; every size and constant is an argument.  ``scaling``: (factor, original,
    fast, slow) or None; ``mlp``: "dense", "moe" or None."""
    rot = dict(base=rot_base, dims=rot_dim)
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = None
    if mlp == "dense":
        m = dict(kind="dense", ff=ff)
    elif mlp == "moe":
        m = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    return dict(type="latent_attention" if sink else "latent_attention_2",
                mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale, rot=rot), mlp=m)


def panodra_config(layers, vocab=97, width=64, eps=1e-5, loop=None, logit_scale=0.7, softcap=12.0):
    d = dict(architecture="Panodra", vocab=vocab, width=width, norm=dict(eps=eps), layers=list(layers))
    if loop:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    if logit_scale is not None:
        d["logit_scale"] = logit_scale
    if softcap is not None:
        d["logit_softcap"] = softcap
    return d


# Small Panodra models that differ from one another in every size and option.
PANODRA = {
    # three unlike layers, the last two run three times: no sink / dense, sink + scaled frequencies / experts 3 of 5,
    # sink / no feed-forward
    "A": lambda: panodra_config([
        panodra_layer(),
        panodra_layer(sink=True, heads=2, dim=8, rot_dim=16, vdim=8, kv_rank=24, scale=0.35, rot_base=1e4,
                      scaling=(8.0, 64, 8.0, 1.0), mlp="moe", ff=24, experts=5, top=3),
        panodra_layer(sink=True, heads=4, dim=24, rot_dim=8, vdim=16, kv_rank=32, scale=0.15, mlp=None)], loop=(1, 3, 3)),
    # values of 1 and absent keys: one head, one expert of which a token uses one, no loop, no constant, no cap
    "B": lambda: panodra_config([panodra_layer(heads=1, dim=8, rot_dim=8, vdim=8, kv_rank=16, mlp="moe", ff=16, experts=1, top=1)],
                                vocab=50, width=24, loop=None, logit_scale=None, softcap=None),
    # widths that are no multiple of 8 (bfloat16 rows off the 16-byte borders), a loop of one layer over the first
    "C": lambda: panodra_config([
        panodra_layer(sink=True, heads=3, dim=12, rot_dim=6, vdim=10, kv_rank=12, scale=0.3, ff=28),
        panodra_layer(heads=2, dim=6, rot_dim=4, vdim=6, kv_rank=10, scale=0.4, mlp="moe", ff=12, experts=3, top=2)],
        vocab=33, width=20, loop=(0, 1, 2), logit_scale=1.3, softcap=5.0),
    # head sizes the tensor-core attention takes whole prompts at (64 and 128 with the heads padded), experts that
    # run grouped by expert from 128 tokens on
    "T": lambda: panodra_config([
        panodra_layer(heads=4, dim=32, rot_dim=32, vdim=64, kv_rank=64, scale=0.12, ff=160),
        panodra_layer(sink=True, heads=3, dim=72, rot_dim=24, vdim=88, kv_rank=96, scale=0.1, scaling=(6.0, 128, 16.0, 1.0),
                      mlp="moe", ff=64, experts=4, top=2)], vocab=211, width=128, loop=(0, 2, 2)),
}


def panodra_random_config(seed: int) -> dict:
    """A Panodra configuration drawn from sizes a model of the design may have."""
    import random
    r = random.Random(seed)

    def layer():
        rot_dim = r.choice([8, 16, 32, 64]); dim = r.choice([16, 32, 64, 96, 128])
        return panodra_layer(sink=r.random() < 0.5, heads=r.choice([1, 2, 4, 6, 8]), dim=dim, rot_dim=rot_dim,
                             vdim=r.choice([16, 32, 64, 72, 128]), kv_rank=r.choice([32, 64, 96, 160, 256]),
                             scale=r.choice([(dim + rot_dim) ** -0.5, 0.1, 0.05]), rot_base=r.choice([1e4, 3e5, 1e6]),
                             scaling=r.choice([None, (6.0, 2048, 16.0, 1.0), (16.0, 64, 4.0, 0.5), (2.0, 256, 8.0, 2.0)]),
                             mlp=r.choice(["dense", "moe", "moe", None]), ff=r.choice([64, 96, 160]),
                             experts=r.choice([2, 4, 9]), top=r.choice([1, 2]))
    n = r.choice([1, 2, 3, 4])
    a = r.randrange(n); b = r.randrange(a + 1, n + 1)
    return panodra_config([layer() for _ in range(n)], vocab=r.choice([128, 500, 1000]), width=r.choice([64, 96, 128, 256]),
                          eps=r.choice([1e-5, 1e-6]), loop=r.choice([None, (a, b, r.choice([1, 2, 3]))]),
                          logit_scale=r.choice([None, 0.4, 2.0]), softcap=r.choice([None, 25.0, 8.0]))


def make_panodra_dir(cfg: dict, out_dir: str, seed: int = 1, dtype=torch.bfloat16, std: float = 0.2, edit=None) -> str:
    """A Panodra model folder with seeded random weights; ``edit(name, tensor) -> tensor`` may change them."""
    from idempotent_llm_b200.config import PanodraConfig
    from idempotent_llm_b200.weights import write_random_model, write_safetensors, SafetensorsFile
    write_random_model(PanodraConfig.from_dict(cfg), out_dir, seed=seed, dtype=dtype, std=std)
    if edit is not None:
        path = os.path.join(out_dir, "model.safetensors")
        f = SafetensorsFile(path)
        tensors = [(n, edit(n, f.get(n).clone())) for n in f.names()]
        del f
        write_safetensors(path, tensors)
    return out_dir


read_model_dir = read_lunulix        # (config dict, tensors by name) of any model folder


# ------------------------------------------------------------------------------------- Fuginex
def fuginex_parallel(heads=4, kv_heads=2, dim=16, scale=0.3, window=20, rot_dims=8, rot_base=5000.0,
                     scaling=(4.0, 64, 8.0, 1.0), r_heads=4, r_kv_heads=2, r_dim=12, r_vdim=20, conv=3, ranks=(8, 16),
                     left_scale=1.3, right_scale=0.9, ff=48, weights_of=None):
    """One ``parallel`` layer of a Fuginex config.json; every size and constant is an argument.  ``scaling``: (factor,
    original, fast, slow) or None; ``ranks``: the two low-rank sizes, or None to leave them to the tensors."""
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale)
    if window:
        left["mask"] = dict(size=window)
    if rot_dims:
        left["rot"] = dict(base=rot_base, dims=rot_dims)
        if scaling:
            left["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    right = dict(heads=r_heads, kv_heads=r_kv_heads, dim=r_dim, vdim=r_vdim, conv=conv)
    if ranks:
        right["decay_rank"], right["gate_rank"] = ranks
    L = dict(type="parallel", mixer=dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale),
             mlp=None if ff is None else dict(kind="dense", ff=ff))
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


def fuginex_attention(heads=4, kv_heads=2, dim=24, vdim=16, scale=0.25, ff=40, weights_of=None):
    L = dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale),
             mlp=None if ff is None else dict(kind="dense", ff=ff))
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


def fuginex_config(layers, vocab=97, width=32, eps=1e-5):
    import copy
    layers = [copy.deepcopy(L) for L in layers]
    for L in layers:                              # a layer that borrows tensors repeats its owner's entry
        if L.get("weights_of") is not None:
            o = layers[L["weights_of"]]
            L.update(type=o["type"], mixer=copy.deepcopy(o["mixer"]), mlp=copy.deepcopy(o["mlp"]))
    return dict(architecture="Fuginex", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)


# Small Fuginex models that differ from one another in every size and option.
FUGINEX = {
    # both kinds of layer, two layers run again with the first ones' tensors (in another order than they came),
    # a window shorter than a page, grouped heads on both sides
    "A": lambda: fuginex_config([fuginex_parallel(), fuginex_attention(),
                                 fuginex_attention(weights_of=1), fuginex_parallel(weights_of=0)]),
    # values of 1 and absent options: one head everywhere, no window, no rotation, no feed-forward, two taps,
    # constants of 1, low-rank sizes left to the tensors
    "B": lambda: fuginex_config([fuginex_parallel(heads=1, kv_heads=1, dim=8, window=None, rot_dims=0, r_heads=1, r_kv_heads=1,
                                                  r_dim=8, r_vdim=8, conv=2, ranks=None, left_scale=1.0, right_scale=1.0, ff=None),
                                 fuginex_attention(heads=1, kv_heads=1, dim=8, vdim=8, ff=None)], vocab=50, width=24),
    # widths that are no multiple of 8 (bfloat16 rows off the 16-byte borders), a rotation of the whole head without
    # scaling, a window of one page and one key, no filter, odd low-rank sizes
    "C": lambda: fuginex_config([fuginex_parallel(heads=3, kv_heads=1, dim=12, scale=0.2, window=65, rot_dims=12, scaling=None,
                                                  r_heads=3, r_kv_heads=3, r_dim=10, r_vdim=6, conv=1, ranks=(5, 3), ff=28),
                                 fuginex_attention(heads=3, kv_heads=3, dim=10, vdim=12, ff=28)] * 2, vocab=33, width=20, eps=1e-6),
    # head sizes the tensor-core attention has (64 and 128), keys of 128 and values of 64 in the recurrence
    "T": lambda: fuginex_config([fuginex_parallel(heads=4, kv_heads=2, dim=64, scale=0.12, window=100, rot_dims=32,
                                                  scaling=(8.0, 128, 16.0, 2.0), r_heads=2, r_kv_heads=1, r_dim=128, r_vdim=64,
                                                  conv=4, ranks=(16, 24), ff=96),
                                 fuginex_attention(heads=4, kv_heads=1, dim=128, vdim=128, scale=0.09, ff=96),
                                 fuginex_parallel(weights_of=0)], vocab=211, width=64),
}


def fuginex_random_config(seed: int) -> dict:
    """A Fuginex configuration drawn from sizes a model of the design may have: one to four layers of both kinds in any
    order, some run again with another's tensors, grouped and ungrouped heads, windows below, at and above a page,
    rotation of none, part or all of a head with or without scaling, filters of 1 to 4 taps, layers without
    feed-forward."""
    import random
    r = random.Random(seed)

    def layer():
        if r.random() < 0.4:
            kv = r.choice([1, 2]); dim = r.choice([32, 64, 96, 128])
            return fuginex_attention(heads=kv * r.choice([1, 2, 4]), kv_heads=kv, dim=dim, vdim=r.choice([dim, 32, 64, 80]),
                                     scale=r.choice([dim ** -0.5, 0.1]), ff=r.choice([None, 64, 160]))
        kv = r.choice([1, 2, 4]); dim = r.choice([32, 48, 64, 128]); rkv = r.choice([1, 2, 4])
        rot = r.choice([0, dim // 2, dim, 16])
        return fuginex_parallel(heads=kv * r.choice([1, 2, 4]), kv_heads=kv, dim=dim, scale=r.choice([dim ** -0.5, 0.1, 0.2]),
                                window=r.choice([None, 7, 64, 70, 129, 200]), rot_dims=rot, rot_base=r.choice([1e4, 4e5, 1e6]),
                                scaling=r.choice([None, (2.0, 1024, 16.0, 1.0), (8.0, 64, 4.0, 0.5), (16.0, 256, 8.0, 2.0)]) if rot else None,
                                r_heads=rkv * r.choice([1, 2]), r_kv_heads=rkv, r_dim=r.choice([16, 32, 40, 64, 128]),
                                r_vdim=r.choice([16, 24, 32, 64, 128]), conv=r.choice([1, 2, 3, 4]),
                                ranks=r.choice([None, (8, 8), (24, 16), (12, 40)]), left_scale=r.choice([1.0, 1.3, 0.4]),
                                right_scale=r.choice([1.0, 0.8, 0.7]), ff=r.choice([None, 64, 160, 256]))
    layers = [layer() for _ in range(r.choice([1, 2, 3]))]
    for _ in range(r.choice([0, 1, 2])):
        layers.insert(r.randrange(1, len(layers) + 1), dict(weights_of=None))      # filled in below
    own = [i for i, L in enumerate(layers) if "type" in L]
    for i, L in enumerate(layers):
        if "type" not in L:
            L["weights_of"] = r.choice(own)
    return fuginex_config(layers, vocab=r.choice([128, 500, 1000]), width=r.choice([64, 96, 128, 256]),
                          eps=r.choice([1e-5, 1e-6]))


def make_fuginex_dir(cfg: dict, out_dir: str, seed: int = 1, dtype=torch.bfloat16, std: float = 0.15, edit=None) -> str:
    """A Fuginex model folder with seeded random weights; ``edit(name, tensor) -> tensor`` may change them."""
    from idempotent_llm_b200.config import FuginexConfig
    from idempotent_llm_b200.weights import write_random_model, write_safetensors, SafetensorsFile
    write_random_model(FuginexConfig.from_dict(cfg), out_dir, seed=seed, dtype=dtype, std=std)
    if edit is not None:
        path = os.path.join(out_dir, "model.safetensors")
        f = SafetensorsFile(path)
        tensors = [(n, edit(n, f.get(n).clone())) for n in f.names()]
        del f
        write_safetensors(path, tensors)
    return out_dir


# ------------------------------------------------------------------------------------- Pununex
def pununex_delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, mlp="dense"):
    """One ``delta`` layer of a Pununex config.json; ``mlp``: None, "dense", an inner size, or a dict as config.json has it."""
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv), mlp=pununex_mlp(mlp))


def pununex_parallel(heads=4, kv_heads=2, dim=24, vdim=16, scale=0.25, softcap=10.0, window=20, keep_first=3, r_heads=2,
                     r_kv_heads=1, r_dim=12, r_vdim=20, conv=4, left_scale=1.3, right_scale=0.6, mlp="moe"):
    """One ``parallel`` layer; absent options (no cap, no window, no kept tokens) are left out of the dict."""
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if softcap:
        left["softcap"] = softcap
    if window:
        left["mask"] = dict(size=window)
        if keep_first:
            left["mask"]["keep_first"] = keep_first
    right = dict(heads=r_heads, kv_heads=r_kv_heads, dim=r_dim, vdim=r_vdim, conv=conv)
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale),
                mlp=pununex_mlp(mlp))


def pununex_moe(experts=6, identity=2, top=3, groups=(4, 2), scale=1.5, ff=24, shared=40):
    router = dict(experts=experts, top=top, scale=scale)
    if identity:
        router["identity"] = identity
    if groups:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    d = dict(kind="moe", expert=dict(ff=ff), router=router)
    if shared:
        d["shared"] = dict(ff=shared)
    return d


def pununex_mlp(mlp):
    if mlp is None or isinstance(mlp, dict):
        return mlp
    if mlp == "dense":
        return dict(kind="dense", ff=48)
    if mlp == "moe":
        return pununex_moe()
    return dict(kind="dense", ff=int(mlp))


def pununex_config(layers, vocab=97, width=32, eps=1e-5, bigram=(53, 5, 11)):
    import copy
    d = dict(architecture="Pununex", vocab=vocab, width=width, norm=dict(eps=eps), layers=[copy.deepcopy(L) for L in layers])
    if bigram:
        d["embedding"] = dict(bigram=dict(buckets=bigram[0], mul_prev=bigram[1], mul_cur=bigram[2]))
    return d


# Small Pununex models that differ from one another in every size and option.
PUNUNEX = {
    # both kinds of layer in both orders, grouped heads on every side, a window shorter than a page with kept first
    # tokens, experts in groups with identity experts and a shared expert, a dense feed-forward
    "A": lambda: pununex_config([pununex_delta(), pununex_parallel(), pununex_parallel(mlp="dense", window=33, keep_first=1),
                                 pununex_delta(mlp="moe")]),
    # values of 1 and absent options: one head everywhere, no cap, no window, one tap, constants of 1, one expert per
    # token, no identity experts, no groups, no shared expert, a layer without feed-forward, no bigram table
    "B": lambda: pununex_config([pununex_parallel(heads=1, kv_heads=1, dim=8, vdim=8, softcap=None, window=None, r_heads=1,
                                                  r_kv_heads=1, r_dim=8, r_vdim=8, conv=1, left_scale=1.0, right_scale=1.0,
                                                  mlp=pununex_moe(experts=3, identity=0, top=1, groups=None, scale=1.0, shared=None)),
                                 pununex_delta(heads=1, kv_heads=1, dim=8, vdim=8, conv=2, mlp=None)], vocab=50, width=24, bigram=None),
    # widths that are no multiple of 8 (bfloat16 rows off the 16-byte borders), a window of one page and one key that
    # keeps a whole page, groups that shut nobody out, multipliers larger than the table (two layers:
    # rows of 20 elements round coarsely in bfloat16, and every norm behind a sublayer blows that up again)
    "C": lambda: pununex_config([pununex_parallel(heads=3, kv_heads=1, dim=12, vdim=6, scale=0.2, softcap=4.0, window=65, keep_first=64,
                                                  r_heads=3, r_kv_heads=3, r_dim=10, r_vdim=6, conv=2,
                                                  mlp=pununex_moe(experts=5, identity=1, top=2, groups=(3, 3), scale=0.7, ff=12, shared=20)),
                                 pununex_delta(heads=3, kv_heads=1, dim=10, vdim=12, conv=4, mlp=60)], vocab=33, width=20, eps=1e-6,
                                bigram=(7, 1000003, 999983)),
    # head sizes the tensor-core attention has, keys of 128 and values of 64 in the recurrences, many experts
    "T": lambda: pununex_config([pununex_parallel(heads=4, kv_heads=1, dim=64, vdim=64, scale=0.12, softcap=30.0, window=100, keep_first=5,
                                                  r_heads=2, r_kv_heads=1, r_dim=128, r_vdim=64, conv=4,
                                                  mlp=pununex_moe(experts=16, identity=0, top=2, groups=(2, 1), scale=2.5, ff=32, shared=64)),
                                 pununex_delta(heads=2, kv_heads=2, dim=64, vdim=128, conv=4, mlp=96),
                                 pununex_parallel(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.09, softcap=None, window=70, keep_first=70,
                                                  r_heads=4, r_kv_heads=4, r_dim=32, r_vdim=32, conv=3, mlp=None)], vocab=211, width=64,
                                bigram=(211, 31, 1)),
}


def pununex_random_config(seed: int) -> dict:
    """A Pununex configuration drawn from sizes a model of the design may have: one to four layers of both kinds in any
    order, grouped and ungrouped heads, windows below, at and above a page with none to many kept tokens, caps, filters
    of 1 to 4 taps, feed-forwards of every kind."""
    import random
    r = random.Random(seed)

    def mlp():
        kind = r.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return r.choice([64, 160])
        count = r.choice([1, 2, 4])
        per = r.choice([2, 3, 4])
        identity = r.choice([0, 1, 2])
        keep = r.randint(1, count)
        return pununex_moe(experts=count * per - identity, identity=identity, top=r.randint(1, min(3, keep * per)),
                           groups=None if count == 1 and r.random() < 0.5 else (count, keep), scale=r.choice([1.0, 2.0, 0.5]),
                           ff=r.choice([16, 40, 64]), shared=r.choice([None, 32, 72]))

    def layer():
        if r.random() < 0.4:
            kv = r.choice([1, 2])
            return pununex_delta(heads=kv * r.choice([1, 2]), kv_heads=kv, dim=r.choice([16, 32, 40, 64, 128]),
                                 vdim=r.choice([16, 24, 32, 64]), conv=r.choice([1, 2, 3, 4]), mlp=mlp())
        kv = r.choice([1, 2, 4]); dim = r.choice([32, 48, 64, 128]); rkv = r.choice([1, 2, 4])
        window = r.choice([None, 7, 64, 70, 129, 200])
        return pununex_parallel(heads=kv * r.choice([1, 2, 4]), kv_heads=kv, dim=dim, vdim=r.choice([dim, 16, 40, 64]),
                                scale=r.choice([dim ** -0.5, 0.1, 0.2]), softcap=r.choice([None, 5.0, 20.0, 50.0]), window=window,
                                keep_first=r.choice([0, 1, 4, 33, 64, 90]) if window else 0, r_heads=rkv * r.choice([1, 2]),
                                r_kv_heads=rkv, r_dim=r.choice([16, 32, 40, 64, 128]), r_vdim=r.choice([16, 24, 32, 64, 128]),
                                conv=r.choice([1, 2, 3, 4]), left_scale=r.choice([1.0, 1.3, 0.4]),
                                right_scale=r.choice([1.0, 0.8, 0.7]), mlp=mlp())
    V = r.choice([128, 500, 1000])
    return pununex_config([layer() for _ in range(r.choice([1, 2, 3, 4]))], vocab=V, width=r.choice([64, 96, 128, 256]),
                          eps=r.choice([1e-5, 1e-6]), bigram=r.choice([None, (V - 1, 3, 7), (2003, 40503, 12289)]))


def make_pununex_dir(cfg: dict, out_dir: str, seed: int = 1, dtype=torch.bfloat16, std: float = 0.15, edit=None) -> str:
    """A Pununex model folder with seeded random weights; ``edit(name, tensor) -> tensor`` may change them."""
    from idempotent_llm_b200.config import PununexConfig
    from idempotent_llm_b200.weights import write_random_model, write_safetensors, SafetensorsFile
    write_random_model(PununexConfig.from_dict(cfg), out_dir, seed=seed, dtype=dtype, std=std)
    if edit is not None:
        path = os.path.join(out_dir, "model.safetensors")
        f = SafetensorsFile(path)
        tensors = [(n, edit(n, f.get(n).clone())) for n in f.names()]
        del f
        write_safetensors(path, tensors)
    return out_dir
