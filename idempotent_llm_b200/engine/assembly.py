"""From a ModelSpec to (a) the tensors the model declares and (b) the model.

The generic decoder: token embedding, the schedule of blocks, final norm and
head, as the reference's step runs them (src/detllm/model.py:233-286), except
that logits are computed only for the rows that are asked for.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.spec import CacheNeed
from ..config.specs import ModelSpec
from ..parts.base import BLOCKS, EMBEDDINGS, MIXERS, NORMS, CastStream, NormedDelta, Runtime
from ..weights.loader import TensorDecl


def declare_weights(spec: ModelSpec) -> List[TensorDecl]:
    decls = [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden))]
    if spec.embedding is not None:
        decls += EMBEDDINGS.get(spec.embedding.kind).declare(spec.embedding, "")
    for layer in spec.layers:
        decls += BLOCKS.get(layer.kind).declare(layer)
    decls += NORMS.get(spec.final_norm.kind).declare(spec.final_norm, spec.final_norm_prefix)
    if spec.mix_in_name:
        decls.append(TensorDecl(spec.mix_in_name, (spec.hidden, 2 * spec.hidden)))
    # tied: an lm_head in the file is tolerated and ignored; untied: it is required
    decls.append(TensorDecl(spec.head_name, (spec.vocab_size, spec.hidden), optional=spec.tie_embeddings))
    # a tensor that several parts share (a table all layers read) is declared by each of them, alike
    seen, unique = {}, []
    for d in decls:
        if d.name in seen:
            if seen[d.name] != d:
                raise ValueError(f"tensor {d.name} is declared twice, differently")
            continue
        seen[d.name] = d
        unique.append(d)
    return unique


EMBEDDING_CACHE_ID = -1     # the cache entry of what a token embedding keeps per sequence (mixers' entries count from 0)


def cache_needs(spec: ModelSpec) -> Dict[int, CacheNeed]:
    """cache id -> need, from the mixer of the schedule entry that writes it (and from the token embedding, if it is
    of a kind that keeps something per sequence)."""
    needs: Dict[int, CacheNeed] = {}
    if spec.embedding is not None:
        need = EMBEDDINGS.get(spec.embedding.kind).cache_need(spec.embedding)
        if need is not None and need.state_shape is not None:
            needs[EMBEDDING_CACHE_ID] = need
    for e in spec.schedule:
        need = MIXERS.get(spec.layers[e.layer].mixer.kind).cache_need(spec.layers[e.layer].mixer)
        if e.writes_cache:
            needs[e.cache] = need
    return needs


class CausalLM:
    """Embedding -> blocks in schedule order -> final norm -> head."""

    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.embed = weights[spec.embed_name].to(rt.dtype).contiguous()
        if spec.tie_embeddings:
            self.head = self.embed
        else:
            self.head = weights[spec.head_name].to(rt.dtype).contiguous()
        self.embedding = None
        if spec.embedding is not None:
            self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding, weights, "", rt)
        self.blocks = [BLOCKS.get(layer.kind)(layer, weights, layer.prefix, rt) for layer in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, weights,
                                                          spec.final_norm_prefix, rt)
        self.mix_in = weights[spec.mix_in_name].to(rt.dtype).contiguous() if spec.mix_in_name else None
        self._programs = {}
        self.graph_safe = all(getattr(part, "graph_safe", True) for b in self.blocks
                              for part in vars(b).values())
        # False if a part runs steps of different shapes on different kernels (the same sums in another order)
        self.same_bits_across_steps = all(getattr(part, "same_bits_across_steps", True) for b in self.blocks
                                          for part in vars(b).values())

    def program(self, cache):
        """The model's kernel calls over ``cache`` as a step program (``kernels/program.py``), made once; None
        if a part cannot emit its calls, the kernels hold no programs (32-bit; separate epilogues), or a
        stand-in for the kernels has none."""
        key = id(cache)
        if key not in self._programs:
            self._programs[key] = (cache, self._emit(cache))   # (the cache is kept: its id stays its own)
        return self._programs[key][1]

    def _emit(self, cache):
        K = self.rt.kernels
        if not hasattr(K, "use_programs"):
            return None
        from ..kernels.program import NotProgrammable, StepProgram
        hidden = self.spec.hidden
        try:
            if float(getattr(self.spec, "embed_scale", 1.0)) != 1.0:
                raise NotProgrammable("a scaled embedding is called from forward")
            if self.mix_in is not None or self.spec.logit_scale != 1.0 or self.spec.logit_softcap:
                raise NotProgrammable("a stream mixed with the embedding, or scaled and capped logits, are called from forward")
            if self.embedding is not None:
                raise NotProgrammable("a token embedding with state is called from forward")
            prog = StepProgram(K)
            h = prog.buffer("stream", per_token=4 * hidden)
            prog.embed(self.embed, h)
            for e in self.spec.schedule:
                block = self.blocks[e.layer]
                state = cache.state_of(e.cache)
                if not hasattr(block, "emit") or (state is not None and state.numel()):
                    raise NotProgrammable("a block without emit, or with per-sequence state")
                block.emit(prog, h, cache.view(e.cache), state, e.writes_cache)
            if not hasattr(self.final_norm, "emit"):
                raise NotProgrammable("the final norm has no emit")
            x = prog.buffer("head.x", per_row=2 * hidden)
            self.final_norm.emit(prog, h, x, rows=True)
            logits = prog.buffer("logits")
            prog.gemm_store(x, self.head, hidden, logits, rows=True)
            return prog.finish(logits, self.head.shape[0])
        except NotProgrammable:
            return None

    def forward(self, ctx, cache, want_rows: torch.Tensor) -> torch.Tensor:
        """Run the step's tokens; returns 32-bit logits ``[len(want_rows), vocab]``."""
        K = self.rt.kernels
        if getattr(K, "use_programs", False):
            prog = self.program(cache)
            if prog is not None:
                return prog.run(ctx, want_rows)
        scale = float(getattr(self.spec, "embed_scale", 1.0))
        pending = None
        if self.embedding is not None:
            h, pending = self.embedding.forward(self.embed, ctx, cache.state_of(EMBEDDING_CACHE_ID))
        else:
            h = K.embed(ctx.tokens, self.embed) if scale == 1.0 else K.embed_scaled(ctx.tokens, self.embed, scale)
        pad = {"pad": True} if self.spec.hidden % 8 else {}
        x0 = h.clone() if self.mix_in is not None else None         # the embedding output, kept for the mixes
        for e in self.spec.schedule:
            if e.mix_in:
                # the stream (what is pending added first) and the embedding output side by side, times one matrix
                if isinstance(pending, (NormedDelta, CastStream)):
                    pending.add_into(h, K)
                    pending = None
                h, pending = K.gemm_store(K.concat_cast(h, pending, x0), self.mix_in, **pad), None
            h, pending = self.blocks[e.layer].forward(h, pending, ctx, cache.view(e.cache),
                                                      cache.state_of(e.cache), e.writes_cache)
        x = self.final_norm.forward(h, pending, ctx, rows=want_rows)
        logits = K.gemm_store(x, self.head, **pad)
        if self.spec.logit_scale != 1.0 or self.spec.logit_softcap:
            K.logit_cap(logits, self.spec.logit_scale, self.spec.logit_softcap or 0.0)
        return logits

    def weight_bytes(self) -> int:
        seen, n = set(), 0

        def add(t):
            nonlocal n
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()

        def walk(o, depth=0):
            if isinstance(o, torch.Tensor):
                add(o)
            elif depth < 4 and hasattr(o, "__dict__"):
                for k, v in vars(o).items():
                    if k in ("rt", "spec"):
                        continue
                    if isinstance(v, (list, tuple)):
                        for i in v:
                            walk(i, depth + 1)
                    else:
                        walk(v, depth + 1)
        walk(self)
        return n
