"""Interfaces of the parts a layer is put together from, and their registries.

Every part is built from its own spec (sizes and constants as parameters), a
dict of weights by checkpoint name, the name prefix of its tensors, and the
``Runtime`` (device, compute dtype, kernels).  No part sees the model's
configuration.  The registries map a spec's ``kind`` to the implementing class;
registering another class under another kind adds a part without touching
this package.

Interfaces (duck-typed; the base classes document them):

* ``Norm.forward(h, delta, ctx, rows=None) -> x``: ``h`` is the 32-bit residual
  stream ``[N, hidden]``; if ``delta`` (32-bit partial sums ``[P, N, hidden]``) is
  given it is added into ``h`` first, in place, in 32-bit; ``x`` is the normed
  result in the compute dtype.  ``rows`` selects token rows (then ``h`` is left
  untouched and only those rows are returned).
* ``Mixer.forward(x, ctx, kv, state, writes_cache) -> delta`` and
  ``Mixer.cache_need(spec) -> CacheNeed``: ``kv`` is the ``KVView`` of the cache
  entry (or None), ``state`` the per-sequence state tensor ``[max_seqs, ...]`` of
  the entry (or None), indexed with ``ctx.slots``.
* ``FeedForward.forward(x, ctx) -> delta``.
* ``PositionEncoding.tables(ctx)``: whatever its mixer kernels need for the
  step's tokens (computed once per step and shared between layers).
* A token embedding other than the plain lookup (``EMBEDDINGS``): ``declare(spec, prefix)``,
  ``cache_need(spec)`` (per-sequence state it keeps between steps, or None) and
  ``forward(table, ctx, state) -> (h, pending)`` with ``h`` the 32-bit stream.
* ``Block.forward(h, pending, ctx, kv, state, writes_cache) -> (h, pending)``:
  ``pending`` is a delta not yet added to ``h``; the next norm adds it.

A mixer or feed-forward whose class sets ``accepts_residual = True`` also takes ``residual=h``
and may add its output into ``h`` itself (fused into its last kernel) and return None.

Optional, beside ``forward``: ``emit``.  A part whose kernel calls never change from step to step may
write them down once in a ``StepProgram`` (``kernels/program.py``), which the library then runs for
every step with one call from the host: ``Norm.emit(prog, h, out, rows=False)``,
``Mixer.emit(prog, x, h, kv, state, writes_cache)`` and ``FeedForward.emit(prog, x, h)`` (both add their
output into the stream ``h``), ``PositionEncoding.emit(prog) -> its table's buffers``,
``Block.emit(prog, h, kv, state, writes_cache)``; buffers are the program's, by index.  ``emit`` must
make exactly the calls ``forward`` makes.  A part without it, or one that raises ``NotProgrammable``,
makes its model run call by call from ``forward``: nothing else changes.

``delta`` is always 32-bit ``[P, N, hidden]``: P partial sums whose total is the
part's output (P is 1 unless a matrix product was split along its inner axis);
the consumer adds them in ascending order.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

import torch

from ..cache.spec import CacheNeed
from ..weights.loader import TensorDecl


@dataclass
class Runtime:
    device: torch.device
    dtype: torch.dtype          # compute/storage dtype of activations, weights and cache
    kernels: object             # idempotent_llm_b200.kernels.Kernels (or a stand-in with its methods)
    shared: dict = field(default_factory=dict)   # what several parts of one model hold in common (a table cast once)

    def shared_tensor(self, weights, name: str, dtype) -> "torch.Tensor":
        """``weights[name]`` in ``dtype``, converted once however many parts ask for it."""
        key = (name, dtype)
        t = self.shared.get(key)
        if t is None:
            t = self.shared[key] = weights[name].to(dtype).contiguous()
        return t


class NormedDelta:
    """A pending delta that is normed before it is added: ``h += y / sqrt(mean(y^2) + eps) * weight``.  A block that
    ends with a norm behind its last sublayer may hand this on instead of adding it itself, so that the next
    block's first norm does both in one pass over the row; any other consumer calls ``add_into`` first."""

    def __init__(self, y, weight, eps: float):
        self.y, self.weight, self.eps = y, weight, eps

    def add_into(self, h, kernels) -> None:
        kernels.post_pre_norm(h, self.y, self.weight, self.eps)


class CastStream:
    """A pending "delta" that adds nothing: the stream is up to date, and ``x`` holds it in the storage dtype already
    (written by the pass that last touched the stream).  A block whose first sublayer reads the stream itself takes
    ``x`` instead of casting again; every other consumer treats it as no delta at all."""

    def __init__(self, x):
        self.x = x

    def add_into(self, h, kernels) -> None:
        return None


class Part:
    # False for a part that synchronises with the host inside ``forward`` (reads device values):
    # a model with such a part runs its single-token steps without CUDA graphs.
    graph_safe = True
    # False for a part whose result for a token depends, in its last bits, on the step's shape (it runs prompts and
    # single tokens on different kernels): tools that compare runs bit for bit then compare up to rounding.
    same_bits_across_steps = True

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        return []


class Norm(Part):
    def forward(self, h, delta, ctx, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    def tables(self, ctx):
        raise NotImplementedError


class Mixer(Part):
    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed()

    def forward(self, x, ctx, kv, state, writes_cache: bool):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError


class Block(Part):
    def forward(self, h, pending, ctx, kv, state, writes_cache: bool):
        raise NotImplementedError


class _Registry:
    def __init__(self, what: str):
        self.what = what
        self._by_kind: Dict[str, type] = {}

    def register(self, kind: str, cls: type = None):
        if cls is None:                       # decorator form
            def deco(c):
                self._by_kind[kind] = c
                return c
            return deco
        self._by_kind[kind] = cls
        return cls

    def get(self, kind: str) -> type:
        try:
            return self._by_kind[kind]
        except KeyError:
            raise KeyError(f"no {self.what} registered under kind {kind!r}; "
                           f"known: {sorted(self._by_kind)}") from None

    def kinds(self):
        return sorted(self._by_kind)


NORMS = _Registry("norm")
EMBEDDINGS = _Registry("token embedding")
POSITIONS = _Registry("position encoding")
MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
BLOCKS = _Registry("block")
