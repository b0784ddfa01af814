"""Norms.  RMS norm: ``x / sqrt(mean(x^2) + eps) * weight``, all in 32-bit; and, at the end of the file, a norm
without statistics (``DyT``: ``tanh(alpha x) * w + b``) and the layer norm with weight and bias.

The reference's float form is ``x / sqrt(mean(x^2))`` (tests/test_ops.py:198-199,
scripts/attribute_error.py:48-51) with the weight folded into the consumer
(src/detllm/prepare.py:342-343); its integer runtime clamps instead of adding
eps (src/detllm/ops/di_rmsnorm.py:14, 50).  Here eps is added to the mean
inside the square root and the weight multiplies afterwards.
"""

from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import NORMS, CastStream, Norm, NormedDelta


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    @classmethod
    def declare(cls, spec, prefix):
        return [TensorDecl(prefix + spec.weight, (spec.size,), init="one_plus_normal")]

    def __init__(self, spec, weights, prefix, rt):
        self.spec = spec
        self.rt = rt
        self.weight = weights[prefix + spec.weight].to(torch.float32).contiguous()

    def forward(self, h, delta, ctx, rows=None):
        if isinstance(delta, CastStream):
            delta = None
        if isinstance(delta, NormedDelta):
            if rows is None:                      # the norm behind the last sublayer and this one in one pass
                return self.rt.kernels.post_pre_norm(h, delta.y, delta.weight, delta.eps, w_pre=self.weight,
                                                     eps_pre=self.spec.eps)
            delta.add_into(h, self.rt.kernels)
            delta = None
        return self.rt.kernels.add_rmsnorm(h, delta, self.weight, self.spec.eps, rows=rows)

    def emit(self, prog, h, out, rows=False):
        prog.add_rmsnorm(h, self.weight, self.spec.eps, out, self.spec.size, rows=rows)


@NORMS.register("dyt")
class DyT(Norm):
    """``tanh(alpha x) * w + b`` element by element in 32-bit: no mean, no variance, so a row's elements do not
    depend on one another.  A pending delta is added into the stream in the same pass."""

    @classmethod
    def declare(cls, spec, prefix):
        name = prefix + spec.weight
        return [TensorDecl(name, (spec.size,), init="one_plus_normal"),
                TensorDecl(name + spec.bias_suffix, (spec.size,)),
                TensorDecl(name + spec.alpha_suffix, (), init="half_plus_normal")]

    def __init__(self, spec, weights, prefix, rt):
        self.spec, self.rt = spec, rt
        name = prefix + spec.weight
        self.weight = weights[name].to(torch.float32).contiguous()
        self.bias = weights[name + spec.bias_suffix].to(torch.float32).contiguous()
        self.alpha = float(weights[name + spec.alpha_suffix].to(torch.float32).item())     # one number, read once at load

    def forward(self, h, delta, ctx, rows=None):
        if isinstance(delta, (NormedDelta, CastStream)):
            delta.add_into(h, self.rt.kernels)
            delta = None
        return self.rt.kernels.add_dyt(h, delta, self.weight, self.bias, self.alpha, rows=rows)


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(variance + eps) * w + b`` in 32-bit, the variance the mean of the squared deviations.  A
    pending delta is added into the stream in the same pass."""

    @classmethod
    def declare(cls, spec, prefix):
        name = prefix + spec.weight
        return [TensorDecl(name, (spec.size,), init="one_plus_normal"), TensorDecl(name + spec.bias_suffix, (spec.size,))]

    def __init__(self, spec, weights, prefix, rt):
        self.spec, self.rt = spec, rt
        name = prefix + spec.weight
        self.weight = weights[name].to(torch.float32).contiguous()
        self.bias = weights[name + spec.bias_suffix].to(torch.float32).contiguous()

    def forward(self, h, delta, ctx, rows=None):
        if isinstance(delta, (NormedDelta, CastStream)):
            delta.add_into(h, self.rt.kernels)
            delta = None
        return self.rt.kernels.add_layernorm(h, delta, self.weight, self.bias, self.spec.eps, rows=rows)
