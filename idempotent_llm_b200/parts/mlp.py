"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))``, no bias
(reference: src/detllm/model.py:415-427; float form ``g * sigmoid(g) * u`` in
tests/test_ops.py:240-242 and scripts/attribute_error.py:37-40).  Gate and up
are one matrix here (rows concatenated)."""

from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import FEED_FORWARDS, FeedForward


# the kernels' numbers of the gated activations (csrc/common.cuh: gated_act)
ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu": 2}


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    accepts_residual = True

    @classmethod
    def declare(cls, spec, prefix):
        nm = spec.names
        return [TensorDecl(prefix + nm.gate, (spec.intermediate, spec.hidden)),
                TensorDecl(prefix + nm.up, (spec.intermediate, spec.hidden)),
                TensorDecl(prefix + nm.down, (spec.hidden, spec.intermediate))]

    def __init__(self, spec, weights, prefix, rt):
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} is not built; known: {sorted(ACTIVATIONS)}")
        self.act = ACTIVATIONS[spec.activation]
        self.spec = spec
        self.rt = rt
        nm = spec.names
        gate, up = weights[prefix + nm.gate].to(rt.dtype), weights[prefix + nm.up].to(rt.dtype)
        # with the fused kernels the activation is the epilogue of the gate/up product, which wants
        # gate and up rows interleaved in tiles; otherwise the rows are simply concatenated
        # the activation as the product's epilogue wants rows on 16-byte borders; other widths take the product with
        # padded operands and the activation as a kernel of its own
        aligned = not (rt.dtype == torch.bfloat16 and (spec.hidden % 8 or spec.intermediate % 8))
        self.fused = bool(getattr(rt.kernels, "fused", False)) and aligned
        self.pad = {} if aligned else {"pad": True}
        if self.fused:
            self.w_gate_up = rt.kernels.tile_gate_up(gate, up)
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = weights[prefix + nm.down].to(rt.dtype).contiguous()

    def emit(self, prog, x, h):
        """The calls of ``forward`` on the fused path, adding into the stream ``h``."""
        from ..kernels.program import NotProgrammable
        if not self.fused or self.act != 0:
            raise NotProgrammable("the activation as a kernel of its own, or another than silu, is called from forward")
        s = self.spec
        y = prog.buffer("feed_forward.y", per_token=2 * s.intermediate)
        prog.gemm_swiglu(x, self.w_gate_up, s.hidden, s.intermediate, y)
        prog.gemm_residual(y, self.w_down, s.intermediate, h)

    def forward(self, x, ctx, residual=None):
        """Returns the delta ``[P, N, hidden]``, or None after adding it into ``residual`` in place."""
        K = self.rt.kernels
        if self.fused:
            y = (K.gemm_swiglu(x, self.w_gate_up, self.spec.intermediate) if self.act == 0
                 else K.gemm_gated(x, self.w_gate_up, self.spec.intermediate, self.act))
            if residual is not None:
                K.gemm_residual(y, self.w_down, residual)
                return None
            return K.gemm(y, self.w_down)
        gu = K.gemm(x, self.w_gate_up, **self.pad)          # [P, N, 2 * intermediate]
        y = K.swiglu(gu) if self.act == 0 else K.gated_act(gu[0], self.act)      # [N, intermediate]
        return K.gemm(y, self.w_down, **self.pad)           # [P, N, hidden]


# the kernels' numbers of the activations of one argument (csrc/elementwise.cu: act_cast)
UNARY_ACTIVATIONS = {"relu2": 2}


@FEED_FORWARDS.register("dense_mlp")
class DenseMLP(FeedForward):
    """``down(act(up(x)))`` without a gate; ``relu2`` is the square of relu.  The activation runs in 32-bit on the
    up product's 32-bit output and is rounded a single time, to the down product's input."""

    accepts_residual = True

    @classmethod
    def declare(cls, spec, prefix):
        nm = spec.names
        return [TensorDecl(prefix + nm.up, (spec.intermediate, spec.hidden)),
                TensorDecl(prefix + nm.down, (spec.hidden, spec.intermediate))]

    def __init__(self, spec, weights, prefix, rt):
        if spec.activation not in UNARY_ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} is not built; known: {sorted(UNARY_ACTIVATIONS)}")
        self.spec, self.rt, self.act = spec, rt, UNARY_ACTIVATIONS[spec.activation]
        nm = spec.names
        self.w_up = weights[prefix + nm.up].to(rt.dtype).contiguous()
        self.w_down = weights[prefix + nm.down].to(rt.dtype).contiguous()
        self.pad = {"pad": True} if rt.dtype == torch.bfloat16 and (spec.hidden % 8 or spec.intermediate % 8) else {}

    def forward(self, x, ctx, residual=None):
        K = self.rt.kernels
        if residual is not None and getattr(K, "fused", False) and not self.pad:
            K.dense_ff(x, self.w_up, self.w_down, residual, self.act)       # the three calls below from one
            return None
        y = K.act_cast(K.gemm_store(x, self.w_up, **self.pad), self.act)
        return K.gemm(y, self.w_down, **self.pad)
