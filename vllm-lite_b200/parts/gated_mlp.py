"""Gated feed-forward with a choice of activation and optional biases:
down(f(gate(h) + b_g, up(h) + b_u)) + b_d, f(g, u) = silu(g) u, relu(g) u, or the capped swish
g' sigmoid(alpha g') (u' + shift) with g' = min(g, limit), u' = clamp(u, -limit, limit).

gate and up are stacked into one matrix (gate rows, then up rows) so that one product serves both;
the activation is one kernel on the stacked result and adds the two projections' biases on the way (float32);
the down projection's bias is added by the linear layer.
The SwiGLU part (`parts/mlp.py`) is the bias-free special case whose activation the product kernels
fuse; this part serves what that one does not take.  Without a gate (`gated` False) it is down(f(up(h))) with f a
function of one argument (the square of max(v, 0))."""
from __future__ import annotations

import torch

from .linear import Linear
from .registry import FEED_FORWARDS
from .spec import GatedMlpSpec, TensorDecl


@FEED_FORWARDS.register("gated_mlp")
class GatedMlp:
    graph_safe = True

    @staticmethod
    def declare(spec: GatedMlpSpec) -> dict:
        gate, up, down = spec.names
        I, H = spec.intermediate_size, spec.hidden_size
        if not spec.gated:
            return {up: TensorDecl((I, H)), down: TensorDecl((H, I))}
        d = {gate: TensorDecl((I, H)), up: TensorDecl((I, H)), down: TensorDecl((H, I))}
        if spec.bias:
            d.update({gate + spec.bias_suffix: TensorDecl((I,)), up + spec.bias_suffix: TensorDecl((I,)),
                      down + spec.bias_suffix: TensorDecl((H,))})
        return d

    def __init__(self, spec: GatedMlpSpec, weights: dict, ctx):
        from ..csrc import ops
        known = ops.ACTIVATIONS if spec.gated else ops.UNARY_ACTIVATIONS
        if spec.activation not in known or (spec.bias and not spec.gated):
            raise ValueError(f"gated_mlp: activation {spec.activation!r} ({'with' if spec.gated else 'without'} a gate); "
                             f"known: {', '.join(known)}")
        self.spec = spec
        self.dtype = ctx.dtype
        gate, up, down = spec.names
        if not spec.gated:
            self.gate_up_bias = None
            self.gate_up = Linear(weights[up])
            self.down = Linear(weights[down])
            return
        b = spec.bias_suffix
        self.gate_up_bias = None
        if spec.bias:
            self.gate_up_bias = torch.cat([weights[gate + b].float(), weights[up + b].float()], dim=0).contiguous()
        self.gate_up = Linear(torch.cat([weights[gate], weights[up]], dim=0).contiguous())
        self.down = Linear(weights[down], weights[down + b].float() if spec.bias else None)

    def __call__(self, h, step):
        from ..csrc import ops
        gu = self.gate_up(h, step, "mlp.gate_up")
        act = step.workspace.get(step.tag + "mlp.act", (gu.shape[0], self.spec.intermediate_size), gu.dtype)
        s = self.spec
        if not s.gated:
            return self.down(ops.unary_act(gu, act, s.activation), step, "mlp.down")
        ops.gated_act(gu, act, s.activation, 0, s.alpha, s.limit, s.up_shift, bias=self.gate_up_bias)
        return self.down(act, step, "mlp.down")
