"""RMS norm: h = x / sqrt(mean(x^2) + eps) * w, in float32, with the pending
residual added into the stream by the same kernel
(crates/model/src/components/norm/rms_norm.rs:26-49 of the reference)."""
from __future__ import annotations

import torch

from .registry import NORMS
from .spec import NormSpec, TensorDecl


@NORMS.register("rms_norm")
class RmsNorm:
    factorable = True          # h = (x * weight) * scale(x): neighbours may fuse it (parts/base.py, ScaledRows)

    @staticmethod
    def declare(spec: NormSpec) -> dict:
        if not spec.has_weight:
            return {}
        # a weight stored around zero (offset + w) starts around zero in the random-weights mode as well
        return {spec.tensor: TensorDecl(() if spec.scalar else (spec.size,), init="linear" if spec.offset else "norm")}

    def __init__(self, spec: NormSpec, weights: dict, ctx):
        self.spec = spec
        self.dtype = ctx.dtype
        # A vector of `size` numbers: kept as float32 on the device (exact from bfloat16).  A norm with one number
        # for all coordinates holds that number `size` times, so every kernel sees a vector; a norm without a tensor
        # holds ones; a weight stored around zero is kept as offset + w (one float32 rounding, done once).
        if not spec.has_weight:
            w = torch.ones(spec.size, dtype=torch.float32, device=ctx.device)
        else:
            w = weights[spec.tensor].to(device=ctx.device, dtype=torch.float32)
            if spec.offset:
                w = w + float(spec.offset)
        self.weight = (w.reshape(1).expand(spec.size) if spec.scalar else w).contiguous()

    adds_bias = True           # add_normed takes the bias that the sub-layer's last product left out
    takes_pair = True          # ... and a `ScaledPair` (two sub-layers side by side) in place of y

    def add_normed(self, y, x, step, cast=None, mult=1.0, bias=None):
        """x += mult * norm(y + bias): what a block that norms its sub-layers' OUTPUTS calls; `cast` (a buffer in the
        activation dtype, or None) receives the new x.  y may be a `ScaledPair`.  Returns cast."""
        from ..csrc import ops
        from .base import ScaledPair
        if isinstance(y, ScaledPair):
            ops.rmsnorm_add(y.a, self.weight, self.spec.eps, mult, x, cast, bias=bias, pair=(y.b, y.a_scale, y.b_scale))
        else:
            ops.rmsnorm_add(y, self.weight, self.spec.eps, mult, x, cast, bias=bias)
        return cast

    def fused_rms(self):
        """(weight, eps): what a kernel that applies this norm itself needs (the attention mixer's
        kernel norms every head while it rotates it)."""
        return self.weight, self.spec.eps

    def __call__(self, x, delta, step, rows=None, tag="norm"):
        from ..csrc import ops
        R = x.shape[0] if rows is None else rows.shape[0]
        out = step.workspace.get(step.tag + tag, (R, self.spec.size), self.dtype)
        return ops.add_rmsnorm(x, delta, self.weight, self.spec.eps, out, rows=rows)


@NORMS.register("layer_norm")
class LayerNorm:
    """h = (x - mean x) / sqrt(var x + eps) * w, var = the mean of the squared deviations, no bias; float32.
    Beside the interface of every norm (`__call__`: the stream's rows, a pending delta added first) it offers
    `add_normed`, what a block that norms its sub-layers' outputs calls."""

    @staticmethod
    def declare(spec: NormSpec) -> dict:
        return {spec.tensor: TensorDecl((spec.size,), init="norm")}

    def __init__(self, spec: NormSpec, weights: dict, ctx):
        self.spec = spec
        self.dtype = ctx.dtype
        self.weight = weights[spec.tensor].to(device=ctx.device, dtype=torch.float32).contiguous()

    def add_normed(self, y, x, step, cast=None, mult=1.0):
        """x += norm(y); `cast` (a buffer in the activation dtype, or None) receives the new x.  Returns cast."""
        from ..csrc import ops
        if mult != 1.0:
            raise NotImplementedError("the layer norm's kernel adds its result as it is")
        ops.layernorm_add(y, self.weight, self.spec.eps, x, cast)
        return cast

    def __call__(self, x, delta, step, rows=None, tag="norm"):
        from ..csrc import ops
        if delta is not None:
            raise NotImplementedError("the layer norm takes the stream as it is; a pending delta belongs to a pre-norm block")
        R = x.shape[0] if rows is None else rows.shape[0]
        out = step.workspace.get(step.tag + tag, (R, self.spec.size), self.dtype)
        return ops.layernorm_rows(x, rows, self.weight, self.spec.eps, out)


@NORMS.register("dyn_tanh")
class DynTanh:
    """h = tanh(alpha x) * w + b, element by element in float32: alpha a learned scalar, w and b vectors; no mean and
    no variance are computed, so the spec's eps is not used.  A block that keeps several streams applies it inside
    its own pass over the streams (`elementwise()` hands it the three tensors)."""

    @staticmethod
    def declare(spec: NormSpec) -> dict:
        return {spec.tensor: TensorDecl((spec.size,), init="norm"),
                spec.tensor + spec.bias_suffix: TensorDecl((spec.size,)),
                spec.tensor + spec.alpha_suffix: TensorDecl((), init="norm")}

    def __init__(self, spec: NormSpec, weights: dict, ctx):
        self.spec = spec
        self.dtype = ctx.dtype
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()
        self.weight = f32(weights[spec.tensor])
        self.bias = f32(weights[spec.tensor + spec.bias_suffix])
        self.alpha = f32(weights[spec.tensor + spec.alpha_suffix]).reshape(1)

    def elementwise(self):
        return self.alpha, self.weight, self.bias

    def __call__(self, x, delta, step, rows=None, tag="norm"):
        from ..csrc import ops
        R = x.shape[0] if rows is None else rows.shape[0]
        out = step.workspace.get(step.tag + tag, (R, self.spec.size), self.dtype)
        return ops.dyt_rows(x, delta, rows, self.alpha, self.weight, self.bias, out)
