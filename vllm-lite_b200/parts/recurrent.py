"""Mixers that keep a state of fixed size per request instead of a growing cache: a selective state space, a
matrix memory with exponential gates, a delta rule with a decay per key channel, and a memory with a decay per key
channel behind token shifts (time mixing).

Each is: one stacked projection of the input -> (a short causal convolution) -> a scan over the step's tokens from
the state in the request's slot (csrc/recurrent.cu; a decoded token is a portion of one token) -> a gated RMS norm ->
the output projection.  The state of a request is one row of float32 numbers (`FixedState`), zero when the slot is
handed out: the convolution's last inputs first, then the recurrence's own state.  What the design computes in
float32 (gates, decays, step sizes, unit norms, the state) is float32 here whatever the model's dtype.
"""
from __future__ import annotations

import torch

from ..cache.spec import FixedState
from .linear import Linear
from .registry import MIXERS
from .spec import DeltaRuleSpec, MatrixMemorySpec, StateSpaceSpec, TensorDecl, TimeMixSpec


def _f32(t, ctx):
    return t.to(device=ctx.device, dtype=torch.float32).contiguous()


@MIXERS.register("state_space")
class StateSpace:
    graph_safe = True

    @staticmethod
    def _sizes(s: StateSpaceSpec):
        inner = s.num_heads * s.vdim
        conv_ch = inner + 2 * s.groups * s.state
        return inner, conv_ch, 2 * inner + 2 * s.groups * s.state + s.num_heads

    @staticmethod
    def declare(s: StateSpaceSpec) -> dict:
        inner, conv_ch, width = StateSpace._sizes(s)
        w_in, conv, conv_b, dt_bias, a_log, d, norm, o = s.names
        return {w_in: TensorDecl((width, s.hidden_size)), conv: TensorDecl((conv_ch, s.conv), init="conv"),
                conv_b: TensorDecl((conv_ch,)), dt_bias: TensorDecl((s.num_heads,), init="unit"),
                a_log: TensorDecl((s.num_heads,), init="unit"), d: TensorDecl((s.num_heads,), init="norm"),
                norm: TensorDecl((inner,), init="norm"), o: TensorDecl((s.hidden_size, inner))}

    @staticmethod
    def cache_need(s: StateSpaceSpec):
        inner, conv_ch, _ = StateSpace._sizes(s)
        from ..csrc import ops
        return FixedState(((s.conv - 1) * conv_ch + ops.scan_state_floats(s.num_heads, s.state, s.vdim),))

    def __init__(self, s: StateSpaceSpec, weights: dict, ctx):
        from ..csrc import ops
        if s.num_heads % s.groups or (s.num_heads * s.vdim) % s.norm_groups or s.conv < 1:
            raise ValueError(f"state space: {s.num_heads} heads in {s.groups} groups, {s.norm_groups} norm parts, {s.conv} taps")
        ops.scan_lanes(s.state)
        self.spec, self.dtype = s, ctx.dtype
        w_in, conv, conv_b, dt_bias, a_log, d, norm, o = s.names
        self.in_proj = Linear(weights[w_in])
        self.o_proj = Linear(weights[o])
        self.conv, self.conv_b = _f32(weights[conv], ctx), _f32(weights[conv_b], ctx)
        self.dt_bias, self.a_log, self.d = _f32(weights[dt_bias], ctx), _f32(weights[a_log], ctx), _f32(weights[d], ctx)
        self.norm = _f32(weights[norm], ctx)

    def __call__(self, h, step, cache):
        from ..csrc import ops
        s, ws, tag = self.spec, step.workspace, step.tag
        inner, conv_ch, width = self._sizes(s)
        T = h.shape[0]
        proj = self.in_proj(h, step, "ssm.in")
        xbc = ws.get(tag + "ssm.xbc", (T, conv_ch), torch.float32)
        ops.short_conv(proj, inner, conv_ch, self.conv, self.conv_b, cache.state, 0, step.cu_seqlens, step.state_slots, xbc,
                       longest=step.max_query_len)
        y = ws.get(tag + "ssm.y", (T, inner), torch.float32)
        ops.ssd_scan(xbc, proj, width - s.num_heads, self.dt_bias, self.a_log, self.d, cache.state, (s.conv - 1) * conv_ch,
                     step.cu_seqlens, step.state_slots, y, s.num_heads, s.groups, s.state, s.vdim)
        gated = ws.get(tag + "ssm.gated", (T, inner), self.dtype)
        ops.gate_norm(y, proj, 0, "silu", True, self.norm, s.eps, gated, inner // s.norm_groups)
        return self.o_proj(gated, step, "ssm.o")


@MIXERS.register("matrix_memory")
class MatrixMemory:
    graph_safe = True

    @staticmethod
    def declare(s: MatrixMemorySpec) -> dict:
        q, k, v, g, o, norm, i, i_b, f, f_b = s.names
        H, D, P, W = s.num_heads, s.dim, s.vdim, s.hidden_size
        return {q: TensorDecl((H * D, W)), k: TensorDecl((H * D, W)), v: TensorDecl((H * P, W)), g: TensorDecl((H * P, W)),
                o: TensorDecl((W, H * P)), norm: TensorDecl((H * P,), init="norm"), i: TensorDecl((H, W)),
                i_b: TensorDecl((H,), init="unit"), f: TensorDecl((H, W)), f_b: TensorDecl((H,), init="norm")}

    @staticmethod
    def cache_need(s: MatrixMemorySpec):
        from ..csrc import ops
        return FixedState((ops.mlstm_state_floats(s.num_heads, s.dim, s.vdim),))

    def __init__(self, s: MatrixMemorySpec, weights: dict, ctx):
        if not s.gate_cap > 0:
            raise ValueError(f"matrix memory: the gates' cap must be positive, got {s.gate_cap}")
        self.spec, self.dtype = s, ctx.dtype
        q, k, v, g, o, norm, i, i_b, f, f_b = s.names
        self.in_proj = Linear(torch.cat([weights[n] for n in (q, k, v, g, i, f)], dim=0).contiguous())
        self.o_proj = Linear(weights[o])
        self.norm, self.i_b, self.f_b = _f32(weights[norm], ctx), _f32(weights[i_b], ctx), _f32(weights[f_b], ctx)

    def __call__(self, h, step, cache):
        from ..csrc import ops
        s, ws, tag = self.spec, step.workspace, step.tag
        H, D, P = s.num_heads, s.dim, s.vdim
        T = h.shape[0]
        proj = self.in_proj(h, step, "mm.in")
        o = ws.get(tag + "mm.o", (T, H * P), torch.float32)
        ops.mlstm_scan(proj, 0, H * D, 2 * H * D, 2 * H * D + 2 * H * P, 2 * H * D + 2 * H * P + H, self.i_b, self.f_b,
                       s.gate_cap, D ** -0.5, s.denom_eps, cache.state, 0, step.cu_seqlens, step.state_slots, o, H, D, P)
        gated = ws.get(tag + "mm.gated", (T, H * P), self.dtype)
        ops.gate_norm(o, proj, 2 * H * D + H * P, "sigmoid", False, self.norm, s.eps, gated, P)
        return self.o_proj(gated, step, "mm.out")


@MIXERS.register("delta_rule")
class DeltaRule:
    graph_safe = True

    @staticmethod
    def declare(s: DeltaRuleSpec) -> dict:
        q, k, v, conv, b, a_log, norm, a1, a2, dt_bias, g1, g2, o = s.names
        H, G, D, P, W = s.num_heads, s.num_kv_heads, s.dim, s.vdim, s.hidden_size
        return {q: TensorDecl((G * D, W)), k: TensorDecl((G * D, W)), v: TensorDecl((H * P, W)),
                q + conv: TensorDecl((G * D, s.conv), init="conv"), k + conv: TensorDecl((G * D, s.conv), init="conv"),
                v + conv: TensorDecl((H * P, s.conv), init="conv"), b: TensorDecl((H, W)),
                a_log: TensorDecl((H,), init="unit"), norm: TensorDecl((P,), init="norm"),
                a1: TensorDecl((s.decay_rank, W)), a2: TensorDecl((H * D, s.decay_rank)),
                dt_bias: TensorDecl((H * D,), init="unit"), g1: TensorDecl((s.gate_rank, W)),
                g2: TensorDecl((H * P, s.gate_rank)), o: TensorDecl((W, H * P))}

    @staticmethod
    def _conv_channels(s):
        return 2 * s.num_kv_heads * s.dim + s.num_heads * s.vdim

    @staticmethod
    def cache_need(s: DeltaRuleSpec):
        from ..csrc import ops
        return FixedState(((s.conv - 1) * DeltaRule._conv_channels(s) + ops.scan_state_floats(s.num_heads, s.dim, s.vdim),))

    def __init__(self, s: DeltaRuleSpec, weights: dict, ctx):
        from ..csrc import ops
        if s.num_heads % s.num_kv_heads or s.conv < 1:
            raise ValueError(f"delta rule: {s.num_kv_heads} key heads do not divide {s.num_heads} heads, or no tap")
        ops.scan_lanes(s.dim)
        self.spec, self.dtype = s, ctx.dtype
        q, k, v, conv, b, a_log, norm, a1, a2, dt_bias, g1, g2, o = s.names
        self.in_proj = Linear(torch.cat([weights[n] for n in (q, k, v, b)], dim=0).contiguous())
        self.low_proj = Linear(torch.cat([weights[a1], weights[g1]], dim=0).contiguous())
        # second stage of both low-rank pairs as one product: [[a2, 0], [0, g2]]; the zero blocks add exact zeros
        HD, HP, ra, rg = weights[a2].shape[0], weights[g2].shape[0], s.decay_rank, s.gate_rank
        up = torch.zeros((HD + HP, ra + rg), dtype=weights[a2].dtype, device=weights[a2].device)
        up[:HD, :ra] = weights[a2]
        up[HD:, ra:] = weights[g2]
        self.up_proj = Linear(up)
        self.o_proj = Linear(weights[o])
        self.conv = _f32(torch.cat([weights[q + conv], weights[k + conv], weights[v + conv]], dim=0), ctx)
        self.a_log, self.dt_bias, self.norm = _f32(weights[a_log], ctx), _f32(weights[dt_bias], ctx), _f32(weights[norm], ctx)

    def __call__(self, h, step, cache):
        from ..csrc import ops
        s, ws, tag = self.spec, step.workspace, step.tag
        H, G, D, P = s.num_heads, s.num_kv_heads, s.dim, s.vdim
        C = self._conv_channels(s)
        T = h.shape[0]
        proj = self.in_proj(h, step, "dr.in")
        low = self.low_proj(h, step, "dr.low")
        up = self.up_proj(low, step, "dr.up")                      # [decay (H*D) | gate (H*P)]
        qkv = ws.get(tag + "dr.qkv", (T, C), torch.float32)
        ops.short_conv(proj, 0, C, self.conv, None, cache.state, 0, step.cu_seqlens, step.state_slots, qkv,
                       longest=step.max_query_len)
        o = ws.get(tag + "dr.o", (T, H * P), torch.float32)
        ops.delta_scan(qkv, up, 0, self.dt_bias, self.a_log, proj, C, D ** -0.5, s.unit_eps, cache.state, (s.conv - 1) * C,
                       step.cu_seqlens, step.state_slots, o, H, G, D, P)
        gated = ws.get(tag + "dr.gated", (T, H * P), self.dtype)
        ops.gate_norm(o, up, H * D, "sigmoid", False, self.norm, s.eps, gated, P)
        return self.o_proj(gated, step, "dr.out")


@MIXERS.register("time_mix")
class TimeMix:
    """A memory per head with a decay per key channel, read through five token shifts of the input (`TimeMixSpec`).

    token shifts (one kernel, five mixes) -> W_r, W_k, W_v, W_g, W_w1 each on its own mix -> tanh -> W_w2 -> the decays
    exp(-exp(z + w0)) in place (`ops.decay_from_raw`) -> the scan (`ops.decay_scan`) -> RMS norm per head,
    weight, silu gate (`ops.gate_norm`) -> W_o.  The state of a request is one row of float32: the input row of its last
    token, then the heads' memories in the scan's own layout.  r, k, v and the raw decay leave their products in float32
    (the products add in float32 anyway), so nothing that enters the recurrence is rounded to the model's dtype."""
    graph_safe = True
    MIXES = "rkvgw"

    @staticmethod
    def declare(s: TimeMixSpec) -> dict:
        mu, r, k, v, g, w1, w2, w0, u, norm, o = s.names
        HD, W = s.num_heads * s.dim, s.hidden_size
        d = {mu + m: TensorDecl((W,), init="unit") for m in TimeMix.MIXES}
        d.update({r: TensorDecl((HD, W)), k: TensorDecl((HD, W)), v: TensorDecl((HD, W)), g: TensorDecl((HD, W)),
                  w1: TensorDecl((s.decay_rank, W)), w2: TensorDecl((HD, s.decay_rank)), w0: TensorDecl((HD,), init="unit"),
                  u: TensorDecl((s.num_heads, s.dim), init="unit"), norm: TensorDecl((HD,), init="norm"),
                  o: TensorDecl((W, HD))})
        return d

    @staticmethod
    def cache_need(s: TimeMixSpec):
        from ..csrc import ops
        return FixedState((s.hidden_size + ops.decay_state_floats(s.num_heads, s.dim, s.dim),))

    def __init__(self, s: TimeMixSpec, weights: dict, ctx):
        from ..csrc import ops
        if s.num_heads <= 0 or s.dim <= 0 or s.decay_rank <= 0:
            raise ValueError(f"time mix: {s.num_heads} heads of {s.dim}, decay rank {s.decay_rank}")
        ops.decay_scan_shape(s.dim, s.dim)
        self.spec, self.dtype = s, ctx.dtype
        mu, r, k, v, g, w1, w2, w0, u, norm, o = s.names
        self.mu = _f32(torch.stack([weights[mu + m] for m in self.MIXES]), ctx)          # [5, W]
        self.r, self.k, self.v, self.g = (Linear(weights[n]) for n in (r, k, v, g))
        self.w1, self.w2 = Linear(weights[w1]), Linear(weights[w2])
        self.o_proj = Linear(weights[o])
        self.w0, self.u, self.norm = _f32(weights[w0], ctx), _f32(weights[u].reshape(-1), ctx), _f32(weights[norm], ctx)

    def __call__(self, h, step, cache):
        from ..csrc import ops
        s, ws, tag = self.spec, step.workspace, step.tag
        H, D, W = s.num_heads, s.dim, s.hidden_size
        T = h.shape[0]
        mixes = ws.get(tag + "tm.mix", (len(self.MIXES), T, W), self.dtype)
        ops.token_shift_multi(h, self.mu, cache.state, 0, step.cu_seqlens, step.state_slots, step.req_index, step.positions,
                              mixes)
        f32 = torch.float32
        r = self.r(mixes[0], step, "tm.r", out_dtype=f32)
        k = self.k(mixes[1], step, "tm.k", out_dtype=f32)
        v = self.v(mixes[2], step, "tm.v", out_dtype=f32)
        g = self.g(mixes[3], step, "tm.g")
        low = self.w1(mixes[4], step, "tm.w1")
        low = ops.unary_act(low, ws.get(tag + "tm.w1t", tuple(low.shape), low.dtype), "tanh")
        w = ops.decay_from_raw(self.w2(low, step, "tm.w2", out_dtype=f32), 0, self.w0)
        o = ws.get(tag + "tm.o", (T, H * D), f32)
        ops.decay_scan((r, 0), (k, 0), (v, 0), (w, 0), self.u, cache.state, W, step.cu_seqlens, step.state_slots, o, H, D, D)
        gated = ws.get(tag + "tm.gated", (T, H * D), self.dtype)
        ops.gate_norm(o, g, 0, "silu", False, self.norm, s.eps, gated, D)
        return self.o_proj(gated, step, "tm.out")
