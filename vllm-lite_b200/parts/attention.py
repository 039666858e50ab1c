"""Grouped-query attention with per-head norm of q and k before the rotation.

project -> head norm -> rotation -> cache write -> attention over the pages ->
output projection (crates/model/src/components/attention/rope_gqa.rs:261-305 of
the reference).  The three projections are bound by their own tensor names and
stacked at load time into one [q | k | v] matrix, which keeps every output row's
arithmetic unchanged.  A prompt portion, a continuation and a decoded token are
the same case: every token's key and value are written first, then each query
reads positions 0..its own (or its window) from the pages.
"""
from __future__ import annotations

import torch

from ..cache.spec import PagedKV
from .base import sub_weights
from .linear import Linear
from .registry import MIXERS, NORMS, POSITIONS
from .spec import AttentionSpec, TensorDecl


MAX_HEAD_DIM = 256


def check_attention_sizes(spec: AttentionSpec):
    """What the attention kernels take, checked when a model is planned or built instead of in its first
    step: head sizes in steps of 16 up to 256, and kv heads that divide the query heads."""
    if spec.num_heads <= 0 or spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
        raise ValueError(f"{spec.num_kv_heads} kv heads do not divide {spec.num_heads} query heads")
    if spec.head_dim % 16 or not 16 <= spec.head_dim <= MAX_HEAD_DIM:
        raise ValueError(f"head_dim {spec.head_dim}: the attention kernels take multiples of 16 from 16 to {MAX_HEAD_DIM}")
    if spec.qk_norm is not None and spec.qk_norm.size != spec.head_dim:
        raise ValueError("the head norm runs over head_dim")
    if spec.window is not None and spec.window <= 0:
        raise ValueError(f"window {spec.window} must be positive (None reads every earlier key)")


def _pad_heads(w, heads, size, padded):
    """Rows (or entries) of `heads` heads of `size` each, every head padded with zeros to `padded`."""
    if size == padded:
        return w
    shape = (heads, size) + tuple(w.shape[1:])
    out = torch.zeros((heads, padded) + tuple(w.shape[1:]), dtype=w.dtype, device=w.device)
    out[:, :size] = w.reshape(shape)
    return out.reshape((heads * padded,) + tuple(w.shape[1:]))


def _pair_order(head_dim, rotary_dim, device):
    """The order of a head's features that puts neighbours (2i, 2i+1) of the first rotary_dim features at (i, i + rotary_dim/2):
    q.k does not change when q and k are permuted alike, so an interleaved rotation is the rotate-half one on permuted heads."""
    idx = torch.arange(head_dim, device=device)
    idx[:rotary_dim] = torch.cat([torch.arange(0, rotary_dim, 2, device=device), torch.arange(1, rotary_dim, 2, device=device)])
    return idx


@MIXERS.register("gqa_attention")
class GqaAttention:
    graph_safe = True          # launches only stream-ordered kernels: a step can be captured in a CUDA graph

    @staticmethod
    def declare(spec: AttentionSpec) -> dict:
        vd = spec.v_head_dim or spec.head_dim
        qd, kd, vdim = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.num_kv_heads * vd
        q, k, v, o = spec.names
        qb, kb, vb, ob = spec.bias_names
        d = {q: TensorDecl((qd, spec.hidden_size)), k: TensorDecl((kd, spec.hidden_size)),
             v: TensorDecl((vdim, spec.hidden_size)), o: TensorDecl((spec.hidden_size, spec.num_heads * vd))}
        if spec.bias:
            d.update({qb: TensorDecl((qd,)), kb: TensorDecl((kd,)), vb: TensorDecl((vdim,))})
        if spec.out_bias:
            d[ob] = TensorDecl((spec.hidden_size,))
        if spec.distance_bias is not None:
            d.update({spec.distance_bias[0]: TensorDecl((spec.num_heads,), init="unit"),
                      spec.distance_bias[1]: TensorDecl((spec.num_heads,), init="rate")})
        if spec.gate is not None:
            d[spec.gate] = TensorDecl((spec.num_heads * vd, spec.hidden_size))
        if spec.qk_norm is not None:
            for side in spec.norm_prefixes:
                for name, decl in NORMS.get(spec.qk_norm.kind).declare(spec.qk_norm).items():
                    d[side + name] = decl
        if spec.position is not None:
            for name, decl in POSITIONS.get(spec.position.kind).declare(spec.position).items():
                d["rotary." + name] = decl
        return d

    @staticmethod
    def padded_head_dim(spec: AttentionSpec) -> int:
        """The head size the kernels see: key and value heads of one size, a multiple of 16.  Heads of other sizes are
        padded with zero features when the weights are bound (zero rows of q, k, v, zero columns of o), which changes no
        score and no output; the head norm's mean then runs over the padded size and is set right by its weight and eps."""
        return -(-max(spec.head_dim, spec.v_head_dim or spec.head_dim) // 16) * 16

    @staticmethod
    def cache_need(spec: AttentionSpec):
        return PagedKV(spec.num_kv_heads, GqaAttention.padded_head_dim(spec), spec.window)

    def __init__(self, spec: AttentionSpec, weights: dict, ctx):
        import dataclasses
        hd, vd, pd = spec.head_dim, spec.v_head_dim or spec.head_dim, self.padded_head_dim(spec)
        self.true_spec = spec
        # an attention with options on its scores or around them runs its own sequence of kernels (`_call_with_options`);
        # with a query factor or a value norm the head work is a kernel of its own, which knows the heads' true sizes
        self.own_head_work = spec.q_temp is not None or spec.v_norm is not None
        self.with_options = bool(self.own_head_work or spec.softcap or spec.distance_bias is not None or spec.unit_sink
                                 or spec.gate is not None)
        if self.own_head_work and (spec.position is not None or spec.bias or
                                   (spec.qk_norm is not None and spec.qk_norm.kind != "rms_norm")):
            raise ValueError("a query factor or a value norm goes with RMS head norms, no rotation and no projection bias")
        # what the kernels see: heads of the padded size (scale and window as given)
        spec = dataclasses.replace(spec, head_dim=pd, v_head_dim=None,
                                   scale=spec.scale if spec.scale is not None else hd ** -0.5,
                                   qk_norm=None if spec.qk_norm is None else dataclasses.replace(spec.qk_norm, size=pd))
        check_attention_sizes(spec)
        self.spec = spec
        self.dtype = ctx.dtype
        nq, nkv = spec.num_heads, spec.num_kv_heads
        qn, kn, vn, on = spec.names
        wq, wk, wv, wo = weights[qn], weights[kn], weights[vn], weights[on]
        biases = [weights[n].float() for n in spec.bias_names[:3]] if spec.bias else None
        order = None
        rot = self.true_spec.position
        if rot is not None and getattr(rot, "interleaved", False):
            order = _pair_order(hd, rot.dim, wq.device)
            wq = wq.reshape(nq, hd, -1)[:, order].reshape(nq * hd, -1)
            wk = wk.reshape(nkv, hd, -1)[:, order].reshape(nkv * hd, -1)
            if biases is not None:
                biases[0] = biases[0].reshape(nq, hd)[:, order].reshape(-1)
                biases[1] = biases[1].reshape(nkv, hd)[:, order].reshape(-1)
        wq, wk, wv = _pad_heads(wq, nq, hd, pd), _pad_heads(wk, nkv, hd, pd), _pad_heads(wv, nkv, vd, pd)
        if vd != pd:
            wo = _pad_heads(wo.t().contiguous(), nq, vd, pd).t().contiguous()
        bias = None
        if biases is not None:
            bias = torch.cat([_pad_heads(biases[0], nq, hd, pd), _pad_heads(biases[1], nkv, hd, pd),
                              _pad_heads(biases[2], nkv, vd, pd)], dim=0)
        stacked = [wq, wk, wv]
        self.gate_col = None
        if spec.gate is not None:
            # the gate's rows follow the value heads' padding; sigmoid(0) times a padded zero stays zero
            stacked.append(_pad_heads(weights[spec.gate], nq, vd, pd))
            self.gate_col = (nq + 2 * nkv) * pd
            if bias is not None:
                bias = torch.cat([bias, torch.zeros(nq * pd, dtype=bias.dtype, device=bias.device)], dim=0)
        self.qkv_proj = Linear(torch.cat(stacked, dim=0).contiguous(), bias)
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()
        self.distance = None
        if spec.distance_bias is not None:
            self.distance = (f32(weights[spec.distance_bias[0]]), f32(weights[spec.distance_bias[1]]))
        self.sinks = torch.zeros(nq, dtype=torch.float32, device=ctx.device) if spec.unit_sink else None
        self.o_proj = Linear(wo.contiguous(), weights[spec.bias_names[3]].float() if spec.out_bias else None)
        self.q_norm = self.k_norm = None
        # The kernel that rotates and writes the cache also applies an RMS norm to every head.  A head norm
        # that says it is one (`fused_rms()` -> (weight, eps)) runs there; any other kind must change the
        # heads itself (`apply_heads`), and the kernel is then given no norm.
        self.fused_head_norm = None
        self.head_weights = (None, None)
        if spec.qk_norm is not None and self.own_head_work:
            # the head-work kernel divides by the mean over the true size itself: weights are padded, nothing else
            if spec.qk_norm.has_weight:
                tn = self.true_spec.qk_norm
                self.head_weights = tuple(_pad_heads(f32(sub_weights(weights, side)[tn.tensor]) + float(tn.offset), 1, hd, pd)
                                          for side in spec.norm_prefixes)
        elif spec.qk_norm is not None:
            cls = NORMS.get(spec.qk_norm.kind)
            true_norm = self.true_spec.qk_norm
            norms = []
            for side in spec.norm_prefixes:
                nw = dict(sub_weights(weights, side))
                if order is not None or pd != hd:
                    # the norm's weights follow their features; over a padded head sum(x^2) / pd stands for sum(x^2) / hd:
                    # x / sqrt(ss/hd + eps) = x sqrt(hd/pd) / sqrt(ss/pd + eps hd/pd)
                    for name, decl in cls.declare(true_norm).items():
                        if tuple(decl.shape) == (hd,):
                            w = nw[name].float()
                            w = w[order] if order is not None else w
                            nw[name] = _pad_heads(w * (hd / pd) ** 0.5, 1, hd, pd)
                norms.append(cls(dataclasses.replace(spec.qk_norm, eps=spec.qk_norm.eps * hd / pd), nw, ctx))
            self.q_norm, self.k_norm = norms
            if hasattr(self.q_norm, "fused_rms"):
                (qw, eps), (kw, _) = self.q_norm.fused_rms(), self.k_norm.fused_rms()
                self.fused_head_norm = (qw, kw, eps)
            elif pd != hd:
                raise TypeError(f"norm kind {spec.qk_norm.kind!r} cannot norm heads that are padded from {hd} to {pd} features")
            elif not hasattr(self.q_norm, "apply_heads"):
                raise TypeError(f"norm kind {spec.qk_norm.kind!r} cannot serve as a head norm: it offers neither "
                                f"fused_rms() nor apply_heads(qkv, first_head, num_heads, head_dim, step)")
        self.position = None
        if spec.position is not None:
            pos = dataclasses.replace(spec.position, head_dim=pd, rotary_dim=spec.position.dim, interleaved=False) \
                if hasattr(spec.position, "rotary_dim") else spec.position
            self.position = POSITIONS.get(pos.kind)(pos, sub_weights(weights, "rotary."), ctx)
        self.scale = spec.scale

    def factors_norms(self, M) -> bool:
        """For M rows: the input may come as `ScaledRows` and the result may go `into_stream`."""
        return not self.with_options and self.qkv_proj.factors_norms(M) and self.o_proj.factors_norms(M)

    def _call_with_options(self, h, step, cache):
        """project (q | k | v | gate) -> head work -> attention with the score options -> output gate -> output projection."""
        from ..csrc import ops
        from . import attention_dispatch
        s, ts = self.spec, self.true_spec
        group = step.groups[cache.group]
        qkv = self.qkv_proj(h, step, "attn.qkv")
        slots = group.slots if cache.writes else None
        if self.own_head_work:
            qk = ts.qk_norm
            ops.head_norm_write(qkv, step.positions, slots, self.head_weights[0], self.head_weights[1],
                                qk.eps if qk is not None else 0.0, ts.head_dim if qk is not None else 0,
                                ts.v_norm is not None, ts.v_head_dim or ts.head_dim, ts.q_temp, cache.k, cache.v,
                                s.num_heads, s.num_kv_heads, s.head_dim, step.err, v_eps=ts.v_norm)
        else:
            fused = self.position.fused_rotary() if self.position is not None else None
            if self.position is not None and fused is None:
                self.position.apply(qkv, step.positions, s.num_heads, s.num_kv_heads, s.head_dim, step)
            inv_freq, rot = fused if fused is not None else (None, 0)
            if self.q_norm is not None and self.fused_head_norm is None:
                self.q_norm.apply_heads(qkv, 0, s.num_heads, s.head_dim, step)
                self.k_norm.apply_heads(qkv, s.num_heads, s.num_kv_heads, s.head_dim, step)
            qw, kw, eps = self.fused_head_norm if self.fused_head_norm is not None else (None, None, 0.0)
            ops.qk_norm_rope_write(qkv, step.positions, slots, qw, kw, eps, inv_freq, rot, cache.k, cache.v,
                                   s.num_heads, s.num_kv_heads, s.head_dim, step.err)
        out = step.workspace.get(step.tag + "attn.out", (qkv.shape[0], s.num_heads * s.head_dim), self.dtype)
        attention_dispatch.run(qkv, out, cache, group, step, s, self.scale, sinks=self.sinks, softcap=ts.softcap,
                               distance=self.distance)
        if self.gate_col is not None:
            ops.sigmoid_gate(out, qkv, self.gate_col)
        return self.o_proj(out, step, "attn.o")

    def __call__(self, h, step, cache, sink=None):
        from ..csrc import ops
        if self.with_options:
            return self._call_with_options(h, step, cache)
        s = self.spec
        group = step.groups[cache.group]
        qkv = self.qkv_proj(h, step, "attn.qkv")
        fused = self.position.fused_rotary() if self.position is not None else None
        if self.position is not None and fused is None:
            # an encoding that the fused kernel does not know acts on the q and k parts of qkv itself
            # (after the projections, before the head norm's kernel writes the cache)
            self.position.apply(qkv, step.positions, s.num_heads, s.num_kv_heads, s.head_dim, step)
        inv_freq, rot = fused if fused is not None else (None, 0)
        if self.q_norm is not None and self.fused_head_norm is None:
            # a head norm of a kind of its own: it edits the q heads and the k heads of qkv in place
            self.q_norm.apply_heads(qkv, 0, s.num_heads, s.head_dim, step)
            self.k_norm.apply_heads(qkv, s.num_heads, s.num_kv_heads, s.head_dim, step)
        qw, kw, eps = self.fused_head_norm if self.fused_head_norm is not None else (None, None, 0.0)
        slots = group.slots if cache.writes else None
        from . import attention_dispatch
        fold = None
        if attention_dispatch.folds_head_work(qkv.dtype, step, s, group, qkv.shape[0]):
            fold = (qw, kw, eps, inv_freq, rot, slots)          # the attention kernel does it on the way
        else:
            ops.qk_norm_rope_write(qkv, step.positions, slots, qw, kw, eps, inv_freq, rot, cache.k, cache.v,
                                   s.num_heads, s.num_kv_heads, s.head_dim, step.err)
        out = step.workspace.get(step.tag + "attn.out", (qkv.shape[0], s.num_heads * s.head_dim), self.dtype)
        attention_dispatch.run(qkv, out, cache, group, step, s, self.scale, fold=fold)
        if sink is not None:
            return self.o_proj.into_stream(out, sink, step, "attn.o")
        return self.o_proj(out, step, "attn.o")
