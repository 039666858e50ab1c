"""Attention behind short convolutions, with the keys as values and a choice of weighting.

    [q | k | g] = W h             one stacked product: queries, keys, one gate logit per head
    q, k <- causal convolution over time, per channel, of the product plus its bias (`ops.short_conv` adds the bias
            as it reads; the last taps - 1 projected rows of a request are part of its state)
    v = k;  q, k <- row / rms(whole row) * weight;  rotation of the first features of every head;  q kept, k and v
            written to the pages (steps of single tokens: `ops.conv_rows_norm_rope_write`, one kernel with the
            convolution; other steps: `ops.short_conv`, then `ops.rows_norm_rope_write`; the same bits)
    o_h = sum over the visible keys j of w_j v_j,  w_j = sigmoid(scale q_h.k_j + pb[h])  (or a softmax), keys cut by
            `chunk` and `window`, times sigmoid(g_h)     (the framework's attention kernels with their options)
    out = W_o o (+ b)

A request keeps pages of keys and values (`PagedKV`, with the chunk as the rule by which pages are given back) and a
row of float32 state: the convolution's last inputs.  Heads whose size is no multiple of 16 are padded with zero
features where the kernels see them (cache rows, q, the columns of W_o); the whole-row norm divides by the true count.
What the design computes in float32 (the convolution's sums, the norms, angles, scores, weights, the gate) is float32
whatever the model's dtype.
"""
from __future__ import annotations

import torch

from ..cache.spec import FixedState, PagedKV, Several
from .linear import Linear
from .registry import MIXERS, POSITIONS
from .spec import ConvAttentionSpec, TensorDecl

MAX_HEAD_DIM = 256


@MIXERS.register("conv_attention")
class ConvAttention:
    graph_safe = True

    @staticmethod
    def _sizes(s: ConvAttentionSpec):
        return s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim, -(-s.head_dim // 16) * 16

    @staticmethod
    def declare(s: ConvAttentionSpec) -> dict:
        Cq, Ck, _ = ConvAttention._sizes(s)
        q, k, g, o, pb = s.names
        d = {q: TensorDecl((Cq, s.hidden_size)), k: TensorDecl((Ck, s.hidden_size)), o: TensorDecl((s.hidden_size, Cq)),
             q + s.conv_suffix: TensorDecl((Cq, s.conv), init="conv"), k + s.conv_suffix: TensorDecl((Ck, s.conv), init="conv"),
             q + s.norm_suffix: TensorDecl((Cq,), init="norm"), k + s.norm_suffix: TensorDecl((Ck,), init="norm")}
        if s.bias:
            d.update({q + s.bias_suffix: TensorDecl((Cq,)), k + s.bias_suffix: TensorDecl((Ck,))})
        if s.out_bias:
            d[o + s.bias_suffix] = TensorDecl((s.hidden_size,))
        if s.gate:
            d[g] = TensorDecl((s.num_heads, s.hidden_size))
        if s.head_bias:
            d[pb] = TensorDecl((s.num_heads,), init="unit")
        return d

    @staticmethod
    def cache_need(s: ConvAttentionSpec):
        Cq, Ck, pd = ConvAttention._sizes(s)
        pages = PagedKV(s.num_kv_heads, pd, s.window, s.chunk)
        # (one tap keeps nothing; the state row then is a single unused number, so that every layer is laid out alike)
        return Several((pages, FixedState((max((s.conv - 1) * (Cq + Ck), 1),))))

    def __init__(self, s: ConvAttentionSpec, weights: dict, ctx):
        from ..csrc import ops
        Cq, Ck, pd = self._sizes(s)
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_kv_heads} kv heads do not divide {s.num_heads} query heads")
        if not 0 < s.head_dim <= MAX_HEAD_DIM:
            raise ValueError(f"head_dim {s.head_dim}: the attention kernels take head sizes up to {MAX_HEAD_DIM}")
        if s.conv < 1 or (s.chunk is not None and s.chunk <= 0) or (s.window is not None and s.window <= 0):
            raise ValueError(f"conv attention: {s.conv} taps, chunk {s.chunk}, window {s.window}")
        if s.weighting not in ops.WEIGHTINGS or (s.head_bias and s.weighting != "sigmoid"):
            raise ValueError(f"conv attention: weighting {s.weighting!r} (a bias per head belongs to the sigmoid)")
        self.spec, self.dtype = s, ctx.dtype
        self.Cq, self.Ck, self.pd = Cq, Ck, pd
        q, k, g, o, pb = s.names
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()
        stack = [weights[q], weights[k]] + ([weights[g]] if s.gate else [])
        # the biases of q and k are added by the convolution's kernel as it reads the product (the gate has none)
        self.in_bias = f32(torch.cat([weights[q + s.bias_suffix].float(), weights[k + s.bias_suffix].float()])) if s.bias else None
        # the stacked rows are padded to a multiple of 8, so that every row of the product starts on 16 bytes
        width = Cq + Ck + (s.num_heads if s.gate else 0)
        self.width = -(-width // 8) * 8
        w = torch.cat(stack, dim=0)
        if self.width != width:
            w = torch.cat([w, torch.zeros((self.width - width, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
        self.in_proj = Linear(w.contiguous())
        wo = weights[o]
        if pd != s.head_dim:                       # zero columns for the padded features of every head
            wp = torch.zeros((wo.shape[0], s.num_heads, pd), dtype=wo.dtype, device=wo.device)
            wp[:, :, :s.head_dim] = wo.reshape(wo.shape[0], s.num_heads, s.head_dim)
            wo = wp.reshape(wo.shape[0], s.num_heads * pd)
        self.o_proj = Linear(wo.contiguous(), weights[o + s.bias_suffix].float() if s.out_bias else None)
        self.taps = f32(torch.cat([weights[q + s.conv_suffix], weights[k + s.conv_suffix]], dim=0))
        self.q_norm, self.k_norm = f32(weights[q + s.norm_suffix]), f32(weights[k + s.norm_suffix])
        self.head_bias = f32(weights[pb]) if s.head_bias else None
        self.inv_freq, self.rot = None, 0
        if s.position is not None:
            table = POSITIONS.get(s.position.kind)(s.position, {}, ctx)
            fused = table.fused_rotary()
            if fused is None or getattr(s.position, "interleaved", False):
                raise TypeError("conv attention rotates inside its own kernel: it takes the rotate-half rotary table")
            self.inv_freq, self.rot = fused
        self.scale = s.scale if s.scale is not None else s.head_dim ** -0.5
        # what the attention kernels are told: heads of the padded size
        import dataclasses
        self.kernel_spec = dataclasses.replace(s, head_dim=pd)

    def take_out_bias(self):
        """Hands the output projection's bias to the caller (a block whose norm reads the product anyway); the part
        then returns W_o o alone."""
        bias, self.o_proj.bias = self.o_proj.bias, None
        return bias

    def __call__(self, h, step, cache):
        from ..csrc import ops
        from . import attention_dispatch
        s, ws, tag = self.spec, step.workspace, step.tag
        pages, conv_state = cache.parts[0], cache.parts[1]
        group = step.groups[pages.group]
        T = h.shape[0]
        proj = self.in_proj(h, step, "ca.in")
        C = self.Cq + self.Ck
        q = ws.get(tag + "ca.q", (T, s.num_heads * self.pd), self.dtype)
        slots = group.slots if pages.writes else None
        if step.max_query_len == 1 and ops.conv_rows_fused_ok(C):
            # single tokens: convolution, norms, rotation and the cache rows in one launch, the convolved row stays on
            # the chip.  (Portions of prompts go through the two kernels, the same bits: the convolution's kernel
            # shares a channel's taps among 64 tokens, the one launch would fetch them for every token.)
            ops.conv_rows_norm_rope_write(proj, self.taps, self.in_bias, conv_state.state, 0, step.cu_seqlens, step.state_slots,
                                          step.req_index, step.max_query_len, step.positions, slots, self.q_norm, self.k_norm,
                                          s.eps, self.inv_freq, self.rot, q, pages.k, pages.v, s.num_heads, s.num_kv_heads,
                                          s.head_dim, step.err, padded_head_dim=self.pd)
        else:
            qk = ws.get(tag + "ca.qk", (T, C), torch.float32)
            ops.short_conv(proj, 0, C, self.taps, None, conv_state.state, 0, step.cu_seqlens, step.state_slots, qk,
                           act=False, longest=step.max_query_len, in_bias=self.in_bias)
            ops.rows_norm_rope_write(qk, step.positions, slots, self.q_norm, self.k_norm, s.eps, self.inv_freq, self.rot, q,
                                     pages.k, pages.v, s.num_heads, s.num_kv_heads, s.head_dim, step.err, padded_head_dim=self.pd)
        out = ws.get(tag + "ca.out", (T, s.num_heads * self.pd), self.dtype)
        gate = proj[:, C:C + s.num_heads] if s.gate else None
        attention_dispatch.run(q, out, pages, group, step, self.kernel_spec, self.scale, weighting=s.weighting,
                               chunk=s.chunk, head_bias=self.head_bias, gate=gate)
        return self.o_proj(out, step, "ca.o")
