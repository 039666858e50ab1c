"""Latent attention: keys and values of every head are expanded from ONE cached row per token.

    c_q = rmsnorm(W_dq h) * w_q        q_h = W_uq[h] c_q                      (dim numbers a head)
    c   = rmsnorm(W_dkv h) * w_kv      k_h = W_uk[h] c,  v_h = W_uv[h] c      (c: kv_rank numbers, the cached row)
    p   = softmax_j(scale * q_h . k_j,h  [, sink_h])  over the window;   out = W_o concat_h(sum_j p_j v_j,h)

Only c is kept, so the attention runs in the latent space: with a_h = W_uk[h]^T q_h (kv_rank numbers),
q_h . k_j,h = a_h . c_j, and sum_j p_j v_j,h = W_uv[h] (sum_j p_j c_j).  To the attention kernels this is
one shared key/value head of size kv_rank whose keys and values are the same rows (a `PagedLatent` cache
group: one plane of pages), with `num_heads` query heads on it; the two per-head maps around it are one
launch of small products each (`ops.gemm_heads`).  kv_rank is rounded up to the next multiple of 16 with
zero columns (rows of the cache and of both per-head matrices), which changes no sum.

Steps: [W_dq; W_dkv] h in one product -> both RMS norms and the cache write in one kernel -> W_uq ->
absorb W_uk -> attention over the latent pages (window, optional sink) -> expand by W_uv -> W_o.
A sink is a learned number per head that joins the softmax denominator as exp(sink_h): no key, no
value, not scaled.

A position encoding, when the description has one (`rot_dim` > 0), lives in a part of its own: every query head has
rot_dim more features behind its dim, and W_dkv gives rot_dim more numbers per token that are not normed, one key
part for all heads; both are rotated by the position and the score is scale * (q . k + q_rot . k_rot).  The cached
row is then [c | k_rot]; the query the kernels see is [a_h | q_rot] (the per-head matrix of the absorb step is
[[W_uk^T, 0], [0, I]]: the identity block hands the rotated part through exactly), and the expand step reads the
first kv_rank columns of the attention's result alone (zero columns in the per-head matrix).
An output gate (`gate`) multiplies the concatenated heads by sigmoid(W_g h); W_g is stacked under the two
down-projections, so it costs no product of its own.
"""
from __future__ import annotations

from collections import namedtuple

import torch

from ..cache.spec import PagedLatent
from .linear import Linear
from .registry import MIXERS
from .spec import LatentAttentionSpec, TensorDecl

MAX_LATENT = 256            # widest cached row the attention kernels take

# what the attention dispatcher reads of a mixer's description
# (shared_row: keys and values are the same rows of one shared head, which the choice of the decode chunks may use)
HeadLayout = namedtuple("HeadLayout", "num_heads num_kv_heads head_dim window shared_row", defaults=(False,))


def padded_rank(kv_rank: int) -> int:
    return -(-kv_rank // 16) * 16


def check_latent_sizes(spec: LatentAttentionSpec):
    for name in ("hidden_size", "num_heads", "dim", "vdim", "q_rank", "kv_rank"):
        if getattr(spec, name) <= 0:
            raise ValueError(f"latent attention: {name} must be positive, got {getattr(spec, name)}")
    if spec.rot_dim < 0 or (spec.rot_dim > 0) != (spec.position is not None):
        raise ValueError("latent attention: a rotated part (rot_dim) and a position encoding come together")
    if spec.position is not None and (spec.position.dim > spec.rot_dim or spec.position.dim % 2):
        raise ValueError(f"latent attention: {spec.position.dim} rotated features in a part of {spec.rot_dim}")
    if padded_rank(spec.kv_rank + spec.rot_dim) > MAX_LATENT:
        raise ValueError(f"latent attention: kv_rank {spec.kv_rank} + rot_dim {spec.rot_dim} is beyond the {MAX_LATENT} numbers "
                         f"a cached row may hold")
    if spec.window is not None and spec.window <= 0:
        raise ValueError(f"window {spec.window} must be positive (None reads every earlier key)")


@MIXERS.register("latent_attention")
class LatentAttention:
    graph_safe = True

    @staticmethod
    def declare(spec: LatentAttentionSpec) -> dict:
        dq, dqn, uq, dkv, dkvn, uk, uv, o, sink = spec.names
        H = spec.num_heads
        d = {dq: TensorDecl((spec.q_rank, spec.hidden_size)), dqn: TensorDecl((spec.q_rank,), init="norm"),
             uq: TensorDecl((H * (spec.dim + spec.rot_dim), spec.q_rank)),
             dkv: TensorDecl((spec.kv_rank + spec.rot_dim, spec.hidden_size)), dkvn: TensorDecl((spec.kv_rank,), init="norm"),
             uk: TensorDecl((H * spec.dim, spec.kv_rank)), uv: TensorDecl((H * spec.vdim, spec.kv_rank)),
             o: TensorDecl((spec.hidden_size, H * spec.vdim))}
        if spec.sink:
            d[sink] = TensorDecl((H,))
        if spec.gate is not None:
            d[spec.gate] = TensorDecl((H * spec.vdim, spec.hidden_size))
        return d

    @staticmethod
    def cache_need(spec: LatentAttentionSpec):
        return PagedLatent(padded_rank(spec.kv_rank + spec.rot_dim), spec.window)

    def __init__(self, spec: LatentAttentionSpec, weights: dict, ctx):
        check_latent_sizes(spec)
        self.spec = spec
        self.dtype = ctx.dtype
        dq, dqn, uq, dkv, dkvn, uk, uv, o, sink = spec.names
        H, D, V, R, P = spec.num_heads, spec.dim, spec.vdim, spec.kv_rank, spec.rot_dim
        self.rank = padded_rank(R + P)
        down = [weights[dq], weights[dkv]] + ([weights[spec.gate]] if spec.gate is not None else [])
        self.down = Linear(torch.cat(down, dim=0).contiguous())
        self.gate_col = spec.q_rank + R + P if spec.gate is not None else None
        self.rotary = None
        if spec.position is not None:
            from .registry import POSITIONS
            table = POSITIONS.get(spec.position.kind)(spec.position, {}, ctx)
            self.rotary = table.fused_rotary()           # (inv_freq, rotated features)
            if self.rotary is None:
                raise TypeError(f"position kind {spec.position.kind!r} offers no table of inverse frequencies")
        self.q_norm = weights[dqn].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.kv_norm = weights[dkvn].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.uq = Linear(weights[uq])
        # a_h = W_uk[h]^T q_h: per head a [rank, dim] matrix (the transpose, rows beyond kv_rank zero)
        wk = weights[uk].view(H, D, R)
        absorb = torch.zeros((H, self.rank, D + P), dtype=wk.dtype, device=wk.device)
        absorb[:, :R, :D] = wk.transpose(1, 2)
        if P:                                             # the rotated part passes through: an identity block
            absorb[:, R:R + P, D:] = torch.eye(P, dtype=wk.dtype, device=wk.device)
        self.absorb = absorb.contiguous()
        # v_h = W_uv[h] (sum p c): per head [vdim, rank] (columns beyond kv_rank zero)
        wv = weights[uv].view(H, V, R)
        expand = torch.zeros((H, V, self.rank), dtype=wv.dtype, device=wv.device)
        expand[:, :, :R] = wv
        self.expand = expand.contiguous()
        self.o = Linear(weights[o])
        self.sinks = weights[sink].to(device=ctx.device, dtype=torch.float32).contiguous() if spec.sink else None
        self.scale = spec.scale if spec.scale is not None else D ** -0.5
        self.layout = HeadLayout(H, 1, self.rank, spec.window, True)

    def __call__(self, h, step, cache):
        from ..csrc import ops
        from . import attention_dispatch
        s, ws, tag = self.spec, step.workspace, step.tag
        T = h.shape[0]
        H = s.num_heads
        group = step.groups[cache.group]
        proj = self.down(h, step, "latent.down")
        cq = ws.get(tag + "latent.cq", (T, s.q_rank), self.dtype)
        ops.latent_norm_write(proj, s.q_rank, s.kv_rank, self.q_norm, self.kv_norm, s.eps, cq,
                              group.slots if cache.writes else None, cache.k, step.err, rot_dim=s.rot_dim,
                              rotary=self.rotary, positions=step.positions)
        q = self.uq(cq, step, "latent.q")
        if self.rotary is not None and self.rotary[1] > 0:
            ops.rope_heads(q, s.dim, s.dim + s.rot_dim, H, self.rotary[0], self.rotary[1], step.positions)
        qa = ops.gemm_heads(q, self.absorb, ws.get(tag + "latent.qa", (T, H * self.rank), self.dtype))
        ctx = ws.get(tag + "latent.ctx", (T, H * self.rank), self.dtype)
        attention_dispatch.run(qa, ctx, cache, group, step, self.layout, self.scale, sinks=self.sinks)
        v = ops.gemm_heads(ctx, self.expand, ws.get(tag + "latent.v", (T, H * s.vdim), self.dtype))
        if self.gate_col is not None:
            ops.sigmoid_gate(v, proj, self.gate_col)
        return self.o(v, step, "latent.o")
