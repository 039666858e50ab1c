"""Routed experts: every token is sent through `top` of `num_experts` small gated feed-forwards.

    z = W_r h (float32), score = sigmoid(z) or softmax(z); the `top` largest scores choose the experts
    out = sum_e E_e(w_e h)            (`scale_input`: the weight multiplies the expert's INPUT)
       or sum_e w_e E_e(h)
    E(y) = W_down (f(W_gate y, W_up y)),  f as in `ops.gated_act` (for "capped_swish":
           g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(alpha g') (u' + up_shift))
       or, for an expert without a gate (`gated` False), W_down f(W_up y) with f of `ops.UNARY_ACTIVATIONS`

No host decision anywhere, so a step stays a fixed sequence of launches (and a decode step a CUDA graph):
the router kernel writes ids and weights, one block sorts the (token, choice) pairs by expert into tiles
of rows (every expert's rows padded to whole tiles), a gather kernel lays the (scaled) inputs out in that
order, two grouped products with the activation between them run over the tiles, each tile with its
expert's matrices, and a last kernel sums a token's results in the order of its choices.  A row's
arithmetic does not depend on where it was sorted to, so logits do not depend on the batch.

In bfloat16 (sizes permitting) the first product does the work of its neighbours: it reads the tokens'
rows through the sorted index (no sorted copy), applies the expert weight to its float32 sums
(W (s h) = s (W h)) and the activation to its own tile (gate and up rows interleaved in blocks of 8), so
the step is router, sort, two products and the sum: five launches instead of seven.

Options of the router (`ops.moe_route`): a bias on the logits, a bias on the scores that only the choice sees, groups of
neighbouring experts that count by their largest or by the sum of their largest choice values, renormalised weights.
A `shared` feed-forward (any registered kind) runs for every token beside the experts and is added to their sum.
"""
from __future__ import annotations

import torch

from .base import prefixed, sub_weights
from .registry import FEED_FORWARDS
from .spec import RoutedExpertsSpec, TensorDecl

SMALL_STEP_PAIRS = 64       # up to this many (token, choice) pairs the tiles hold 16 rows, else 64


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts:
    graph_safe = True

    @staticmethod
    def declare(spec: RoutedExpertsSpec) -> dict:
        gate, up, down = spec.names
        I, H = spec.intermediate_size, spec.hidden_size
        d = {spec.router: TensorDecl((spec.num_experts, H))}
        if spec.router_bias is not None:
            d[spec.router + spec.router_bias] = TensorDecl((spec.num_experts,))
        if spec.choice_bias is not None:
            d[spec.choice_bias] = TensorDecl((spec.num_experts,), init="unit")
        if spec.shared is not None:
            d.update(prefixed(FEED_FORWARDS.get(spec.shared.kind).declare(spec.shared), spec.shared_prefix))
        for e in range(spec.num_experts):
            p = spec.expert_prefix.format(e)
            d.update({p + up: TensorDecl((I, H)), p + down: TensorDecl((H, I))})
            if spec.gated:
                d[p + gate] = TensorDecl((I, H))
        return d

    def __init__(self, spec: RoutedExpertsSpec, weights: dict, ctx):
        from ..csrc import ops
        if not 0 < spec.top <= spec.num_experts:
            raise ValueError(f"routed experts: top {spec.top} of {spec.num_experts} experts")
        if spec.groups < 1 or spec.num_experts % spec.groups or not 1 <= spec.keep_groups <= spec.groups \
                or spec.keep_groups * (spec.num_experts // spec.groups) < spec.top:
            raise ValueError(f"routed experts: {spec.num_experts} experts in {spec.groups} groups of which {spec.keep_groups} "
                             f"are kept cannot offer {spec.top} choices")
        known = ops.ACTIVATIONS if spec.gated else ops.UNARY_ACTIVATIONS
        if spec.activation not in known or spec.score not in ops.ROUTER_SCORES:
            raise ValueError(f"routed experts: activation {spec.activation!r} ({'with' if spec.gated else 'without'} a gate) / "
                             f"score {spec.score!r} not known")
        self.spec = spec
        self.dtype = ctx.dtype
        gate, up, down = spec.names
        E = spec.num_experts
        names = [spec.expert_prefix.format(e) for e in range(E)]
        # The router's logits are float32 sums whatever the model's dtype.  A router stored in bfloat16 beside
        # bfloat16 rows stays as it is: the products of two bfloat16 numbers are exact in float32, so the tensor
        # cores add the same numbers as a float32 product of the widened matrix would.
        r = weights[spec.router]
        keep = r.dtype == torch.bfloat16 and ctx.dtype == torch.bfloat16 and spec.hidden_size % 8 == 0
        self.router = r.contiguous() if keep else r.to(device=ctx.device, dtype=torch.float32).contiguous()
        self.router_bias = None
        if spec.router_bias is not None:
            self.router_bias = weights[spec.router + spec.router_bias].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.choice_bias = None
        if spec.choice_bias is not None:
            self.choice_bias = weights[spec.choice_bias].to(device=ctx.device, dtype=torch.float32).contiguous()
        if spec.group_top < 1 or spec.renorm_eps < 0:
            raise ValueError(f"routed experts: group_top {spec.group_top}, renorm_eps {spec.renorm_eps}")
        # one more feed-forward that every token passes, added to the experts' sum
        self.shared = None
        if spec.shared is not None:
            self.shared = FEED_FORWARDS.get(spec.shared.kind)(spec.shared, sub_weights(weights, spec.shared_prefix), ctx)
            self.graph_safe = bool(getattr(self.shared, "graph_safe", False))
        I, H = spec.intermediate_size, spec.hidden_size
        # columns of the first product: gate and up rows, or the up rows alone
        self.first_n = 2 * I if spec.gated else I
        self.fused = I % 8 == 0 and ops.gemm_grouped_fused_ok(ctx.dtype, H, self.first_n, spec.activation)
        if not spec.gated:
            self.gate_up = torch.stack([weights[p + up] for p in names]).contiguous()           # [E, I, H]
        elif self.fused:
            # per expert blocks of 8 gate rows followed by their 8 up rows: [E, 2I, H]
            self.gate_up = torch.stack([torch.stack([weights[p + gate].view(I // 8, 8, H), weights[p + up].view(I // 8, 8, H)],
                                                    dim=1).reshape(2 * I, H) for p in names]).contiguous()
        else:
            # per expert [gate rows; up rows], stacked over experts: [E, 2I, H]
            self.gate_up = torch.stack([torch.cat([weights[p + gate], weights[p + up]], dim=0) for p in names]).contiguous()
        self.down = torch.stack([weights[p + down] for p in names]).contiguous()          # [E, H, I]

    def __call__(self, h, step):
        from ..csrc import ops
        s, ws, tag = self.spec, step.workspace, step.tag
        T, E, top, I, H = h.shape[0], s.num_experts, s.top, s.intermediate_size, s.hidden_size
        pairs = T * top
        big = self.fused and ops.gemm_grouped_tc5_ok(self.dtype, pairs, E, H) and I % 8 == 0
        # tiles of 16 rows while an expert gets 16 rows or fewer on average (decoding: the products are then bound
        # by the experts' weights, and taller tiles would spend their time on rows of padding)
        bm = ops.TC5_GROUPED_TILE if big else (16 if pairs <= max(SMALL_STEP_PAIRS, 16 * E) else 64)
        cap = ops.moe_sorted_rows(pairs, E, bm)
        ids = ws.get(tag + "moe.ids", (T, top), torch.int32)
        weights = ws.get(tag + "moe.weights", (T, top), torch.float32)
        sorted_rows = ws.get(tag + "moe.sorted", (cap,), torch.int32)
        tile_group = ws.get(tag + "moe.tiles", (cap // bm,), torch.int32)
        place = ws.get(tag + "moe.place", (pairs,), torch.int32)
        logits = ws.get(tag + "moe.logits", (ops.router_slices(H), T, E), torch.float32)
        ops.moe_route(h, self.router, top, ids, weights, logits, s.score, s.renormalize, s.groups, s.keep_groups,
                      bias=self.router_bias, choice_bias=self.choice_bias, group_top=s.group_top, renorm_eps=s.renorm_eps)
        ops.moe_align(ids, E, bm, sorted_rows, tile_group, place)
        act = ws.get(tag + "moe.act", (cap, I), self.dtype)
        if big:
            # many rows: both products on the tcgen05 tensor cores, from a sorted copy of the tokens' rows
            rows = ops.moe_gather(h, sorted_rows, weights, top, ws.get(tag + "moe.rows", (cap, H), self.dtype), False)
            ops.gemm_grouped_tc5(rows, self.gate_up, act, tile_group, step.err, sorted_rows,
                                 weights if s.scale_input else None, s.activation, s.alpha, s.limit, s.up_shift)
            res = ops.gemm_grouped_tc5(act, self.down, ws.get(tag + "moe.down", (cap, H), self.dtype), tile_group, step.err)
            return ops.moe_combine(res, place, weights, top, ws.get(tag + "moe.out", (T, H), self.dtype), not s.scale_input,
                                   add=self._shared(h, step))
        if self.fused:
            ops.gemm_grouped_fused(h, self.gate_up, act, tile_group, bm, sorted_rows, top,
                                   weights if s.scale_input else None, s.activation, s.alpha, s.limit, s.up_shift)
        else:
            rows = ops.moe_gather(h, sorted_rows, weights, top, ws.get(tag + "moe.rows", (cap, H), self.dtype), s.scale_input)
            gu = ops.gemm_grouped(rows, self.gate_up, ws.get(tag + "moe.gate_up", (cap, self.first_n), self.dtype), tile_group, bm)
            if s.gated:
                ops.gated_act(gu, act, s.activation, 0, s.alpha, s.limit, s.up_shift)
            else:
                ops.unary_act(gu, act, s.activation)
        res = ops.gemm_grouped(act, self.down, ws.get(tag + "moe.down", (cap, H), self.dtype), tile_group, bm)
        out = ws.get(tag + "moe.out", (T, H), self.dtype)
        return ops.moe_combine(res, place, weights, top, out, not s.scale_input, add=self._shared(h, step))

    def _shared(self, h, step):
        """The shared feed-forward's rows (None without one): the kernel that sums a token's choices adds them last."""
        return None if self.shared is None else self.shared(h, step)
