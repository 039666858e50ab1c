"""A mixer behind a token shift: its input row is mixed with the row of the token before,

    h_t <- h_t + (h_(t-1) - h_t) * mu        (element by element, float32; zeros before a sequence's first token)

where h_(t-1) is the input as it was before this replacement.  The wrapped mixer may be of any registered kind, with
its own tensors (under `inner_prefix`) and its own cache or state; the shift keeps one row of float32 per request (the
last input row it saw) in a state slot of its own, so a portion of a prompt, a continuation and a decoded token are
one case.  The part reads the float32 stream itself (`reads_stream`): the mix is made of the stream's full
precision and rounded once to the activation dtype.
"""
from __future__ import annotations

import torch

from ..cache.spec import FixedState, Several
from .base import CallCache, prefixed, sub_weights
from .registry import MIXERS
from .spec import TensorDecl, TokenShiftSpec


@MIXERS.register("token_shift")
class TokenShift:
    reads_stream = True        # the block hands it the float32 stream, not its rounding

    @staticmethod
    def declare(s: TokenShiftSpec) -> dict:
        d = {s.tensor: TensorDecl((s.hidden_size,), init="unit")}
        d.update(prefixed(MIXERS.get(s.inner.kind).declare(s.inner), s.inner_prefix))
        return d

    @staticmethod
    def cache_need(s: TokenShiftSpec):
        inner = MIXERS.get(s.inner.kind).cache_need(s.inner)
        own = FixedState((s.hidden_size,))
        if inner is None:
            return own
        return Several((own,) + (tuple(inner.parts) if isinstance(inner, Several) else (inner,)))

    def __init__(self, s: TokenShiftSpec, weights: dict, ctx):
        self.spec, self.dtype = s, ctx.dtype
        self.mu = weights[s.tensor].to(device=ctx.device, dtype=torch.float32).contiguous()
        cls = MIXERS.get(s.inner.kind)
        self.inner = cls(s.inner, sub_weights(weights, s.inner_prefix), ctx)
        need = cls.cache_need(s.inner)
        self._inner_parts = None if need is None else (len(need.parts) if isinstance(need, Several) else 0)
        self.graph_safe = bool(getattr(self.inner, "graph_safe", False))

    def take_out_bias(self):
        """The bias of the wrapped mixer's last product, if that mixer can leave it to the caller (else None)."""
        take = getattr(self.inner, "take_out_bias", None)
        return take() if take is not None else None

    def __call__(self, x, step, cache):
        """x: the float32 stream [T, hidden]."""
        from ..csrc import ops
        if self._inner_parts is None:
            own, inner = cache, None
        elif self._inner_parts == 0:
            own, inner = cache.parts[0], cache.parts[1]
        else:
            own, inner = cache.parts[0], CallCache(parts=cache.parts[1:])
        h = step.workspace.get(step.tag + "shift.h", tuple(x.shape), self.dtype)
        ops.token_shift(x, self.mu, own.state, 0, step.cu_seqlens, step.state_slots, step.req_index, step.positions, h)
        return self.inner(h, step, inner)
