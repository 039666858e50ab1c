"""Two mixers side by side on the same input: out = left_scale * left(h) + right_scale * right(h).

Each side is a mixer of any registered kind with its own tensors (under `prefixes`) and its own cache or state: the
part asks for `Several` needs and hands each side its own `CallCache`.  A caller whose next step reads the sum anyway (a norm
on the mixer's output) may ask for the two results as they are (`as_pair`) and form the sum itself."""
from __future__ import annotations

from ..cache.spec import Several
from .base import prefixed, sub_weights
from .registry import MIXERS
from .spec import ParallelMixerSpec


@MIXERS.register("parallel_mixer")
class ParallelMixer:
    @staticmethod
    def declare(s: ParallelMixerSpec) -> dict:
        d = {}
        for side, prefix in zip((s.left, s.right), s.prefixes):
            d.update(prefixed(MIXERS.get(side.kind).declare(side), prefix))
        return d

    @staticmethod
    def cache_need(s: ParallelMixerSpec):
        needs = [MIXERS.get(side.kind).cache_need(side) for side in (s.left, s.right)]
        return Several(tuple(needs))

    def __init__(self, s: ParallelMixerSpec, weights: dict, ctx):
        self.spec, self.dtype = s, ctx.dtype
        self.left = MIXERS.get(s.left.kind)(s.left, sub_weights(weights, s.prefixes[0]), ctx)
        self.right = MIXERS.get(s.right.kind)(s.right, sub_weights(weights, s.prefixes[1]), ctx)
        self.graph_safe = bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    returns_pair = True        # __call__(as_pair=True) leaves the sum to the caller (`ScaledPair`)

    def __call__(self, h, step, cache, as_pair=False):
        from ..csrc import ops
        a = self.left(h, step, cache.parts[0])
        b = self.right(h, step, cache.parts[1])
        if as_pair:
            from .base import ScaledPair
            return ScaledPair(a, self.spec.left_scale, b, self.spec.right_scale)
        out = step.workspace.get(step.tag + "par.out", tuple(a.shape), self.dtype)
        return ops.scaled_sum(a, self.spec.left_scale, b, self.spec.right_scale, out)
