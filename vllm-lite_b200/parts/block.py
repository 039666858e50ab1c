"""Pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
(crates/model/src/components/decoder_block/mod.rs:66-85 of the reference).

The residual stream is float32.  A sub-layer's output is not added at once: it is
left pending and the next norm's kernel adds it while it reads the stream.  In a
step of few rows the norms' kernels are saved altogether where the neighbouring
parts can: the part before a norm adds its result into the stream itself and
leaves the norm's output in factored form (`ScaledRows`), which the part after
the norm takes as it is."""
from __future__ import annotations

import torch

from .base import StreamSink, prefixed, sub_weights
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from .spec import BlockSpec

@BLOCKS.register("pre_norm")
class PreNormBlock:
    @staticmethod
    def declare(spec: BlockSpec) -> dict:
        norm1, mixer, norm2, ffn = spec.names
        d = {}
        d.update(prefixed(NORMS.get(spec.norm1.kind).declare(spec.norm1), norm1))
        d.update(prefixed(MIXERS.get(spec.mixer.kind).declare(spec.mixer), mixer))
        d.update(prefixed(NORMS.get(spec.norm2.kind).declare(spec.norm2), norm2))
        d.update(prefixed(FEED_FORWARDS.get(spec.ffn.kind).declare(spec.ffn), ffn))
        return d

    @staticmethod
    def cache_need(spec: BlockSpec):
        return MIXERS.get(spec.mixer.kind).cache_need(spec.mixer)

    def __init__(self, spec: BlockSpec, weights: dict, ctx):
        self.spec = spec
        norm1, mixer, norm2, ffn = spec.names
        self.norm1 = NORMS.get(spec.norm1.kind)(spec.norm1, sub_weights(weights, norm1), ctx)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, sub_weights(weights, mixer), ctx)
        self.norm2 = NORMS.get(spec.norm2.kind)(spec.norm2, sub_weights(weights, norm2), ctx)
        self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn, sub_weights(weights, ffn), ctx)
        self.graph_safe = bool(getattr(self.mixer, "graph_safe", False) and getattr(self.ffn, "graph_safe", False))

    chains_norms = True        # __call__ takes `next_norm`

    def input_norm_for_fusion(self, M):
        """The first norm, if the block before may compute it for M rows in factored form."""
        ok = getattr(self.norm1, "factorable", False) and _factors(self.mixer, M)
        return self.norm1 if ok else None

    def __call__(self, residual, step, cache, next_norm=None):
        """next_norm: the norm that will read the stream after this block, when its reader can take
        the factored form (`input_norm_for_fusion` of the next block)."""
        M = step.num_tokens
        residual.cast = None                                      # this block's kernels write x without it
        if residual.normed is not None and residual.normed_for is self.norm1:
            h = residual.normed                                   # left by the block before
        else:
            h = self.norm1(residual.x, residual.pending, step, tag="norm1")
        residual.pending = residual.normed = residual.normed_for = None
        if _factors(self.mixer, M) and getattr(self.norm2, "factorable", False) and _factors(self.ffn, M):
            h = self.mixer(h, step, cache, sink=_sink(residual, self.norm2))
        else:
            a = self.mixer(h, step, cache)
            h = self.norm2(residual.x, a, step, tag="norm2")
        if next_norm is not None and _factors(self.ffn, M):
            residual.normed = self.ffn(h, step, sink=_sink(residual, next_norm))
            residual.normed_for = next_norm
        else:
            residual.pending = self.ffn(h, step)


def _factors(part, M) -> bool:
    f = getattr(part, "factors_norms", None)
    return bool(f and f(M))


def _sink(residual, norm) -> StreamSink:
    return StreamSink(residual.x, norm.weight, norm.spec.eps, norm.spec.size)


@BLOCKS.register("post_norm")
class PostNormBlock:
    """x += m norm1(mixer(x)); x += m norm2(ffn(x)) (m = `spec.residual_mult`): the norms sit on the sub-layers' outputs
    and the sub-layers read the stream itself (its rounding to the activation dtype; a mixer that says `reads_stream`
    is given the float32 stream as it is).  The norm's kernel adds its result into
    the float32 stream and leaves the new stream in the activation dtype for the next sub-layer.  A block
    without a feed-forward (`spec.ffn` None) is its first half alone."""

    @staticmethod
    def declare(spec: BlockSpec) -> dict:
        norm1, mixer, norm2, ffn = spec.names
        d = {}
        d.update(prefixed(NORMS.get(spec.norm1.kind).declare(spec.norm1), norm1))
        d.update(prefixed(MIXERS.get(spec.mixer.kind).declare(spec.mixer), mixer))
        if spec.ffn is not None:
            d.update(prefixed(NORMS.get(spec.norm2.kind).declare(spec.norm2), norm2))
            d.update(prefixed(FEED_FORWARDS.get(spec.ffn.kind).declare(spec.ffn), ffn))
        return d

    @staticmethod
    def cache_need(spec: BlockSpec):
        return MIXERS.get(spec.mixer.kind).cache_need(spec.mixer)

    def __init__(self, spec: BlockSpec, weights: dict, ctx):
        self.spec = spec
        self.dtype = ctx.dtype
        norm1, mixer, norm2, ffn = spec.names
        self.norm1 = NORMS.get(spec.norm1.kind)(spec.norm1, _exact(weights, norm1, spec.norm1), ctx)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, sub_weights(weights, mixer), ctx)
        self.norm2 = self.ffn = None
        if spec.ffn is not None:
            self.norm2 = NORMS.get(spec.norm2.kind)(spec.norm2, _exact(weights, norm2, spec.norm2), ctx)
            self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn, sub_weights(weights, ffn), ctx)
        for norm in (self.norm1, self.norm2):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise TypeError(f"norm kind {norm.spec.kind!r} cannot norm a sub-layer's output into the stream: "
                                f"it offers no add_normed(y, x, step, cast)")
        self.mult = float(spec.residual_mult)
        # a mixer whose last product has a bias may leave it to the norm's kernel, which reads that product anyway
        self.bias1 = None
        if getattr(self.norm1, "adds_bias", False) and hasattr(self.mixer, "take_out_bias"):
            self.bias1 = self.mixer.take_out_bias()
        self.graph_safe = bool(getattr(self.mixer, "graph_safe", False)
                               and (self.ffn is None or getattr(self.ffn, "graph_safe", False)))

    def _stream_input(self, residual, step):
        if residual.pending is not None or residual.normed is not None:
            raise NotImplementedError("a post-norm block after a block that leaves its result pending")
        if self.dtype == torch.float32:
            return residual.x, None
        buf = step.workspace.get(step.tag + "stream.cast", residual.x.shape, self.dtype)
        if residual.cast is None:
            from ..csrc import ops
            residual.cast = ops.cast(residual.x, buf)
        return residual.cast, buf

    def __call__(self, residual, step, cache):
        kw = {} if self.mult == 1.0 else {"mult": self.mult}
        if getattr(self.mixer, "reads_stream", False):
            # the mixer's first step works on the float32 stream itself (and on other rows of it)
            if residual.pending is not None or residual.normed is not None:
                raise NotImplementedError("a post-norm block after a block that leaves its result pending")
            buf = None if self.dtype == torch.float32 else step.workspace.get(step.tag + "stream.cast", residual.x.shape, self.dtype)
            y = self.mixer(residual.x, step, cache)
        else:
            h, buf = self._stream_input(residual, step)
            y = self.mixer(h, step, cache)
        # the feed-forward reads the new stream in the activation dtype; after the last norm of the block only a
        # following block that asks for it does
        residual.cast = self.norm1.add_normed(y, residual.x, step, buf, **kw, **({} if self.bias1 is None else {"bias": self.bias1}))
        if self.ffn is not None:
            h = residual.x if buf is None else residual.cast
            y = self.ffn(h, step)
            residual.cast = self.norm2.add_normed(y, residual.x, step, buf, **kw)


@BLOCKS.register("sandwich")
class SandwichBlock:
    """x += post1(mixer(norm1(x))); x += post2(ffn(norm2(x))): every sub-layer between a norm on its input and a norm on
    its output.  The input norms read the float32 stream through their own kernel; the output norms add their result into
    it (`add_normed`).  A block without a feed-forward (`spec.ffn` None) is its first half alone."""

    @staticmethod
    def declare(spec: BlockSpec) -> dict:
        norm1, mixer, norm2, ffn = spec.names
        post1, post2 = spec.post_names
        d = {}
        d.update(prefixed(NORMS.get(spec.norm1.kind).declare(spec.norm1), norm1))
        d.update(prefixed(MIXERS.get(spec.mixer.kind).declare(spec.mixer), mixer))
        d.update(prefixed(NORMS.get(spec.post_norms[0].kind).declare(spec.post_norms[0]), post1))
        if spec.ffn is not None:
            d.update(prefixed(NORMS.get(spec.norm2.kind).declare(spec.norm2), norm2))
            d.update(prefixed(FEED_FORWARDS.get(spec.ffn.kind).declare(spec.ffn), ffn))
            d.update(prefixed(NORMS.get(spec.post_norms[1].kind).declare(spec.post_norms[1]), post2))
        return d

    @staticmethod
    def cache_need(spec: BlockSpec):
        return MIXERS.get(spec.mixer.kind).cache_need(spec.mixer)

    def __init__(self, spec: BlockSpec, weights: dict, ctx):
        if spec.post_norms is None:
            raise ValueError("a sandwich block names the two norms on its sub-layers' outputs (post_norms)")
        self.spec = spec
        self.dtype = ctx.dtype
        norm1, mixer, norm2, ffn = spec.names
        post1, post2 = spec.post_names
        self.norm1 = NORMS.get(spec.norm1.kind)(spec.norm1, _exact(weights, norm1, spec.norm1), ctx)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, sub_weights(weights, mixer), ctx)
        self.post1 = NORMS.get(spec.post_norms[0].kind)(spec.post_norms[0], _exact(weights, post1, spec.post_norms[0]), ctx)
        self.norm2 = self.ffn = self.post2 = None
        if spec.ffn is not None:
            self.norm2 = NORMS.get(spec.norm2.kind)(spec.norm2, _exact(weights, norm2, spec.norm2), ctx)
            self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn, sub_weights(weights, ffn), ctx)
            self.post2 = NORMS.get(spec.post_norms[1].kind)(spec.post_norms[1], _exact(weights, post2, spec.post_norms[1]), ctx)
        for norm in (self.post1, self.post2):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise TypeError(f"norm kind {norm.spec.kind!r} cannot norm a sub-layer's output into the stream: "
                                f"it offers no add_normed(y, x, step, cast)")
        self.graph_safe = bool(getattr(self.mixer, "graph_safe", False)
                               and (self.ffn is None or getattr(self.ffn, "graph_safe", False)))

    def __call__(self, residual, step, cache):
        if residual.normed is not None:
            raise NotImplementedError("a sandwich block after a block that leaves a norm's output in factored form")
        h = self.norm1(residual.x, residual.pending, step, tag="norm1")
        residual.pending = None
        residual.cast = None
        if getattr(self.mixer, "returns_pair", False) and getattr(self.post1, "takes_pair", False):
            y = self.mixer(h, step, cache, as_pair=True)          # two mixers side by side: the norm's kernel adds them as it reads
        else:
            y = self.mixer(h, step, cache)
        self.post1.add_normed(y, residual.x, step, None)
        if self.ffn is not None:
            h = self.norm2(residual.x, None, step, tag="norm2")
            y = self.ffn(h, step)
            self.post2.add_normed(y, residual.x, step, None)


def _exact(weights, prefix, norm_spec):
    """The tensors of a norm whose prefix may be its weight's whole name (`tensor` == "")."""
    if getattr(norm_spec, "tensor", "weight") == "":
        return {"": weights[prefix]} if prefix in weights else {}
    return sub_weights(weights, prefix)


@BLOCKS.register("hyper_connection")
class HyperConnectionBlock:
    """A block over several copies x_1 .. x_S of the stream (float32 [T, S, H], made of S copies of the single stream
    by the first such block).  Sub-layer q with the learned in_q [S], out_q [S], mix_q [S, S] (indexed [from, to]):

        u = sum_s in_q[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + out_q[t] y   (all t at once)

    and the single stream is the sum of the copies.  A write-back and the read that follows it are one pass over the
    streams (`ops.hc_step`), also across blocks: the last write-back of a block is left to the next block of this kind
    (`Residual.deferred`), or to the model's end, which also asks for the sum."""

    takes_deferred = True

    @staticmethod
    def declare(spec: BlockSpec) -> dict:
        norm1, mixer, norm2, ffn = spec.names
        d = {}
        d.update(prefixed(NORMS.get(spec.norm1.kind).declare(spec.norm1), norm1))
        d.update(prefixed(MIXERS.get(spec.mixer.kind).declare(spec.mixer), mixer))
        subs = [0]
        if spec.ffn is not None:
            d.update(prefixed(NORMS.get(spec.norm2.kind).declare(spec.norm2), norm2))
            d.update(prefixed(FEED_FORWARDS.get(spec.ffn.kind).declare(spec.ffn), ffn))
            subs.append(1)
        from .spec import TensorDecl
        for q in subs:
            hc, S = spec.hyper[q], spec.hyper[q].streams
            a, o, m = hc.names
            p = spec.hyper_prefixes[q]
            d.update({p + a: TensorDecl((S,), init="norm"), p + o: TensorDecl((S,), init="norm"),
                      p + m: TensorDecl((S, S), init="identity")})
        return d

    @staticmethod
    def cache_need(spec: BlockSpec):
        return MIXERS.get(spec.mixer.kind).cache_need(spec.mixer)

    def __init__(self, spec: BlockSpec, weights: dict, ctx):
        from ..csrc import ops
        self.spec = spec
        self.dtype = ctx.dtype
        self.streams = int(spec.streams)
        if not 1 <= self.streams <= ops.HC_MAX_STREAMS:
            raise ValueError(f"a hyper-connection block keeps 1 to {ops.HC_MAX_STREAMS} streams, got {self.streams}")
        norm1, mixer, norm2, ffn = spec.names
        self.norm1 = NORMS.get(spec.norm1.kind)(spec.norm1, sub_weights(weights, norm1), ctx)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, sub_weights(weights, mixer), ctx)
        self.norm2 = self.ffn = None
        if spec.ffn is not None:
            self.norm2 = NORMS.get(spec.norm2.kind)(spec.norm2, sub_weights(weights, norm2), ctx)
            self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn, sub_weights(weights, ffn), ctx)
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()
        self.hc = []
        for q in range(2 if spec.ffn is not None else 1):
            a, o, m = spec.hyper[q].names
            p = spec.hyper_prefixes[q]
            self.hc.append((f32(weights[p + a]), f32(weights[p + o]), f32(weights[p + m])))
        self.graph_safe = bool(getattr(self.mixer, "graph_safe", False)
                               and (self.ffn is None or getattr(self.ffn, "graph_safe", False)))

    def _read(self, residual, step, q, pending):
        """h for sub-layer q, after the write-back `pending` = (y, mix, out) of the sub-layer before (or None)."""
        from ..csrc import ops
        norm = self.norm1 if q == 0 else self.norm2
        in_w = self.hc[q][0]
        T, H = residual.x.shape
        single = None
        if residual.streams is None or residual.streams.shape != (T, self.streams, H):
            if pending is not None:
                raise RuntimeError("a write-back is pending for streams that do not exist")
            residual.streams = step.workspace.get(step.tag + "streams", (T, self.streams, H), torch.float32)
            single = residual.x
        h = step.workspace.get(step.tag + f"hc.h{q}", (T, H), self.dtype)
        y, mix, out_w = pending if pending is not None else (None, None, None)
        fused = getattr(norm, "elementwise", None)
        if fused is not None:
            ops.hc_step(residual.streams, single=single, y=y, mix=mix, out_w=out_w, in_w=in_w, norm=fused(), h=h)
            return h
        # a norm of another kind reads the plain sum u through its own kernel
        u = step.workspace.get(step.tag + "hc.u", (T, H), torch.float32)
        ops.hc_step(residual.streams, single=single, y=y, mix=mix, out_w=out_w, in_w=in_w, h=u)
        return norm(u, None, step, tag=f"hc.norm{q}")

    def __call__(self, residual, step, cache):
        from ..csrc import ops
        if residual.pending is not None or residual.normed is not None:
            raise NotImplementedError("a hyper-connection block after a block that leaves its result pending")
        pending = None
        if residual.deferred is not None:
            pending, residual.deferred = residual.deferred.pending, None
        h = self._read(residual, step, 0, pending)
        y = self.mixer(h, step, cache)
        last = (y, self.hc[0][2], self.hc[0][1])
        if self.ffn is not None:
            h = self._read(residual, step, 1, last)
            y = self.ffn(h, step)
            last = (y, self.hc[1][2], self.hc[1][1])
        residual.cast = None
        residual.deferred = _DeferredWriteBack(residual, last)


class _DeferredWriteBack:
    """The last write-back of a hyper-connection block, not yet done.  The next block of the kind takes `pending`
    and does it in its first pass; called (by `Residual.settle`) it is done alone, and the single stream x
    becomes the sum of the copies."""

    def __init__(self, residual, pending):
        self.residual, self.pending = residual, pending

    def __call__(self, _next=None):
        from ..csrc import ops
        r = self.residual
        y, mix, out_w = self.pending
        ops.hc_step(r.streams, y=y, mix=mix, out_w=out_w, total=r.x)
        r.deferred = None
