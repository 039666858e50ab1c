"""Chooses the attention kernel for a step.

Every kernel computes the same function of (query token, its request's pages);
which one runs depends on the dtype and on the shape of the step only.  The
float32 path always takes the one kernel whose order of additions depends on
positions alone, so its results are bit-for-bit independent of the batch.  In
bfloat16 the tensor-core kernels run: requests that bring one token (decoding)
go to the kernel that splits each token's key range over many blocks, requests
that bring a portion of a prompt to one that walks tiles of query tokens (the
tcgen05 kernel when a portion is long enough to fill its 128-row tiles and it
takes the head and page size, else the mma.sync kernel); a step that holds both
kinds launches both, each on its own tokens.
"""
from __future__ import annotations

import torch

from .base import QUERY_TILE


FOLD_MAX_CHUNKS = 4      # most chunks per token with which the decode attention still does the head work itself


def folds_head_work(dtype, step, spec, group, num_tokens) -> bool:
    """Whether `run` will do the head norm, the rotation and the cache write of this step itself (pass `fold`),
    so that the mixer launches no kernel for them: a decode step (every request brings one token) that the
    block-per-chunk kernel serves with few chunks per token (every chunk's block prepares the query heads
    again).  Measured at Qwen3-8B sizes, a step with / without: batch 8 at 4,096 keys (4 chunks) 3.77 / 3.79 ms,
    batch 16 at 1,024 keys (1 chunk) 3.99 / 4.06; batch 4 (8 chunks) 3.635 / 3.61, batch 1 (16 chunks) 3.07 / 3.065."""
    from ..csrc import ops
    if not (ops.flash_supported(dtype, spec.head_dim) and step.max_query_len == 1):
        return False
    if ops.flash_decode_streams(dtype, num_tokens, spec.num_kv_heads, spec.head_dim, group.page_size, group.max_context):
        return False
    chunk = ops.decode_chunk_for(num_tokens, spec.num_kv_heads, group.max_context, head_dim=spec.head_dim)
    return -(-int(group.max_context) // chunk) <= FOLD_MAX_CHUNKS


def _decode(ops, args, step, spec, group, num_tokens, max_context, token_index=None, fold=None, sinks=None, variant=None,
            shape=None):
    chunk = ops.decode_chunk_for(num_tokens, spec.num_kv_heads, max_context, head_dim=spec.head_dim)
    own_merge = True
    if variant is not None:
        # the keys a token reads end at its block of the mask: chunks as short as serve that reach, merged inside the launch
        reach = min(int(max_context), int(variant["mask_chunk"] or max_context), int(spec.window or max_context))
        chunk = min(chunk, 256 if reach <= 1024 else (512 if reach <= 2048 else 1024))
    if getattr(spec, "shared_row", False) and spec.num_heads >= 16:
        # One shared row for 16 heads and more (latent attention): the step is bound by the blocks' own pace, not by
        # bytes, and runs best with about four chunks over the keys a token reads, merged by the merge kernel
        # (measured, 64 tokens x 32 heads x 4,096 keys: 57 us against 71 with the chunks merged inside the launch;
        # 64 x 16 heads, window 1,024 of 4,096: 19 us with chunks of 256 against 29 with chunks of 1,024).
        reach = min(int(max_context), int(spec.window)) if spec.window else int(max_context)
        chunk = 256 if reach <= 1024 else (512 if reach <= 2048 else 1024)
        own_merge = False
    S, n_acc, n_ml = ops.decode_attention_scratch(num_tokens, spec.num_heads, spec.head_dim, max_context, chunk)
    part_acc = step.workspace.get(step.tag + "attn.part_acc", (n_acc,), torch.float32)
    part_ml = step.workspace.get(step.tag + "attn.part_ml", (n_ml,), torch.float32)
    # one set of counters for all layers of a step shape: every launch leaves them zero
    arrivals = step.workspace.zeros(step.tag + "attn.arrivals", ops.flash_decode_arrivals(num_tokens, spec.num_heads, spec.num_kv_heads),
                                    torch.int32) if own_merge else None
    return ops.flash_decode(*args, max_context, part_acc, part_ml, step.err, chunk=chunk, token_index=token_index,
                            arrivals=arrivals, fold=fold, sinks=sinks, **(variant or {}), **(shape or {}))


def _variant_decode_ok(ops, spec, num_tokens, max_context, mask_chunk) -> bool:
    """Whether the block-per-chunk kernel can merge the chunks of this step itself, which its options ask for."""
    chunk = ops.decode_chunk_for(num_tokens, spec.num_kv_heads, max_context, head_dim=spec.head_dim)
    reach = min(int(max_context), int(mask_chunk or max_context), int(spec.window or max_context))
    chunk = min(chunk, 256 if reach <= 1024 else (512 if reach <= 2048 else 1024))
    return -(-int(max_context) // chunk) <= ops.flash_decode_own_merge_cap(spec.head_dim)


def run(qkv, out, cache, group, step, spec, scale, fold=None, sinks=None, weighting="softmax", chunk=None,
        head_bias=None, gate=None, softcap=None, distance=None):
    """`spec`: anything with num_heads, num_kv_heads, head_dim and window.
    `fold` (only where `folds_head_work` said so): (q_weight, k_weight, eps, inv_freq, rotary_dim, slots) of the
    head work that the mixer left undone.
    `sinks` (float32 [num_heads]): a number per head that joins every softmax denominator as exp(sink).
    `weighting` "sigmoid" (with `head_bias`, float32 [num_heads]): a key weighs sigmoid(score + head_bias[h]) by
    itself; `chunk`: positions in blocks of that many, no key of an earlier block is read; `gate` [T, >= num_heads]:
    head h's output is multiplied by sigmoid(gate[t, h]).
    `softcap` c: score <- c tanh(score / c); `distance` (a, b), float32 [num_heads] each: a[h] ln(1 + b[h] (i - j)) is
    taken off the score of the key j that query i reads."""
    from ..csrc import ops
    if softcap or distance is not None:
        return _run_shaped(ops, qkv, out, cache, group, step, spec, scale, sinks, weighting, chunk, head_bias, gate,
                           softcap, distance)
    if weighting != "softmax" or chunk is not None or head_bias is not None or gate is not None:
        return _run_variant(ops, qkv, out, cache, group, step, spec, scale, weighting, chunk, head_bias, gate, sinks)
    if fold is not None and not folds_head_work(qkv.dtype, step, spec, group, qkv.shape[0]):
        raise ValueError("this step's attention kernel does not fold the head norm and rotation in")
    args = (qkv, out, cache.k, cache.v, group.block_table, step.req_index, step.positions,
            spec.num_heads, spec.num_kv_heads, spec.head_dim, scale, spec.window)
    if ops.flash_supported(qkv.dtype, spec.head_dim):
        if step.max_query_len == 1:
            return _decode(ops, args, step, spec, group, qkv.shape[0], group.max_context, fold=fold, sinks=sinks)
        if step.query_tiles is not None:
            tile_args = (qkv, out, cache.k, cache.v, group.block_table, step.query_tiles,
                         spec.num_heads, spec.num_kv_heads, spec.head_dim, scale, spec.window, step.err)
            if step.max_query_len > 64 and ops.flash_tc5_supported(qkv.dtype, spec.head_dim, group.page_size):
                ops.flash_prefill_tc5(*tile_args, sinks=sinks)
            else:
                ops.flash_prefill(*tile_args, tile_rows=QUERY_TILE, sinks=sinks)
            if step.single_tokens is not None:
                _decode(ops, args, step, spec, group, step.single_tokens.shape[0], step.single_context,
                        token_index=step.single_tokens, sinks=sinks)
            return out
    return ops.paged_attention(*args, step.err, sinks=sinks)


def _run_variant(ops, q, out, cache, group, step, spec, scale, weighting, chunk, head_bias, gate, sinks):
    """Attention with another weighting than the softmax, a chunked mask or an output gate: in bfloat16 the tensor-core
    kernels for portions of prompts (tcgen05 for long portions of heads of 64 or 128, else mma.sync) and the
    block-per-chunk kernel for single tokens, each with these options; in float32, or where those do not take the head
    size or the step, the one kernel whose sums depend on positions alone."""
    variant = dict(weighting=weighting, mask_chunk=chunk, head_bias=head_bias, gate=gate)
    args = (q, out, cache.k, cache.v, group.block_table, step.req_index, step.positions,
            spec.num_heads, spec.num_kv_heads, spec.head_dim, scale, spec.window)
    if ops.flash_supported(q.dtype, spec.head_dim):
        if step.max_query_len == 1:
            if _variant_decode_ok(ops, spec, q.shape[0], group.max_context, chunk):
                return _decode(ops, args, step, spec, group, q.shape[0], group.max_context, sinks=sinks, variant=variant)
        elif step.query_tiles is not None and (step.single_tokens is None or _variant_decode_ok(
                ops, spec, step.single_tokens.shape[0], step.single_context, chunk)):
            tile_args = (q, out, cache.k, cache.v, group.block_table, step.query_tiles, spec.num_heads, spec.num_kv_heads,
                         spec.head_dim, scale, spec.window, step.err)
            if step.max_query_len > 64 and ops.flash_tc5_supported(q.dtype, spec.head_dim, group.page_size):
                ops.flash_prefill_tc5(*tile_args, sinks=sinks, **variant)
            else:
                ops.flash_prefill(*tile_args, tile_rows=QUERY_TILE, sinks=sinks, **variant)
            if step.single_tokens is not None:
                _decode(ops, args, step, spec, group, step.single_tokens.shape[0], step.single_context,
                        token_index=step.single_tokens, sinks=sinks, variant=variant)
            return out
    return ops.paged_attention(q, out, cache.k, cache.v, group.block_table, step.req_index, step.positions,
                               spec.num_heads, spec.num_kv_heads, spec.head_dim, scale, spec.window, step.err, sinks=sinks,
                               weighting=weighting, chunk=chunk, head_bias=head_bias, gate=gate)


def _run_shaped(ops, q, out, cache, group, step, spec, scale, sinks, weighting, chunk, head_bias, gate, softcap, distance):
    """Attention whose scores are capped or lose a bias that grows with the distance: in bfloat16 the tensor-core kernels
    for portions of prompts (tcgen05 for long portions of heads of 64 or 128, else mma.sync) and the block-per-chunk kernel
    for single tokens (a mixed step launches both); in float32, for
    other head sizes, or together with another weighting, a chunked mask or a gate per head, the one kernel whose sums
    depend on positions alone."""
    shape = dict(softcap=softcap, distance=distance)
    plain = weighting == "softmax" and chunk is None and head_bias is None and gate is None
    if plain and ops.flash_supported(q.dtype, spec.head_dim):
        args = (q, out, cache.k, cache.v, group.block_table, step.req_index, step.positions,
                spec.num_heads, spec.num_kv_heads, spec.head_dim, scale, spec.window)
        if step.max_query_len == 1:
            return _decode(ops, args, step, spec, group, q.shape[0], group.max_context, sinks=sinks, shape=shape)
        if step.query_tiles is not None:
            tile_args = (q, out, cache.k, cache.v, group.block_table, step.query_tiles, spec.num_heads, spec.num_kv_heads,
                         spec.head_dim, scale, spec.window, step.err)
            if step.max_query_len > 64 and ops.flash_tc5_supported(q.dtype, spec.head_dim, group.page_size):
                ops.flash_prefill_tc5(*tile_args, sinks=sinks, **shape)
            else:
                ops.flash_prefill(*tile_args, tile_rows=QUERY_TILE, sinks=sinks, **shape)
            if step.single_tokens is not None:
                _decode(ops, args, step, spec, group, step.single_tokens.shape[0], step.single_context,
                        token_index=step.single_tokens, sinks=sinks, shape=shape)
            return out
    return ops.paged_attention(q, out, cache.k, cache.v, group.block_table, step.req_index, step.positions,
                               spec.num_heads, spec.num_kv_heads, spec.head_dim, scale, spec.window, step.err, sinks=sinks,
                               weighting=weighting, chunk=chunk, head_bias=head_bias, gate=gate, softcap=softcap,
                               distance=distance)
