"""The Puturax decoder in the engine against the plain implementation (tests/plain_puturax.py).

Small configurations of their own that differ in every size, per layer too (head sizes that are no multiple of 16, value
heads wider and narrower than key heads, a rotated part of which only some features turn, ranks of every kind, a layer
without a feed-forward, layers in other orders) and in every constant, also values that are equal or 1 (one head, as
many key heads as query heads, one group of experts, every expert chosen and one, a query factor that steps at every
position, scales of 1).  Seeded random weights with edits where random numbers would hide a fault: routers with wide
gaps, one far key made to stand out among hundreds, sharp scores so that a step of the query factor moves the logits.
Each mechanism alone against one function of the plain implementation, with state carried across steps and slots; then
whole prompts, the stream after every layer, decoding token by token, portions down to two tokens, mixed batches with
pages and slots used again, long prompts and decoding, and greedy generation through the engine's entry point, the command
line and the replay program.
"""
import copy
import functools
import json
import math

import numpy as np
import pytest
import torch

import helpers as H
import plain_puturax as P

DEV = "cuda:0"


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, dims, base):
    return dict(type="latent_attention", mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank,
                                                    kv_rank=kv_rank, scale=scale, rot=dict(dims=dims, base=base)))


def parallel(heads, kv, dim, vdim, scale, cap, coef, every, rheads, rdim, rank, ls, rs):
    return dict(type="parallel", mixer=dict(left=dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, softcap=cap,
                                                      q_temp=dict(coef=coef, every=every)),
                                            right=dict(heads=rheads, dim=rdim, decay_rank=rank), left_scale=ls, right_scale=rs))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, top, count, keep, shared):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, groups=dict(count=count, keep=keep)),
                shared=dict(ff=shared))


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


def model(vocab, width, eps, emb, layers):
    return dict(architecture="Puturax", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=emb), layers=layers)


# A: every layer its own sizes; a value head wider (24) and narrower (16) than its key head; the query factor steps every
#    16 and every 5 positions; a layer without a feed-forward; experts in 4 groups of which 2 are kept.
# B: the values that are equal or 1: one head, key heads = query heads, ONE group of experts, every expert chosen / one
#    chosen, a query factor that steps at every position, scales 1, an embedding factor of 1; half of the rotated part turns.
# C: pages of 64 positions, heads of 64 and 128 numbers (the sizes of the tensor-core attention kernels), a latent row of
#    96 + 32 numbers, a parallel layer FIRST and a latent one last.
# D: sizes that are multiples of two at best: heads of 20 and 6, a memory of 12 x 12, ranks of 10 and 20, a width of 72, pages of 4.
CONFIGS = {
    "A": model(150, 64, 1e-5, 3.0,
               [layer(latent(4, 16, 8, 16, 24, 40, 0.3, 8, 10000.0), dense(96)),
                layer(parallel(4, 2, 16, 24, 0.9, 5.0, 0.3, 16, 2, 16, 8, 0.8, 0.5), moe(40, 8, 2, 4, 2, 24)),
                layer(parallel(3, 3, 32, 16, 1.3, 30.0, 0.7, 5, 3, 8, 4, 1.2, 0.7), None),
                layer(latent(2, 24, 16, 8, 16, 24, 0.2, 16, 50.0), moe(24, 4, 3, 2, 2, 40))]),
    "B": model(211, 96, 3e-6, 1.0,
               [layer(parallel(1, 1, 48, 48, 1.0, 1.0, 1.0, 1, 1, 32, 1, 1.0, 1.0), moe(48, 5, 5, 1, 1, 16)),
                layer(latent(1, 32, 16, 32, 96, 16, 1.0, 8, 1234.0), moe(32, 6, 1, 6, 1, 8)),
                layer(parallel(6, 6, 16, 16, 0.5, 8.0, 0.1, 64, 6, 16, 16, 1.0, 0.3), dense(32))]),
    "C": model(301, 128, 1e-6, 11.0,
               [layer(parallel(8, 2, 64, 64, 0.7, 20.0, 0.3, 32, 4, 32, 16, 0.8, 0.5), moe(64, 8, 2, 2, 1, 96)),
                layer(parallel(2, 1, 128, 96, 0.5, 12.0, 0.2, 100, 2, 64, 8, 0.5, 1.0), dense(160)),
                layer(latent(8, 32, 32, 32, 80, 96, 0.125, 32, 250000.0), None)]),
    "D": model(97, 72, 2e-5, 0.5,
               [layer(latent(3, 20, 6, 6, 10, 20, 0.22, 6, 3.0), moe(20, 6, 4, 3, 2, 10)),
                layer(parallel(6, 3, 20, 6, 0.6, 3.0, 0.5, 3, 3, 12, 6, 0.9, 0.4), dense(18))]),
}
PAGE = {"A": 8, "B": 16, "C": 64, "D": 4}
SEED = {"A": 51, "B": 52, "C": 53, "D": 54}
# max |engine - plain| / max |plain| over a row of logits; float32 stays near 3e-6 at these sizes, bfloat16 near 3e-2
# (four norms a layer, each after a sub-layer whose result was rounded)
TOL = {"float32": 3e-5, "bfloat16": 5e-2}
CASES = [(w, d) for w in ("A", "B", "C", "D") for d in ("float32", "bfloat16")]


def edited(cfg, sharp=1.0, every=0):
    """The same model with every attention scale of the parallel layers multiplied and every `every` of the query factor moved."""
    cfg = copy.deepcopy(cfg)
    for l in cfg["layers"]:
        if l["type"] == "parallel":
            l["mixer"]["left"]["scale"] *= sharp
            l["mixer"]["left"]["q_temp"]["every"] = max(1, l["mixer"]["left"]["q_temp"]["every"] + every)
    return cfg


def store_of(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


@functools.lru_cache(maxsize=None)
def model_dir(which, store="bfloat16", sharp=1.0):
    """A folder with the configuration and seeded weights; the decays' offsets are moved below zero so that the memories
    forget slowly.  The float32 folders get routers with wide logits, so that the choice of experts changes from token to
    token.  The bfloat16 folders get corrections that grow by a factor of 1.6 in a shuffled order (no two
    of them, and no two sums of two, lie close) and routers as drawn: a choice there hardly ever rests on a close call, which a rounding could turn and which every later token would then carry on
    in its memories (the float32 tests, and the router's own test, hold the choice token by token)."""
    from vllm_lite_b200.weights import write_model_dir
    from vllm_lite_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    cfg = edited(CONFIGS[which], sharp)
    d = H.tmp_root() / f"puturax_{which}_{store}_{sharp}"
    write_model_dir(d, cfg, SEED[which], std=0.08, dtype=torch.float32 if store == "float32" else torch.bfloat16)
    f = SafetensorsFile(d / "model.safetensors")
    tensors = {n: f.read(n).clone() for n in f.names()}
    f.close()
    for name, t in tensors.items():
        if name.endswith(".mlp.router") and store == "float32":
            tensors[name] = (t.float() * 6.0).to(t.dtype)
        if name.endswith(".mlp.correction") and store != "float32":
            order = np.random.default_rng(t.numel() + len(name)).permutation(t.numel())
            tensors[name] = (0.8 * 1.6 ** torch.tensor(order, dtype=torch.float32) - 3.0).to(t.dtype)
        if name.endswith(".right.w0"):
            tensors[name] = (t.float() * 3.0 - 3.0).to(t.dtype)
    write_safetensors(d / "model.safetensors", tensors, metadata={"format": "pt"})
    return d


@functools.lru_cache(maxsize=None)
def plain_model(which, store, sharp=1.0):
    return P.read_model_dir(model_dir(which, store, sharp))


_plain = {}


def plain_run(which, tokens, dtype, sharp=1.0, every=0):
    key = (which, store_of(dtype), sharp, every, tuple(tokens))
    if key not in _plain:
        cfg, w = plain_model(which, store_of(dtype), sharp)
        logits, after = P.forward(edited(cfg, 1.0, every), w, list(tokens))
        _plain[key] = (logits.float(), [a.float() for a in after])
    return _plain[key]


def tokens_for(which, length, seed):
    rng = np.random.default_rng(9000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[which]["vocab"], size=length)]


def make_runner(which, dtype, num_pages, sharp=1.0, page_size=None, max_requests=4, max_context=1024, **kw):
    from vllm_lite_b200.engine import ModelRunner, load_model_dir
    _, plan, weights = load_model_dir(model_dir(which, store_of(dtype), sharp), dtype, DEV)
    return ModelRunner(plan, weights, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32, device=DEV,
                       page_size=page_size or PAGE[which], num_pages=num_pages, max_requests=max_requests,
                       max_context=max_context, **kw)


def assert_rows(rows, which, requests, dtype, what, sharp=1.0, loosen=1.0):
    """float32: every row within the tolerance.  bfloat16: a row's rounding can change which expert a router takes where
    two choice scores lie close, and then that row and those that read it differ by far more than rounding; up to a
    twentieth of the rows (or one row) may, the mechanisms' own tests hold every row."""
    assert rows, "nothing was compared"
    errs = []
    for (rid, pos), row in rows.items():
        ref = plain_run(which, requests[rid], dtype, sharp)[0][pos]
        err = float((row - ref).abs().max()) / max(float(ref.abs().max()), 1e-12)
        if dtype == "float32":
            assert err <= loosen * TOL[dtype], f"{what} {which}/{dtype}: request {rid} position {pos}: {err:.3e}"
        errs.append(err)
    over = [e for e in errs if e > loosen * TOL[dtype]]
    assert len(over) <= max(1, len(errs) // 20), f"{what} {which}/{dtype}: {len(over)} of {len(errs)} rows, worst {max(errs):.3e}"
    errs.sort()
    worst = errs[len(errs) - 1 - len(errs) // 20]
    key = ("puturax " + what, which, dtype)
    H.WORST[key] = max(H.WORST.get(key, 0.0), worst)


def pages_for(which, tokens):
    return -(-tokens // PAGE[which])


# ----------------------------------------------------------------------------------------------
# without a GPU: configuration, plan, cache layout, the plain implementation's own behaviour
# ----------------------------------------------------------------------------------------------

def test_config_reads_every_size_and_constant():
    from vllm_lite_b200.config import plan_from_config_json
    from vllm_lite_b200.parts.model import declare_model
    cfg, plan = plan_from_config_json(CONFIGS["A"])
    assert (cfg.vocab_size, cfg.hidden_size, cfg.eps, cfg.embedding_scale) == (150, 64, 1e-5, 3.0)
    assert plan.embedding.scale == 3.0 and plan.tie_word_embeddings and plan.head.tied and plan.final_norm.offset == 1.0
    assert all(b.kind == "sandwich" and b.norm1.offset == 1.0 and b.post_norms[1].offset == 1.0 for b in plan.layers)
    b0, b1, b2, b3 = plan.layers
    m0 = b0.mixer
    assert (m0.kind, m0.num_heads, m0.dim, m0.rot_dim, m0.vdim, m0.q_rank, m0.kv_rank, m0.scale) == ("latent_attention", 4, 16, 8, 16, 24, 40, 0.3)
    assert (m0.position.dim, m0.position.theta, m0.gate, m0.sink, m0.window) == (8, 10000.0, "g", False, None)
    assert (b3.mixer.position.dim, b3.mixer.rot_dim, b3.mixer.position.theta) == (16, 16, 50.0)
    l1, r1 = b1.mixer.left, b1.mixer.right
    assert (b1.mixer.kind, b1.mixer.left_scale, b1.mixer.right_scale) == ("parallel_mixer", 0.8, 0.5)
    assert (l1.num_heads, l1.num_kv_heads, l1.head_dim, l1.v_head_dim, l1.scale, l1.softcap, l1.q_temp) == (4, 2, 16, 24, 0.9, 5.0, (0.3, 16))
    assert l1.position is None and not l1.qk_norm.has_weight and l1.v_norm == 1e-5 and l1.unit_sink and l1.gate == "g"
    assert l1.distance_bias == ("r1", "r2") and l1.window is None
    assert (r1.kind, r1.num_heads, r1.dim, r1.decay_rank, r1.eps) == ("time_mix", 2, 16, 8, 1e-5)
    assert (b2.mixer.left.q_temp, b2.mixer.left.softcap, b2.mixer.right.decay_rank) == ((0.7, 5), 30.0, 4) and b2.ffn is None
    f0, f1 = b0.ffn, b1.ffn
    assert (f0.kind, f0.gated, f0.activation, f0.intermediate_size) == ("gated_mlp", False, "relu2", 96)
    assert (f1.num_experts, f1.top, f1.groups, f1.keep_groups, f1.group_top, f1.intermediate_size) == (8, 2, 4, 2, 2, 40)
    assert (f1.score, f1.renormalize, f1.renorm_eps, f1.scale_input, f1.choice_bias, f1.activation) == ("sigmoid", True, 1e-20, False, "correction", "silu")
    assert (f1.shared.kind, f1.shared.intermediate_size, f1.shared.activation, f1.shared.gated) == ("gated_mlp", 24, "silu", True)
    names = declare_model(plan)
    assert names["embed"].shape == (150, 64) and names["final.norm"].shape == (64,) and "head" not in names
    assert all(names[f"l0.{n}"].shape == (64,) for n in ("norm1", "norm1b", "norm2", "norm2b"))
    assert names["l0.mix.dq"].shape == (24, 64) and names["l0.mix.uq"].shape == (4 * 24, 24) and names["l0.mix.dkv"].shape == (48, 64)
    assert names["l0.mix.dkv.norm"].shape == (40,) and names["l0.mix.uk"].shape == (64, 40) and names["l0.mix.g"].shape == (64, 64)
    assert names["l0.mlp.up"].shape == (96, 64) and "l0.mlp.gate" not in names
    assert names["l1.mix.left.q"].shape == (64, 64) and names["l1.mix.left.v"].shape == (48, 64) and names["l1.mix.left.g"].shape == (96, 64)
    assert names["l1.mix.left.o"].shape == (64, 96) and names["l1.mix.left.r1"].shape == (4,) and "l1.mix.left.q_norm.weight" not in names
    assert names["l1.mix.right.mu.w"].shape == (64,) and names["l1.mix.right.w1"].shape == (8, 64) and names["l1.mix.right.w2"].shape == (32, 8)
    assert names["l1.mix.right.u"].shape == (2, 16) and names["l1.mix.right.r"].shape == (32, 64) and names["l1.mix.right.norm"].shape == (32,)
    assert names["l1.mlp.router"].shape == (8, 64) and names["l1.mlp.correction"].shape == (8,) and names["l1.mlp.e7.gate"].shape == (40, 64)
    assert names["l1.mlp.shared.down"].shape == (64, 24) and "l2.norm2" not in names and "l2.mlp.router" not in names


def test_the_decay_rank_comes_from_the_tensor_when_the_file_does_not_say():
    from vllm_lite_b200.config import MissingField, plan_from_config_json
    cfg = copy.deepcopy(CONFIGS["D"])
    del cfg["layers"][1]["mixer"]["right"]["decay_rank"]
    with pytest.raises(MissingField, match="decay_rank"):
        plan_from_config_json(cfg)
    _, plan = plan_from_config_json(cfg, shapes={"l1.mix.right.w1": (5, 72)})
    assert plan.layers[1].mixer.right.decay_rank == 5


def test_config_errors_name_the_field():
    from vllm_lite_b200.config import InvalidField, MissingField, plan_from_config_json
    def bad(edit):
        c = copy.deepcopy(CONFIGS["A"])
        edit(c)
        return c
    with pytest.raises(MissingField, match=r"layers\[0\]\.mixer\.rot"):
        plan_from_config_json(bad(lambda c: c["layers"][0]["mixer"].pop("rot")))
    with pytest.raises(InvalidField, match=r"layers\[2\]\.type"):
        plan_from_config_json(bad(lambda c: c["layers"][2].update(type="something_else")))
    with pytest.raises(InvalidField, match="router"):
        plan_from_config_json(bad(lambda c: c["layers"][1]["mlp"]["router"].update(top=5)))         # 2 groups of 2 offer 4
    with pytest.raises(InvalidField, match="kv_heads"):
        plan_from_config_json(bad(lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3)))
    with pytest.raises(InvalidField, match=r"rot\.dims"):
        plan_from_config_json(bad(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10)))
    with pytest.raises(MissingField, match=r"layers\[1\]\.mixer\.right"):
        plan_from_config_json(bad(lambda c: c["layers"][1]["mixer"].pop("right")))
    with pytest.raises(InvalidField, match=r"mlp\.kind"):
        plan_from_config_json(bad(lambda c: c["layers"][0]["mlp"].update(kind="other")))
    for key in ("embedding", "norm", "vocab", "width"):
        with pytest.raises(MissingField, match=key):
            plan_from_config_json(bad(lambda c: c.pop(key)))


def test_layers_hold_a_latent_row_or_pages_and_a_state():
    from vllm_lite_b200.cache import FixedState, PagedKV, PagedLatent, Several
    from vllm_lite_b200.config import plan_from_config_json
    from vllm_lite_b200.parts.model import cache_needs
    _, plan = plan_from_config_json(CONFIGS["A"])
    needs = cache_needs(plan)
    assert needs[0] == PagedLatent(48) and needs[3] == PagedLatent(48)            # 40 + 8 and 24 + 16 -> 48 either way
    assert isinstance(needs[1], Several) and needs[1].parts[0] == PagedKV(2, 32) and isinstance(needs[1].parts[1], FixedState)
    assert needs[1].parts[1].shape[0] >= 64 + 2 * 16 * 16 and needs[2].parts[0] == PagedKV(3, 32)


def test_plain_pieces_behave():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(P.offset_norm(x, torch.zeros(2), 0.0), x / (12.5 ** 0.5))
    assert torch.allclose(P.offset_norm(x, torch.tensor([1.0, -1.0]), 0.0), torch.tensor([[6.0 / 12.5 ** 0.5, 0.0]], dtype=torch.float64))
    q = torch.randn(5, 2, 8, dtype=torch.float64)
    r = P.rotate_half(q, 4, 100.0)
    assert torch.allclose(r[0], q[0]) and torch.equal(r[:, :, 4:], q[:, :, 4:])
    assert torch.allclose(r[:, :, 0] ** 2 + r[:, :, 2] ** 2, q[:, :, 0] ** 2 + q[:, :, 2] ** 2)       # i turns with i + dims / 2
    f = P.query_temperature(9, 0.5, 4)                                       # floor((p + 1) / 4): 0 0 0 1 1 1 1 2 2
    assert torch.allclose(f, torch.tensor([1.0] * 3 + [1 + 0.5 * math.log(2)] * 4 + [1 + 0.5 * math.log(3)] * 2, dtype=torch.float64))
    s = torch.tensor([0.0, 0.0], dtype=torch.float64)
    assert torch.allclose(P.softmax_plus_one(s), torch.tensor([1 / 3, 1 / 3], dtype=torch.float64))   # the sink takes a third
    assert torch.allclose(P.softmax_plus_one(torch.tensor([-50.0], dtype=torch.float64)), torch.tensor([math.exp(-50.0)], dtype=torch.float64), rtol=1e-9)
    d64 = lambda v: torch.tensor(v, dtype=torch.float64)
    assert float(P.distance_bias(d64(2.0), d64(0.5), d64(0.0))) == 0.0
    assert abs(float(P.distance_bias(d64(2.0), d64(0.5), d64(6.0))) - 2 * math.log(4.0)) < 1e-12
    assert abs(float(P.capped(torch.tensor(1000.0, dtype=torch.float64), 7.0)) - 7.0) < 1e-9
    # the memory: one key channel, decay 0.5, bonus 3 for the current token
    one = torch.ones(3, 1, dtype=torch.float64)
    o = P.decayed_memory(one, one, one, 0.5 * one, torch.tensor([3.0], dtype=torch.float64))
    assert torch.allclose(o[:, 0], torch.tensor([3.0, 4.0, 4.5], dtype=torch.float64))
    # choice by score + correction inside the kept groups; weights without the correction; every choice score here is
    # negative, so an expert outside the kept groups would win if it were masked with a zero
    h = torch.eye(4, dtype=torch.float64)[:1]
    router = torch.tensor([[0.0, 0, 0, 0], [2.0, 0, 0, 0], [1.0, 0, 0, 0], [-1.0, 0, 0, 0]])
    corr = torch.tensor([-3.0, -5.0, -2.0, -2.5])
    ids, w = P.route(h, router, corr, 2, 2, 1)       # groups (0, 1): -2.5 + -4.12; (2, 3): -1.27 + -2.23: the second group
    assert ids[0] == [2, 3]
    sg = torch.sigmoid(torch.tensor([1.0, -1.0], dtype=torch.float64))
    assert torch.allclose(w[0], sg / sg.sum())


# ----------------------------------------------------------------------------------------------
# each mechanism alone, against one function of the plain implementation
# ----------------------------------------------------------------------------------------------

def ops():
    from vllm_lite_b200.csrc import ops as o
    return o


def rand(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, dtype, what, tol=None):
    tol = tol or (2e-5 if dtype in (torch.float32, "float32") else 2.5e-2)
    err = float((got.double().cpu() - want.double().cpu()).abs().max()) / max(float(want.abs().max()), 1e-12)
    assert err <= tol, f"{what} ({dtype}): {err:.3e}"


def ints(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def mini_step(lengths, slots, starts=None):
    """A step's description for parts that keep a state: request b brings lengths[b] tokens from position starts[b] on and
    owns state row slots[b]."""
    from vllm_lite_b200.parts.base import StepBatch, Workspace
    starts = starts or [0] * len(lengths)
    T = int(sum(lengths))
    req = [b for b, n in enumerate(lengths) for _ in range(n)]
    pos = [starts[b] + i for b, n in enumerate(lengths) for i in range(n)]
    return StepBatch(tokens=ints([0] * T), positions=ints(pos), req_index=ints(req),
                     cu_seqlens=ints(np.concatenate([[0], np.cumsum(lengths)])), state_slots=ints(slots), logit_rows=ints([]),
                     groups=[], entries=[], err=torch.zeros(1, dtype=torch.int32, device=DEV), workspace=Workspace(torch.device(DEV)),
                     num_tokens=T, num_entries=len(lengths), max_query_len=max(lengths))


# portions of two requests of 13 and 6 tokens: single tokens, portions of two, one request pausing
CUTS = ([1, 2], [1, 0], [2, 1], [1, 3], [8, 0])


def in_portions(n, fn):
    """fn(live, lengths, starts) -> rows of the step, for every step of CUTS; returns every request's rows in order."""
    got, at = [[], []], [0, 0]
    for lens in CUTS:
        live = [b for b in (0, 1) if lens[b]]
        out = fn(live, [lens[b] for b in live], [at[b] for b in live])
        o = 0
        for b in live:
            got[b].append(out[o:o + lens[b]].clone())
            o += lens[b]
            at[b] += lens[b]
    assert at == n
    return [torch.cat(g) for g in got]


def build_part(spec, dtype, seed, registry="MIXERS", edit=None, std=0.15):
    """(part, its tensors as the plain implementation reads them) with seeded random weights."""
    from vllm_lite_b200.parts import registry as R
    from vllm_lite_b200.parts.base import BuildContext
    from vllm_lite_b200.weights import random_tensors
    cls = getattr(R, registry).get(spec.kind)
    tensors = random_tensors(cls.declare(spec), seed, std, 0.1, dtype=dtype)
    if edit:
        edit(tensors)
    part = cls(spec, {k: v.to(DEV) for k, v in tensors.items()}, BuildContext(torch.device(DEV), dtype))
    return part, tensors


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [6, 64, 300, 2048])
def test_norm_with_a_weight_around_zero_before_and_after_a_sublayer(dtype, W):
    """The factor is 1 + w: on the stream's rows (the norm before a sub-layer) and on a sub-layer's output, added into the stream."""
    from vllm_lite_b200.parts import spec as S
    spec = S.NormSpec(W, 1e-5, tensor="", offset=1.0)
    part, tensors = build_part(spec, dtype, 3, "NORMS", std=0.3)
    assert abs(float(tensors[""].float().mean())) < 0.2                    # stored around zero
    x = rand((9, W), 4, torch.float32, 3.0)
    step = mini_step([9], [0])
    close(part(x, None, step), P.offset_norm(x.double().cpu(), tensors[""], 1e-5), dtype, "norm before")
    y = rand((9, W), 5, dtype, 2.0)
    want = x.double().cpu() + P.offset_norm(y.double().cpu(), tensors[""], 1e-5)
    part.add_normed(y, x, step, None)
    close(x, want, torch.float32, "norm after, into the stream", tol=2e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [6, 72, 300, 2048, 5000])
def test_norm_after_two_mixers_side_by_side(dtype, W):
    """The norm after a sub-layer given the two results of mixers side by side and their factors: it norms
    s1 a + s2 b (float32, never rounded to the model's dtype) and adds the result into the stream."""
    w = rand((W,), 30) * 0.3 + 1.0
    a, b = rand((7, W), 31, dtype, 2.0), rand((7, W), 32, dtype, 0.5)
    x = rand((7, W), 33, torch.float32, 3.0)
    y = 0.8 * a.double().cpu() - 1.7 * b.double().cpu()
    want = x.double().cpu() + P.unit_rms(y, 1e-5) * w.double().cpu()
    ops().rmsnorm_add(a, w, 1e-5, 1.0, x, pair=(b, 0.8, -1.7))
    close(x, want, torch.float32, "norm of a pair", tol=3e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pad", [3, 4])
@pytest.mark.parametrize("W", [5, 64, 300])
def test_five_token_shifts_keep_the_row_before(dtype, W, pad):
    """Five mixes of a row with the row before, each with its own mu, over steps of portions and single tokens in state slots
    that are not the requests' numbers; a fresh slot holds zeros."""
    n = [13, 6]
    h = [rand((n[b], W), 10 + b, dtype) for b in (0, 1)]
    mu = rand((5, W), 12, torch.float32, 0.5)
    state = torch.zeros((4, pad + W), dtype=torch.float32, device=DEV)
    slots = [2, 0]

    def fn(live, lens, starts):
        step = mini_step(lens, [slots[b] for b in live], starts)
        rows = torch.cat([h[b][s:s + c] for b, s, c in zip(live, starts, lens)])
        out = torch.empty((5, rows.shape[0], W), dtype=dtype, device=DEV)
        ops().token_shift_multi(rows, mu, state, pad, step.cu_seqlens, step.state_slots, step.req_index, step.positions, out)
        return out.permute(1, 0, 2).contiguous()

    got = in_portions(n, fn)
    for b in (0, 1):
        x = h[b].double().cpu()
        want = torch.stack([x + (P.shifted(x) - x) * mu[s].double().cpu() for s in range(5)], 1)
        close(got[b], want, dtype, f"token shifts of request {b}", tol=2e-6 if dtype == torch.float32 else 1e-2)
        assert torch.equal(state[slots[b], pad:].cpu(), h[b][-1].float().cpu())
    assert float(state[:, :pad].abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("H_,D_,pad", [(2, 16, 3), (3, 12, 3), (1, 64, 3), (4, 32, 0), (2, 128, 0), (1, 200, 4), (2, 64, 8), (1, 512, 0)])
def test_memory_with_a_decay_per_key_channel(H_, D_, pad):
    """The scan alone: states carried over portions and single tokens, in slots used in another order, against the plain
    recurrence; decays between 0.2 and 1, a bonus for the current token."""
    o = ops()
    n = [13, 6]
    HD = H_ * D_
    # (pad: the first column of r inside its rows; 0, 4, 8 keep the rows on 16-byte boundaries, which the staging by
    # asynchronous copies needs; 3 sends every element through a register)
    r, k, v = ([rand((n[b], HD + 2 * pad + 4), 20 + 5 * i + b, torch.float32, 0.7) for b in (0, 1)] for i in range(3))
    z = [rand((n[b], HD), 40 + b, torch.float32, 1.0) for b in (0, 1)]
    w0, u = rand((HD,), 42, torch.float32, 1.0) - 2.0, rand((HD,), 43)
    floats = o.decay_state_floats(H_, D_, D_)
    state = torch.zeros((3, 5 + floats), dtype=torch.float32, device=DEV)
    slots = [1, 2]

    def fn(live, lens, starts):
        step = mini_step(lens, [slots[b] for b in live], starts)
        cat = lambda xs: torch.cat([xs[b][s:s + c] for b, s, c in zip(live, starts, lens)]).contiguous()
        out = torch.empty((sum(lens), HD), dtype=torch.float32, device=DEV)
        w = o.decay_from_raw(cat(z), 0, w0)
        o.decay_scan((cat(r), pad), (cat(k), 0), (cat(v), 4 if pad != 3 else 1), (w, 0), u, state, 5, step.cu_seqlens, step.state_slots, out, H_, D_, D_)
        return out

    got = in_portions(n, fn)
    for b in (0, 1):
        dec = torch.exp(-torch.exp(z[b].double().cpu() + w0.double().cpu())).view(-1, H_, D_)
        vc = 4 if pad != 3 else 1
        rr, kk, vv = r[b][:, pad:pad + HD], k[b][:, :HD], v[b][:, vc:vc + HD]
        want = torch.stack([P.decayed_memory(rr.double().cpu().view(-1, H_, D_)[:, a], kk.double().cpu().view(-1, H_, D_)[:, a],
                                             vv.double().cpu().view(-1, H_, D_)[:, a], dec[:, a], u.double().cpu().view(H_, D_)[a])
                            for a in range(H_)], 1).reshape(-1, HD)
        close(got[b], want, torch.float32, f"memory of request {b}", tol=1e-5)
    assert float(state[0].abs().max()) == 0.0 and float(state[:, :5].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H_,D_,rank,W", [(2, 16, 8, 64), (3, 12, 5, 72), (1, 64, 1, 96), (4, 32, 16, 128)])
def test_time_mixing_in_portions_and_slots(dtype, H_, D_, rank, W):
    """The whole right-hand mixer: token shifts, five projections, the decay through its low rank and tanh, the memory, the
    norm per head, the silu gate, the output; two requests in portions, then one slot freed, zeroed and used by a third."""
    from vllm_lite_b200.parts import spec as S
    from vllm_lite_b200.parts.base import CallCache
    spec = S.TimeMixSpec(W, H_, D_, rank, 1e-5)

    def edit(t):
        t["w0"] = (t["w0"].float() * 2 - 2.0).to(dtype)
        for m in "rkvgw":
            t["mu." + m] = (t["mu." + m].float().abs().clamp(max=1.0)).to(dtype)

    part, tensors = build_part(spec, dtype, 61, edit=edit)
    need = type(part).cache_need(spec)
    state = torch.zeros((3,) + need.shape, dtype=torch.float32, device=DEV)
    n = [13, 6]
    h = [rand((n[b], W), 62 + b, dtype) for b in (0, 1)]
    slots = [2, 0]

    def fn(live, lens, starts):
        step = mini_step(lens, [slots[b] for b in live], starts)
        rows = torch.cat([h[b][s:s + c] for b, s, c in zip(live, starts, lens)]).contiguous()
        return part(rows, step, CallCache(state=state)).clone()

    got = in_portions(n, fn)
    m = dict(heads=H_, dim=D_)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for b in (0, 1):
        close(got[b], P.time_mixing(h[b].double().cpu(), tensors, m, 1e-5), dtype, f"time mixing of request {b}", tol=tol)
    state[slots[1]].zero_()                                                   # what the cache does when it hands a slot out
    h2 = rand((9, W), 70, dtype)
    out = torch.cat([part(h2[:4].contiguous(), mini_step([4], [slots[1]]), CallCache(state=state)).clone(),
                     part(h2[4:].contiguous(), mini_step([5], [slots[1]], [4]), CallCache(state=state)).clone()])
    close(out, P.time_mixing(h2.double().cpu(), tensors, m, 1e-5), dtype, "a slot used again", tol=tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H_,G_,D_,V_,every", [(4, 2, 16, 24, 4), (3, 3, 20, 6, 1), (8, 2, 64, 48, 7), (2, 1, 128, 128, 100), (1, 1, 6, 20, 3)])
def test_head_norms_query_factor_and_value_norm(dtype, H_, G_, D_, V_, every):
    """q and k heads divided by their root mean square (no weight), the query times its factor (positions on both sides of
    every step of the factor), value heads divided by theirs, k and v in the cache rows; heads padded to one size."""
    pd = -(-max(D_, V_) // 16) * 16
    pos = [0, 1, every - 1, every, every + 1, 2 * every - 1, 2 * every, 7 * every - 1, 7 * every, 1000]
    pos = [max(p, 0) for p in pos]
    T, page, coef, eps = len(pos), 4, 0.37, 1e-5
    qkv = torch.zeros((T, (H_ + 2 * G_) * pd + 5), dtype=dtype, device=DEV)
    src = rand((T, H_ + 2 * G_, pd), 80, dtype, 2.0)
    src[:, :H_ + G_, D_:] = 0
    src[:, H_ + G_:, V_:] = 0
    qkv[:, :(H_ + 2 * G_) * pd] = src.view(T, -1)
    slots = [11, 3, 7, 0, 5, 9, 1, 14, 2, 6]
    kc = torch.full((4, G_, page, pd), 7.0, dtype=dtype, device=DEV)
    vc = torch.full((4, G_, page, pd), 7.0, dtype=dtype, device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().head_norm_write(qkv, ints(pos), ints(slots), None, None, eps, D_, True, V_, (coef, every), kc, vc, H_, G_, pd, e, v_eps=eps)
    assert int(e.item()) == 0
    s64 = src.double().cpu()
    factor = torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in pos], dtype=torch.float64)
    wq = P.unit_rms(s64[:, :H_, :D_], eps) * factor[:, None, None]
    wk = P.unit_rms(s64[:, H_:H_ + G_, :D_], eps)
    wv = P.unit_rms(s64[:, H_ + G_:, :V_], eps)
    got = qkv[:, :(H_ + 2 * G_) * pd].view(T, H_ + 2 * G_, pd)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    close(got[:, :H_, :D_], wq, dtype, "queries", tol=tol)
    assert float(got[:, :H_, D_:].abs().max() if D_ < pd else 0.0) == 0.0
    for t, s in enumerate(slots):
        close(kc[s // page, :, s % page, :D_], wk[t], dtype, "cached keys", tol=tol)
        close(vc[s // page, :, s % page, :V_], wv[t], dtype, "cached values", tol=tol)
        assert float(vc[s // page, :, s % page, V_:].abs().max() if V_ < pd else 0.0) == 0.0
    untouched = sorted(set(range(16)) - set(slots))
    assert all(float(kc[s // page, 0, s % page, 0]) == 7.0 for s in untouched)


def paged(seqs, page, G_, Dp, dtype, seed):
    """Scatter every sequence's rows [n, G, Dp] (keys, values) into shuffled pages: (k cache, v cache, block table)."""
    total = sum(-(-k.shape[0] // page) for k, _ in seqs) + 3
    perm = np.random.default_rng(seed).permutation(total).tolist()
    kc = torch.full((total, G_, page, Dp), float("nan"), dtype=dtype)
    vc = torch.full((total, G_, page, Dp), float("nan"), dtype=dtype)
    table = torch.full((len(seqs), max(-(-k.shape[0] // page) for k, _ in seqs)), -1, dtype=torch.int32)
    for b, (k, v) in enumerate(seqs):
        for blk in range(-(-k.shape[0] // page)):
            pg = perm.pop()
            table[b, blk] = pg
            n = min(page, k.shape[0] - blk * page)
            kc[pg, :, :n] = k[blk * page:blk * page + n].transpose(0, 1).to(dtype)
            vc[pg, :, :n] = v[blk * page:blk * page + n].transpose(0, 1).to(dtype)
    return kc.to(DEV), vc.to(DEV), table.to(DEV)


def plain_shaped_attention(q, k, v, scale, cap, r1, r2, sink, first=0):
    """q [n, H, D] (rows before `first` are not read), k, v [n, G, D]: every row's attention over the keys up to its
    own, scores capped, less the distance bias, a sink of score 0 in the denominator."""
    n, H_, _ = q.shape
    G_ = k.shape[1]
    out = torch.zeros(n, H_, v.shape[2], dtype=torch.float64)
    for t in range(first, n):
        dist = torch.arange(t, -1, -1, dtype=torch.float64)
        for a in range(H_):
            g = a // (H_ // G_)
            s = (k[:t + 1, g] @ q[t, a]) * scale
            if cap:
                s = P.capped(s, cap)
            if r1 is not None:
                s = s - P.distance_bias(r1[a], r2[a], dist)
            out[t, a] = (P.softmax_plus_one(s) if sink else torch.softmax(s, 0)) @ v[:t + 1, g]
    return out


def shaped_case(dtype, H_, G_, D_, page, lens, new, seed=0):
    seqs = [(rand((n, G_, D_), 70 + b + seed, dtype).cpu(), rand((n, G_, D_), 72 + b + seed, dtype).cpu()) for b, n in enumerate(lens)]
    kc, vc, table = paged(seqs, page, G_, D_, dtype, 5 + seed)
    req = [b for b, c in enumerate(new) for _ in range(c)]
    pos = [p_ for n, c in zip(lens, new) for p_ in range(n - c, n)]
    q = rand((len(req), H_ * D_), 74 + seed, dtype)
    r1, r2 = rand((H_,), 75 + seed), rand((H_,), 76 + seed).abs() * 0.5 + 0.05
    return seqs, kc, vc, table, req, pos, q, r1, r2


def check_shaped(out, seqs, lens, new, req, q, H_, D_, scale, cap, r1, r2, sink, dtype, what, tol):
    T = len(req)
    for b, (n, c) in enumerate(zip(lens, new)):
        k, v = (t.double() for t in seqs[b])
        qfull = torch.zeros(n, H_, D_, dtype=torch.float64)
        mine = [t for t in range(T) if req[t] == b]
        qfull[n - c:] = q[mine].double().cpu().view(c, H_, D_)
        want = plain_shaped_attention(qfull, k, v, scale, cap, None if r1 is None else r1.double().cpu(),
                                      None if r2 is None else r2.double().cpu(), sink, first=n - c)[n - c:]
        close(out[mine].view(c, H_, D_), want, dtype, what, tol=tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cap,dist,sink", [(4.0, True, True), (0.0, True, False), (2.5, False, True), (30.0, False, False)])
@pytest.mark.parametrize("H_,G_,D_,page", [(4, 2, 16, 8), (6, 6, 32, 16), (8, 2, 64, 64), (3, 1, 48, 4), (2, 2, 128, 16)])
def test_capped_scores_distance_bias_and_unit_sink(dtype, H_, G_, D_, page, cap, dist, sink):
    """Queries of two requests (a portion of a prompt and a single token, as a mixed step brings them) over shuffled pages:
    each option on its own and together, in the kernel whose sums depend on positions alone."""
    lens, new = [150, 83], [61, 1]
    scale = 2.0 * D_ ** -0.5
    seqs, kc, vc, table, req, pos, q, r1, r2 = shaped_case(dtype, H_, G_, D_, page, lens, new)
    out = torch.empty((len(req), H_ * D_), dtype=dtype, device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().paged_attention(q, out, kc, vc, table, ints(req), ints(pos), H_, G_, D_, scale, None, e,
                          sinks=torch.zeros(H_, device=DEV) if sink else None, softcap=cap or None,
                          distance=(r1, r2) if dist else None)
    assert int(e.item()) == 0
    check_shaped(out, seqs, lens, new, req, q, H_, D_, scale, cap, r1 if dist else None, r2 if dist else None, sink, dtype,
                 "shaped attention", 2e-5 if dtype == torch.float32 else 1.5e-2)



@pytest.mark.gpu
@pytest.mark.parametrize("cap,dist,sink", [(4.0, True, True), (0.0, True, False), (2.5, False, True)])
@pytest.mark.parametrize("H_,G_,D_,page", [(4, 2, 16, 8), (6, 6, 32, 16), (8, 2, 64, 64), (3, 1, 48, 4), (2, 2, 128, 16), (40, 2, 32, 16),
                                           (9, 1, 80, 32)])
def test_tensor_core_kernels_take_the_cap_the_distance_bias_and_the_sink(H_, G_, D_, page, cap, dist, sink):
    """The bfloat16 kernels of a mixed step (tiles of a prompt's portion; single tokens, their keys split over blocks that
    merge as a cluster, through scratch, or not at all) against the plain sums and against the kernel that serves float32."""
    dtype = torch.bfloat16
    lens, new = [300, 83, 1200], [170, 1, 1]
    scale = 2.0 * D_ ** -0.5
    seqs, kc, vc, table, req, pos, q, r1, r2 = shaped_case(dtype, H_, G_, D_, page, lens, new, seed=3)
    T = len(req)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    sinks = torch.zeros(H_, device=DEV) if sink else None
    shape = dict(softcap=cap or None, distance=(r1, r2) if dist else None)
    ref = torch.empty((T, H_ * D_), dtype=dtype, device=DEV)
    ops().paged_attention(q, ref, kc, vc, table, ints(req), ints(pos), H_, G_, D_, scale, None, e, sinks=sinks, **shape)
    tiles = torch.tensor([[0, 0, 128, 130], [0, 128, 42, 258]], dtype=torch.int32, device=DEV)
    singles = ints([170, 171])
    for chunk in (64, 256, 1024):                                           # 19 chunks through scratch, 5 as a cluster, 2
        out = torch.full((T, H_ * D_), float("nan"), dtype=dtype, device=DEV)
        ops().flash_prefill(q, out, kc, vc, table, tiles, H_, G_, D_, scale, None, e, tile_rows=128, sinks=sinks, **shape)
        S, na, nm = ops().decode_attention_scratch(2, H_, D_, 1200, chunk)
        arrivals = torch.zeros(ops().flash_decode_arrivals(2, H_, G_), dtype=torch.int32, device=DEV)
        ops().flash_decode(q, out, kc, vc, table, ints(req), ints(pos), H_, G_, D_, scale, None, 1200,
                           torch.empty(na, device=DEV), torch.empty(nm, device=DEV), e, chunk=chunk, token_index=singles,
                           arrivals=arrivals, sinks=sinks, **shape)
        assert int(e.item()) == 0 and int(arrivals.abs().max()) == 0
        close(out, ref, dtype, f"against the float32 kernel, chunks of {chunk}", tol=1.5e-2)
    check_shaped(out, seqs, lens, new, req, q, H_, D_, scale, cap, r1 if dist else None, r2 if dist else None, sink, dtype,
                 "shaped attention on the tensor cores", 1.5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("cap,dist,sink", [(4.0, True, True), (0.0, True, False), (2.5, False, True)])
@pytest.mark.parametrize("H_,G_,D_,page", [(4, 2, 64, 16), (2, 1, 128, 64), (2, 2, 128, 16), (8, 2, 64, 32), (3, 3, 64, 64)])
def test_tcgen05_prompt_kernel_takes_the_cap_the_distance_bias_and_the_sink(H_, G_, D_, page, cap, dist, sink):
    """Tiles of 128 query rows of two requests' portions on the tcgen05 kernel, a portion that starts in the middle of a page
    and a tile that is not full, against the plain sums and the kernel that serves float32."""
    dtype = torch.bfloat16
    lens, new = [700, 300], [300, 129]
    scale = 2.0 * D_ ** -0.5
    seqs, kc, vc, table, req, pos, q, r1, r2 = shaped_case(dtype, H_, G_, D_, page, lens, new, seed=9)
    T = len(req)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    sinks = torch.zeros(H_, device=DEV) if sink else None
    shape = dict(softcap=cap or None, distance=(r1, r2) if dist else None)
    ref = torch.empty((T, H_ * D_), dtype=dtype, device=DEV)
    ops().paged_attention(q, ref, kc, vc, table, ints(req), ints(pos), H_, G_, D_, scale, None, e, sinks=sinks, **shape)
    tiles = torch.tensor([[0, 0, 128, 400], [0, 128, 128, 528], [0, 256, 44, 656], [1, 300, 128, 171], [1, 428, 1, 299]],
                         dtype=torch.int32, device=DEV)
    out = torch.full((T, H_ * D_), float("nan"), dtype=dtype, device=DEV)
    ops().flash_prefill_tc5(q, out, kc, vc, table, tiles, H_, G_, D_, scale, None, e, sinks=sinks, **shape)
    assert int(e.item()) == 0
    close(out, ref, dtype, "against the float32 kernel", tol=1.5e-2)
    check_shaped(out, seqs, lens, new, req, q, H_, D_, scale, cap, r1 if dist else None, r2 if dist else None, sink, dtype,
                 "shaped attention on tcgen05", 1.5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 4, 2), (16, 4, 4, 3), (6, 6, 1, 1), (6, 1, 6, 1), (12, 3, 3, 2), (5, 2, 5, 3), (9, 3, 3, 1)])
def test_choice_by_score_plus_correction_within_the_best_groups(E, top, groups, keep):
    """Negative corrections, so that every choice score lies below zero: an expert outside the kept groups must never win, as it
    would if it were masked with a zero; groups that count by their two best; weights from the scores alone, over their sum."""
    o = ops()
    T, K = 64, 32
    h = rand((T, K), 90, torch.float32)
    router = rand((E, K), 91, torch.float32, 0.5)
    corr = rand((E,), 92, torch.float32, 0.7) - 2.5
    ids = torch.empty((T, top), dtype=torch.int32, device=DEV)
    w = torch.empty((T, top), dtype=torch.float32, device=DEV)
    logits = torch.empty((o.router_slices(K), T, E), dtype=torch.float32, device=DEV)
    o.moe_route(h, router, top, ids, w, logits, "sigmoid", True, groups, keep, choice_bias=corr, group_top=2, renorm_eps=1e-20)
    want_ids, want_w = P.route(h.double().cpu(), router.cpu(), corr.cpu(), top, groups, keep)
    for t in range(T):
        assert ids[t].tolist() == want_ids[t], f"token {t}: {ids[t].tolist()} against {want_ids[t]}"
        close(w[t], want_w[t], torch.float32, "expert weights", tol=1e-5)
    if groups > 1 and keep < groups and E // groups > 1:
        # the same scores without groups pick other experts for some token: the groups are not idle
        o.moe_route(h, router, top, ids, w, logits, "sigmoid", True, 1, 1, choice_bias=corr, group_top=2, renorm_eps=1e-20)
        assert any(ids[t].tolist() != want_ids[t] for t in range(T))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,groups,keep,ff,sff,W,T", [(8, 2, 4, 2, 40, 24, 64, 37), (6, 6, 1, 1, 24, 8, 64, 5), (6, 1, 3, 1, 17, 30, 72, 37),
                                                          (16, 4, 4, 3, 64, 96, 128, 300), (4, 2, 2, 2, 9, 6, 72, 1)])
def test_experts_with_silu_gates_and_a_shared_expert(dtype, E, top, groups, keep, ff, sff, W, T):
    from vllm_lite_b200.parts import spec as S
    shared = S.GatedMlpSpec(W, sff, activation="silu", names=("gate", "up", "down"))
    spec = S.RoutedExpertsSpec(W, ff, E, top, activation="silu", score="sigmoid", renormalize=True, scale_input=False, groups=groups,
                               keep_groups=keep, choice_bias="correction", group_top=2, renorm_eps=1e-20, shared=shared)

    def edit(t):
        t["router"] = (t["router"].float() * 20).to(dtype)                  # wide gaps between the experts' scores
        t["correction"] = (t["correction"].float() * 2 - 1.0).to(dtype)

    part, tensors = build_part(spec, dtype, 8, "FEED_FORWARDS", edit)
    h = rand((T, W), 9, dtype)
    got = part(h, mini_step([T], [0]))
    f = dict(router=dict(experts=E, top=top, groups=dict(count=groups, keep=keep)))
    want = P.expert_mixture(h.double().cpu(), tensors, f)
    close(got, want, dtype, "experts", tol=2e-5 if dtype == torch.float32 else 2.5e-2)
    alone = P.gated_expert(h.double().cpu(), tensors["shared.gate"], tensors["shared.up"], tensors["shared.down"])
    assert float((want - alone).abs().max()) > 0.05 * float(want.abs().max())         # the routed experts weigh in


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ff,W,T", [(96, 64, 37), (18, 72, 5), (160, 128, 300)])
def test_dense_feed_forward_squares_what_is_above_zero(dtype, ff, W, T):
    from vllm_lite_b200.parts import spec as S
    spec = S.GatedMlpSpec(W, ff, activation="relu2", gated=False, names=("gate", "up", "down"))
    part, tensors = build_part(spec, dtype, 18, "FEED_FORWARDS")
    assert sorted(tensors) == ["down", "up"]
    h = rand((T, W), 19, dtype)
    close(part(h, mini_step([T], [0])), P.dense_ff(h.double().cpu(), tensors), dtype, "dense feed-forward")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_rank,kv_rank,rot_dim,rot,H_,D_", [(24, 40, 8, 8, 4, 16), (10, 20, 6, 6, 3, 20), (96, 16, 16, 8, 1, 32), (80, 96, 32, 32, 8, 32)])
def test_latent_norms_rotated_key_part_and_rotated_query_parts(dtype, q_rank, kv_rank, rot_dim, rot, H_, D_):
    """The row [a_q | a_kv | key part]: both norms, the key part rotated (its first `rot` features) and written behind the
    latent in the cache row; then the rotated part of every query head, in place."""
    o = ops()
    pos = [0, 1, 5, 63, 64, 1000, 4097]
    T, page, eps, base = len(pos), 4, 1e-5, 777.0
    width = -(-(kv_rank + rot_dim) // 16) * 16
    proj = rand((T, q_rank + kv_rank + rot_dim + 7), 100, dtype, 1.5)
    wq, wkv = rand((q_rank,), 101) + 1, rand((kv_rank,), 102) + 1
    inv = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device=DEV)
    cache = torch.full((2, 1, page, width), 9.0, dtype=dtype, device=DEV)
    slots = [6, 1, 4, 0, 7, 2, 5]
    cq = torch.empty((T, q_rank), dtype=dtype, device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.latent_norm_write(proj, q_rank, kv_rank, wq, wkv, eps, cq, ints(slots), cache, e, rot_dim=rot_dim, rotary=(inv, rot), positions=ints(pos))
    assert int(e.item()) == 0
    p64 = proj.double().cpu()
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    close(cq, P.plain_norm(p64[:, :q_rank], wq.cpu(), eps), dtype, "query latent", tol=tol)
    want_c = P.plain_norm(p64[:, q_rank:q_rank + kv_rank], wkv.cpu(), eps)
    want_r = P.rotate_half(p64[:, q_rank + kv_rank:q_rank + kv_rank + rot_dim], rot, base, torch.tensor(pos))
    for t, s in enumerate(slots):
        row = cache[s // page, 0, s % page]
        close(row[:kv_rank], want_c[t], dtype, "cached latent", tol=tol)
        close(row[kv_rank:kv_rank + rot_dim], want_r[t], dtype, "cached key part", tol=tol if pos[t] < 1000 else 20 * tol)
        assert float(row[kv_rank + rot_dim:].abs().max() if kv_rank + rot_dim < width else 0.0) == 0.0
    assert float(cache[0, 0, 3, 0]) == 9.0                                           # slot 3 belongs to nobody
    q = rand((T, H_ * (D_ + rot_dim)), 103, dtype)
    q0 = q.clone()
    o.rope_heads(q, D_, D_ + rot_dim, H_, inv, rot, ints(pos))
    want_q = q0.double().cpu().view(T, H_, D_ + rot_dim).clone()
    want_q[:, :, D_:] = P.rotate_half(want_q[:, :, D_:], rot, base, torch.tensor(pos))
    close(q.view(T, H_, -1)[:5], want_q[:5], dtype, "query heads", tol=tol)
    close(q.view(T, H_, -1), want_q, dtype, "query heads far out", tol=20 * tol)
    assert torch.equal(q.view(T, H_, -1)[:, :, :D_], q0.view(T, H_, -1)[:, :, :D_])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sigmoid_gate_on_the_concatenated_heads(dtype):
    x, g = rand((11, 72), 110, dtype), rand((11, 100), 111, dtype, 2.0)
    want = x.double().cpu() * torch.sigmoid(g[:, 20:92].double().cpu())
    ops().sigmoid_gate(x, g, 20)
    close(x, want, dtype, "output gate", tol=2e-6 if dtype == torch.float32 else 8e-3)


# ----------------------------------------------------------------------------------------------
# the model in the engine
# ----------------------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_whole_prompts(which, dtype):
    reqs = {f"r{i}": tokens_for(which, n, i) for i, n in enumerate([1, 2, 37, 150])}
    runner = make_runner(which, dtype, num_pages=pages_for(which, 150) + 1)
    rows = {}
    for rid, toks in reqs.items():
        rows.update(H.run_schedule(runner, [([(rid, toks, list(range(len(toks))))], [rid])]))
    assert_rows(rows, which, reqs, dtype, "whole")


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_stream_after_every_layer(which):
    from vllm_lite_b200.engine import StepEntry
    toks = tokens_for(which, 29, 5)
    runner = make_runner(which, "float32", num_pages=pages_for(which, 64))
    seen = []
    batch = runner.prepare([StepEntry("a", toks, [])])
    runner.model.forward(batch, runner.storage.call_caches, watch=lambda i, x: seen.append(x.clone().cpu()))
    runner.finish(batch)
    runner.check_device_errors()
    want = plain_run(which, toks, "float32")[1]
    assert len(seen) == len(want)
    for i, (a, b) in enumerate(zip(seen, want)):
        close(a, b, "float32", f"stream after layer {i}", tol=2e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_prompt_then_token_by_token(which, dtype):
    """Most of a prompt in one step, then single tokens (replayed from a graph) across page borders and steps of the query
    factor; and a request fed one token at a time from its first (the shifts and the memories start from zeros)."""
    toks, first = tokens_for(which, 140, 11), tokens_for(which, 12, 12)
    runner = make_runner(which, dtype, num_pages=pages_for(which, 140) + pages_for(which, 12) + 1)
    cut = 140 - 75
    schedule = [([("r", toks[:cut], [0, cut - 1])], [])] + [([("r", [toks[p]], [0])], []) for p in range(cut, 140)]
    schedule += [([("s", [first[p]], [0])], []) for p in range(12)]
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, {"r": toks, "s": first}, dtype, "decode")


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_portions_of_changing_size(which, dtype):
    toks = tokens_for(which, 171, 21)
    runner = make_runner(which, dtype, num_pages=pages_for(which, 171) + 1)
    sizes, schedule, at = [2, 37, 3, 2, 64, 1, 5, 33, 2, 22], [], 0
    for n in sizes:
        schedule.append(([("r", toks[at:at + n], [0, n - 1] if n > 1 else [0])], []))
        at += n
    assert at == 171
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, {"r": toks}, dtype, "portions")


def mixed_schedule(which):
    """Up to three live requests in three state slots: portions beside single tokens, requests that pause, end and are
    replaced, so that pages and slots change hands."""
    # (seeds chosen so that no request starts on a token whose first time-mixing output, sign(r . (u k)) v / rms(v) per head,
    # has a sum near zero: bfloat16 rounding can turn that sign, and the float32 tests hold such rows to every bit anyway)
    reqs = {k: tokens_for(which, n, 260 + i) for i, (k, n) in enumerate([("a", 90), ("b", 41), ("c", 7), ("d", 66), ("e", 30)])}
    fed = {k: 0 for k in reqs}
    plan = [[("a", 30), ("b", 2)], [("a", 1), ("b", 17), ("c", 3)], [("a", 29), ("c", 1)], [("b", 1), ("c", 3)],
            [("a", 2), ("b", 21), ("d", 40)], [("a", 28), ("d", 1)], [("d", 2), ("e", 9)], [("d", 23), ("e", 1)], [("e", 20)]]
    schedule = []
    for step in plan:
        entries, end = [], []
        for k, n in step:
            lo = fed[k]
            entries.append((k, reqs[k][lo:lo + n], sorted({0, n - 1})))
            fed[k] += n
            if fed[k] == len(reqs[k]):
                end.append(k)
        schedule.append((entries, end))
    assert all(fed[k] == len(v) for k, v in reqs.items())
    return reqs, schedule


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_mixed_batches_with_pages_and_slots_used_again(which, dtype):
    reqs, schedule = mixed_schedule(which)
    runner = make_runner(which, dtype, num_pages=pages_for(which, 90) + pages_for(which, 66) + pages_for(which, 41) + 1, max_requests=3)
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, reqs, dtype, "mixed")
    assert runner.cache.slots.free_count == 3


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_cuts_and_batches_agree_bitwise_in_float32(which):
    reqs, schedule = mixed_schedule(which)
    runner = make_runner(which, "float32", num_pages=4 * pages_for(which, 90), max_requests=3)
    mixed = H.run_schedule(runner, schedule)
    for rid, toks in reqs.items():
        alone = H.run_schedule(runner, [([(rid, toks, list(range(len(toks))))], [rid])])
        for (r, pos), row in mixed.items():
            if r == rid:
                assert torch.equal(row, alone[(r, pos)]), f"{rid} position {pos} depends on the batch or the cut"


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "C", "D"])
def test_steps_of_the_query_factor_show_in_the_logits(which):
    """Sharp scores: a query factor that steps one position earlier or later moves the logits by far more than the
    tolerance in the plain implementation, and the engine agrees with the right one, in prompts and in decoding."""
    sharp = 6.0
    toks = tokens_for(which, 150, 33)
    right = plain_run(which, toks, "float32", sharp)[0]
    for off in (-1, 1):
        wrong = plain_run(which, toks, "float32", sharp, every=off)[0]
        gap = float((wrong - right).abs().max()) / float(right.abs().max())
        assert gap > 30 * TOL["float32"], f"a factor that steps {off} off would not show ({gap:.2e})"
    runner = make_runner(which, "float32", num_pages=pages_for(which, 150) + 1, sharp=sharp)
    schedule = [([("r", toks[:60], list(range(60)))], [])] + [([("r", [toks[p]], [0])], []) for p in range(60, 150)]
    assert_rows(H.run_schedule(runner, schedule), which, {"r": toks}, "float32", "factor steps", sharp, loosen=2.0)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H_,G_,D_,page", [(8, 2, 64, 64), (4, 4, 32, 16), (2, 1, 128, 8)])
@pytest.mark.parametrize("n,far", [(700, 3), (700, 63), (700, 64), (513, 0), (1300, 640), (1300, 1299 - 1024)])
def test_one_far_key_among_hundreds(dtype, H_, G_, D_, page, n, far):
    """One key far back (at a page's first or last row, at the sequence's first token) whose score stands out although the
    distance bias takes ln(1 + b d) a off it: its value, a marker, must show in the output of the last query, read as the
    last row of a portion and as a single token; without that key the marker is absent."""
    scale = 1.0
    k = rand((n, G_, D_), 120, dtype, 0.05).cpu()
    v = rand((n, G_, D_), 121, dtype, 0.05).cpu()
    q_last = rand((H_, D_), 122, dtype, 0.05).cpu()
    k[far] = 0
    k[far, :, 0] = 6.0
    q_last[:, 0] = 5.0                                             # score 30 before the cap of 25 and the bias
    v[far] = 0
    v[far, :, 1] = 40.0                                            # the marker
    r1 = torch.full((H_,), 1.5, device=DEV)
    r2 = torch.full((H_,), 0.25, device=DEV)
    kc, vc, table = paged([(k, v)], page, G_, D_, dtype, 7)
    for new in (1, 37):
        pos = list(range(n - new, n))
        q = rand((new, H_ * D_), 123, dtype, 0.05)
        q[-1] = q_last.view(-1).to(DEV)
        out = torch.empty((new, H_ * D_), dtype=dtype, device=DEV)
        e = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops().paged_attention(q, out, kc, vc, table, ints([0] * new), ints(pos), H_, G_, D_, scale, None, e,
                              sinks=torch.zeros(H_, device=DEV), softcap=25.0, distance=(r1, r2))
        assert int(e.item()) == 0
        qfull = torch.zeros(n, H_, D_, dtype=torch.float64)
        qfull[n - new:] = q.double().cpu().view(new, H_, D_)
        want = plain_shaped_attention(qfull, k.double(), v.double(), scale, 25.0, r1.double().cpu(), r2.double().cpu(), True, first=n - 1)[-1]
        assert float(want[:, 1].min()) > 10.0                      # the far key holds most of the weight
        close(out[-1].view(H_, D_), want, dtype, f"far key at {far} of {n}, {new} new", tol=2e-5 if dtype == torch.float32 else 2e-2)
        if dtype == torch.bfloat16:                                # the tensor-core kernels: tiles of the portion, or the single token
            out2 = torch.full((new, H_ * D_), float("nan"), dtype=dtype, device=DEV)
            shape = dict(sinks=torch.zeros(H_, device=DEV), softcap=25.0, distance=(r1, r2))
            if new > 1:
                tiles = torch.tensor([[0, 0, new, n - new]], dtype=torch.int32, device=DEV)
                ops().flash_prefill(q, out2, kc, vc, table, tiles, H_, G_, D_, scale, None, e, tile_rows=128, **shape)
            else:
                S, na, nm = ops().decode_attention_scratch(1, H_, D_, n, 256)
                arrivals = torch.zeros(ops().flash_decode_arrivals(1, H_, G_), dtype=torch.int32, device=DEV)
                ops().flash_decode(q, out2, kc, vc, table, ints([0]), ints(pos), H_, G_, D_, scale, None, n, torch.empty(na, device=DEV),
                                   torch.empty(nm, device=DEV), e, chunk=256, arrivals=arrivals, **shape)
            assert int(e.item()) == 0
            close(out2[-1].view(H_, D_), want, dtype, f"far key at {far} of {n}, {new} new, tensor cores", tol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["B", "C"])
def test_long_prompt_whole_against_portions(which):
    """A prompt of 2,300 tokens in one step (the products, the experts and the attention of many rows run on their kernels
    for long steps) against the same prompt in portions of a few hundred tokens and of two: bfloat16 both, so they agree to
    rounding; float32 bit for bit.  The last positions read keys thousands of positions back."""
    from vllm_lite_b200.engine import ModelRunner, load_model_dir
    n = 2300
    toks = tokens_for(which, n, 71)
    want = sorted(set(range(0, n, 97)) | set(range(n - 8, n)))
    for dtype in ("bfloat16", "float32"):
        _, plan, weights = load_model_dir(model_dir(which, store_of(dtype)), dtype, DEV)
        runner = ModelRunner(plan, weights, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32, device=DEV,
                             page_size=PAGE[which], num_pages=pages_for(which, n) + 2, max_requests=2, max_context=4096)
        whole = H.run_schedule(runner, [([("w", toks, want)], ["w"])])
        cuts, schedule, at = [300, 411, 2, 600, 87, 900], [], 0
        for c in cuts:
            schedule.append(([("p", toks[at:at + c], [p - at for p in want if at <= p < at + c])], []))
            at += c
        assert at == n
        parts = H.run_schedule(runner, schedule)
        errs = []
        for p in want:
            a, b = whole[("w", p)], parts[("p", p)]
            if dtype == "float32":
                assert torch.equal(a, b), f"{which}: position {p} depends on the cut"
            errs.append(float((a - b).abs().max()) / max(float(b.abs().max()), 1e-12))
        if dtype == "bfloat16":
            errs.sort()
            assert errs[len(errs) // 2] <= TOL[dtype] and errs[int(0.8 * len(errs))] <= 2 * TOL[dtype], errs[-5:]
        del runner


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """300 tokens one by one after a prompt of four: the memories, the shifts and the caches carry every token."""
    which, length = "D", 300
    toks = tokens_for(which, length, 31)
    runner = make_runner(which, dtype, num_pages=pages_for(which, length) + 1)
    schedule = [([("r", toks[:4], [3])], [])] + [([("r", [toks[p]], [0])], []) for p in range(4, length)]
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, {"r": toks}, dtype, "long decode")


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "C"])
def test_greedy_generation_through_the_engine(which):
    from vllm_lite_b200 import LLMEngine
    prompts = [tokens_for(which, n, 50 + i) for i, n in enumerate([5, 17, 33, 64])]
    eng = LLMEngine(str(model_dir(which, "float32")), dtype="float32", kv_blocks=64, block_size=PAGE[which],
                    max_batch_size=3, max_num_batched_tokens=48, prefill_chunk_size=13, max_model_len=256)
    outs = eng.generate(prompts, max_tokens=20)
    for p, o in zip(prompts, outs):
        toks = list(p)
        assert len(o) == 20
        for t in o:
            row = plain_run(which, toks, "float32")[0][-1]
            assert int(row.argmax()) == t or float(row.max() - row[t]) < 1e-4 * float(row.abs().max())
            toks.append(t)
    assert eng.stats()["finished"] == len(prompts)


@pytest.mark.gpu
def test_greedy_generation_bfloat16_with_the_cache_sized_from_memory():
    """kv_blocks=None: pools and state slots are sized from the GPU's free memory; the tokens the bfloat16 engine picks lie
    at or near the plain implementation's maximum."""
    from vllm_lite_b200 import LLMEngine
    which = "C"
    prompts = [tokens_for(which, n, 80 + i) for i, n in enumerate([9, 70])]
    eng = LLMEngine(str(model_dir(which, "bfloat16")), dtype="bfloat16", kv_blocks=None, block_size=PAGE[which], max_batch_size=4,
                    max_model_len=256)
    outs = eng.generate(prompts, max_tokens=10)
    far = 0
    for p, o in zip(prompts, outs):
        toks = list(p)
        assert len(o) == 10
        for t in o:
            row = plain_run(which, toks, "bfloat16")[0][-1]
            far += float(row.max() - row[t]) > 2 * TOL["bfloat16"] * float(row.abs().max())
            toks.append(t)
    assert far <= 2


@pytest.mark.gpu
def test_command_line_and_replay_program(tmp_path):
    """The command line writes a folder from config.json and generates from it (greedy, float32: the plain implementation's
    tokens); bin/trace_run replays steps on the folder: a portion, then a portion beside another request's, then one token."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(CONFIGS["D"]))
    folder = tmp_path / "model"
    run = lambda *a, **k: subprocess.run([sys.executable, *a], capture_output=True, text=True, cwd=root, timeout=900, **k)
    made = run("-m", "vllm_lite_b200", "init", "--config", str(cfg), "--out", str(folder), "--seed", "5", "--std", "0.08")
    assert made.returncode == 0, made.stderr[-2000:]
    prompt = tokens_for("D", 14, 77)
    out = run("-m", "vllm_lite_b200", "--model", str(folder), "--dtype", "float32", "--kv-blocks", "32", "--max-tokens", "6",
              "--prompt-ids", ",".join(map(str, prompt)), "--log-level", "warn")
    assert out.returncode == 0, out.stderr[-2000:]
    got = [int(t) for t in out.stdout.strip().split(",")]
    pc, pw = P.read_model_dir(folder)
    toks = list(prompt)
    for t in got:
        row = P.forward(pc, pw, toks)[0][-1]
        assert int(row.argmax()) == t or float(row.max() - row[t]) < 1e-4 * float(row.abs().max())
        toks.append(t)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": prompt[:9], "want": [8]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": prompt[9:], "want": [0, 4]}, {"id": "b", "tokens": [3, 1], "want": []}],
              "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": [4], "want": [0]}], "end": ["b"]}]
    outdir = tmp_path / "logits"
    rep = run(str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(outdir),
              "--max-tokens", "64", "--page-size", "8", input="".join(json.dumps(x) + "\n" for x in steps))
    assert rep.returncode == 0, rep.stderr[-2000:]
    assert [l for l in rep.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = P.forward(pc, pw, prompt)[0].float()
    rows = np.fromfile(outdir / "1.f32", dtype="<f4").reshape(2, CONFIGS["D"]["vocab"])
    for row, pos in zip(rows, (9, 13)):
        assert float(np.abs(row - ref[pos].numpy()).max()) <= TOL["float32"] * float(ref[pos].abs().max())
    last = np.fromfile(outdir / "2.f32", dtype="<f4")
    refb = P.forward(pc, pw, [3, 1, 4])[0].float()[2].numpy()
    assert float(np.abs(last - refb).max()) <= TOL["float32"] * float(np.abs(refb).max())
