"""The Sodonex decoder in the engine against the plain implementation (tests/plain_sodonex.py).

Small configurations of their own that differ in every size, per layer too (heads, head sizes that are no multiple of
16, taps, blocks of the mask shorter than a page, equal to one, across page borders and longer than any prompt, partial
and full rotation, a layer without a feed-forward) and in every constant, also values that are 1 (one tap, a block of
one position, one expert chosen, every expert chosen, one head, factors of 1).  Seeded random weights with edits where
random numbers would hide a fault: routers with wide gaps, sharp scores so that one key more or less at a block's edge
moves the logits, one far key made to stand out among hundreds.  Each mechanism alone against one function of the plain
implementation, with state carried across steps and slots; then whole prompts, the stream after every layer, decoding
token by token, portions down to two tokens, mixed batches with pages and slots used again, long decoding, and greedy
generation through the engine's entry point, the command line and the replay program.
"""
import copy
import functools
import json

import numpy as np
import pytest
import torch

import helpers as H
import plain_sodonex as P

DEV = "cuda:0"


def mixer(heads, kv, dim, conv, scale, size, rot, base):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, conv=conv, scale=scale, mask=dict(size=size),
                rot=dict(dims=rot, base=base))


def moe(ff, experts, top):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def layer(mix, mlp):
    return dict(type="attention", mixer=mix, mlp=mlp)


def model(vocab, width, eps, emb, mult, layers):
    return dict(architecture="Sodonex", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=emb),
                residual_mult=mult, layers=layers)


# A: every layer its own sizes; blocks of 7 positions (shorter than a page of 8), of 20 (across pages) and of 33; a head
#    of 24 numbers (padded to 32 for the kernels) that is rotated whole; a layer without a feed-forward; one expert chosen.
# B: the values that are 1: ONE tap (a convolution without memory), a block of ONE position (a token reads itself alone),
#    every expert chosen, one head, factors 1; as many key heads as query heads; a block longer than any prompt.
# C: pages of 64 positions, heads of 64 numbers, blocks of 70 (across a page border), of 64 (a page) and of 128.
# D: sizes that are multiples of two at best: heads of 20 and of 6 numbers, three rotated pairs, an expert width of 20
#    and of 9, a width of 72, pages of 4.
CONFIGS = {
    "A": model(150, 64, 1e-5, 3.0, 0.7,
               [layer(mixer(4, 2, 16, 3, 0.3, 7, 8, 10000.0), moe(40, 6, 2)),
                layer(mixer(2, 1, 24, 2, 0.2, 20, 24, 500.0), None),
                layer(mixer(3, 3, 16, 4, 0.25, 33, 4, 77.0), moe(24, 4, 1))]),
    "B": model(211, 96, 3e-6, 1.0, 1.0,
               [layer(mixer(6, 6, 32, 1, 0.18, 1, 32, 500000.0), moe(48, 5, 5)),
                layer(mixer(1, 1, 48, 5, 0.15, 100, 16, 1234.0), moe(32, 8, 3)),
                layer(mixer(4, 1, 16, 3, 0.3, 4096, 2, 9.0), None)]),
    "C": model(301, 128, 1e-6, 11.0, 0.5,
               [layer(mixer(8, 2, 64, 4, 0.11, 70, 32, 300000.0), moe(64, 8, 2)),
                layer(mixer(4, 4, 64, 2, 0.1, 64, 64, 10000.0), moe(96, 4, 3)),
                layer(mixer(2, 1, 128, 4, 0.09, 128, 64, 1e6), None)]),
    "D": model(97, 72, 2e-5, 0.5, 1.3,
               [layer(mixer(6, 3, 20, 2, 0.22, 5, 6, 50.0), moe(20, 5, 4)),
                layer(mixer(4, 2, 6, 6, 0.4, 9, 6, 3.0), moe(9, 3, 2))]),
}
PAGE = {"A": 8, "B": 16, "C": 64, "D": 4}
SEED = {"A": 41, "B": 42, "C": 43, "D": 44}
# max |engine - plain| / max |plain| over a row of logits; float32 stays near 1e-6 at these sizes, bfloat16 near 1e-2
TOL = {"float32": 3e-5, "bfloat16": 4e-2}
CASES = [(w, d) for w in ("A", "B", "C", "D") for d in ("float32", "bfloat16")]


def edited(cfg, sharp=1.0, block=0):
    """The same model with every attention scale multiplied (weights near 0 or 1) and every block of the mask resized."""
    cfg = copy.deepcopy(cfg)
    for l in cfg["layers"]:
        l["mixer"]["scale"] *= sharp
        l["mixer"]["mask"]["size"] = max(1, l["mixer"]["mask"]["size"] + block)
    return cfg


def store_of(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


@functools.lru_cache(maxsize=None)
def model_dir(which, store="bfloat16", sharp=1.0):
    """A folder with the configuration and seeded weights; the routers are widened so that no test rests on a close call
    between two experts, and the sigmoid's bias per head is moved below zero so that a key weighs little unless its
    score is large."""
    from vllm_lite_b200.weights import write_model_dir
    from vllm_lite_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    cfg = edited(CONFIGS[which], sharp)
    d = H.tmp_root() / f"sodonex_{which}_{store}_{sharp}"
    write_model_dir(d, cfg, SEED[which], std=0.08, dtype=torch.float32 if store == "float32" else torch.bfloat16)
    f = SafetensorsFile(d / "model.safetensors")
    tensors = {n: f.read(n).clone() for n in f.names()}
    f.close()
    for name, t in tensors.items():
        if name.endswith(".mlp.router"):
            tensors[name] = (t.float() * 15.0).to(t.dtype)
        if name.endswith(".mix.pb"):
            tensors[name] = (t.float() - 1.0).to(t.dtype)
    write_safetensors(d / "model.safetensors", tensors, metadata={"format": "pt"})
    return d


@functools.lru_cache(maxsize=None)
def plain_model(which, store, sharp=1.0):
    return P.read_model_dir(model_dir(which, store, sharp))


_plain = {}


def plain_run(which, tokens, dtype, sharp=1.0, block=0):
    key = (which, store_of(dtype), sharp, block, tuple(tokens))
    if key not in _plain:
        cfg, w = plain_model(which, store_of(dtype), sharp)
        logits, after = P.forward(edited(cfg, 1.0, block), w, list(tokens))
        _plain[key] = (logits.float(), [a.float() for a in after])
    return _plain[key]


def tokens_for(which, length, seed):
    rng = np.random.default_rng(7000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[which]["vocab"], size=length)]


def make_runner(which, dtype, num_pages, sharp=1.0, page_size=None, max_requests=4, max_context=1024, **kw):
    from vllm_lite_b200.engine import ModelRunner, load_model_dir
    _, plan, weights = load_model_dir(model_dir(which, store_of(dtype), sharp), dtype, DEV)
    return ModelRunner(plan, weights, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32, device=DEV,
                       page_size=page_size or PAGE[which], num_pages=num_pages, max_requests=max_requests,
                       max_context=max_context, **kw)


def assert_rows(rows, which, requests, dtype, what, sharp=1.0, loosen=1.0):
    """float32: every row within the tolerance.  bfloat16: a row's rounding can change which expert a router takes where
    two logits lie close (one chosen expert of four, three of eight), and then that row and those that read it differ
    by far more than rounding; up to a twentieth of the rows may, the mechanisms' own tests hold every row."""
    assert rows, "nothing was compared"
    worst, errs = 0.0, []
    for (rid, pos), row in rows.items():
        ref = plain_run(which, requests[rid], dtype, sharp)[0][pos]
        err = float((row - ref).abs().max()) / max(float(ref.abs().max()), 1e-12)
        if dtype == "float32":
            assert err <= loosen * TOL[dtype], f"{what} {which}/{dtype}: request {rid} position {pos}: {err:.3e}"
        errs.append(err)
    over = [e for e in errs if e > loosen * TOL[dtype]]
    assert len(over) <= len(errs) // 20, f"{what} {which}/{dtype}: {len(over)} of {len(errs)} rows, worst {max(errs):.3e}"
    errs.sort()
    worst = errs[len(errs) - 1 - len(errs) // 20]
    key = ("sodonex " + what, which, dtype)
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
    assert (cfg.vocab_size, cfg.hidden_size, cfg.eps, cfg.embedding_scale, cfg.residual_mult) == (150, 64, 1e-5, 3.0, 0.7)
    assert plan.embedding.scale == 3.0 and plan.final_norm.scalar and not plan.tie_word_embeddings
    b0, b1, b2 = plan.layers
    assert all(b.kind == "post_norm" and b.residual_mult == 0.7 and b.norm1.scalar for b in plan.layers)
    a0, a1, a2 = (b.mixer.inner for b in plan.layers)
    assert all(b.mixer.kind == "token_shift" and b.mixer.hidden_size == 64 for b in plan.layers)
    assert (a0.num_heads, a0.num_kv_heads, a0.head_dim, a0.conv, a0.scale, a0.chunk) == (4, 2, 16, 3, 0.3, 7)
    assert (a0.position.head_dim, a0.position.dim, a0.position.theta, a0.position.interleaved) == (16, 8, 10000.0, False)
    assert (a1.num_heads, a1.num_kv_heads, a1.head_dim, a1.conv, a1.chunk, a1.position.dim, a1.position.theta) == (2, 1, 24, 2, 20, 24, 500.0)
    assert (a2.num_heads, a2.num_kv_heads, a2.conv, a2.chunk, a2.scale) == (3, 3, 4, 33, 0.25)
    assert a0.weighting == "sigmoid" and a0.gate and a0.head_bias and a0.bias and a0.out_bias and a0.window is None
    assert b1.ffn is None and (b0.ffn.num_experts, b0.ffn.top, b0.ffn.intermediate_size) == (6, 2, 40)
    assert (b2.ffn.num_experts, b2.ffn.top) == (4, 1)
    f = b0.ffn
    assert (f.gated, f.activation, f.score, f.renormalize, f.scale_input, f.router_bias) == (False, "relu2", "softmax", True, False, ".b")
    names = declare_model(plan)
    assert names["embed"].shape == (150, 64) and names["head"].shape == (150, 64) and names["final.norm"].shape == ()
    assert names["l0.norm1"].shape == () and names["l0.norm2"].shape == () and names["l0.shift"].shape == (64,)
    assert names["l0.mix.q"].shape == (64, 64) and names["l0.mix.k"].shape == (32, 64) and names["l0.mix.q.b"].shape == (64,)
    assert names["l0.mix.q.conv"].shape == (64, 3) and names["l0.mix.k.conv"].shape == (32, 3) and names["l0.mix.k.norm"].shape == (32,)
    assert names["l0.mix.g"].shape == (4, 64) and names["l0.mix.pb"].shape == (4,) and names["l0.mix.o.b"].shape == (64,)
    assert names["l1.mix.o"].shape == (64, 48) and "l1.mlp.router" not in names and "l1.norm2" not in names and "l0.mix.v" not in names
    assert names["l2.mlp.e3.up"].shape == (24, 64) and names["l2.mlp.e3.down"].shape == (64, 24) and "l2.mlp.e0.gate" not in names
    assert names["l0.mlp.router"].shape == (6, 64) and names["l0.mlp.router.b"].shape == (6,)


def test_config_errors_name_the_field():
    from vllm_lite_b200.config import InvalidField, MissingField, plan_from_config_json
    bad = copy.deepcopy(CONFIGS["A"])
    del bad["layers"][1]["mixer"]["mask"]
    with pytest.raises(MissingField, match=r"layers\[1\]\.mixer\.mask"):
        plan_from_config_json(bad)
    bad = copy.deepcopy(CONFIGS["A"])
    bad["layers"][2]["type"] = "something_else"
    with pytest.raises(InvalidField, match=r"layers\[2\]\.type"):
        plan_from_config_json(bad)
    bad = copy.deepcopy(CONFIGS["A"])
    bad["layers"][0]["mlp"]["router"]["top"] = 7
    with pytest.raises(InvalidField, match="router"):
        plan_from_config_json(bad)
    bad = copy.deepcopy(CONFIGS["A"])
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    with pytest.raises(InvalidField, match="kv_heads"):
        plan_from_config_json(bad)
    bad = copy.deepcopy(CONFIGS["A"])
    bad["layers"][0]["mixer"]["rot"]["dims"] = 18
    with pytest.raises(InvalidField, match=r"rot\.dims"):
        plan_from_config_json(bad)
    bad = copy.deepcopy(CONFIGS["A"])
    bad["layers"][0]["mixer"]["vdim"] = 24                                  # the values are the keys
    with pytest.raises(InvalidField, match="vdim"):
        plan_from_config_json(bad)
    for key in ("embedding", "residual_mult", "norm", "vocab", "width"):
        bad = copy.deepcopy(CONFIGS["A"])
        del bad[key]
        with pytest.raises(MissingField, match=key):
            plan_from_config_json(bad)


def test_a_layer_holds_pages_and_two_rows_of_state_and_blocks_give_pages_back():
    from vllm_lite_b200.cache import CacheManager, FixedState, PagedKV, Several
    from vllm_lite_b200.cache.manager import CacheLayout
    from vllm_lite_b200.config import plan_from_config_json
    from vllm_lite_b200.parts.model import cache_needs
    _, plan = plan_from_config_json(CONFIGS["A"])
    needs = cache_needs(plan)
    assert all(isinstance(n, Several) and len(n.parts) == 3 for n in needs)
    assert needs[0].parts == (FixedState((64,)), PagedKV(2, 16, None, 7), FixedState((2 * (64 + 32),)))
    assert needs[1].parts[1] == PagedKV(1, 32, None, 20) and needs[1].parts[2] == FixedState((1 * (48 + 24),))
    _, plan_b = plan_from_config_json(CONFIGS["B"])
    assert cache_needs(plan_b)[0].parts[2] == FixedState((1,))             # one tap keeps nothing
    layout = CacheLayout.from_needs(needs, [None] * 3)
    mgr = CacheManager(layout, page_size=8, num_pages=12, max_requests=2)
    mgr.admit("a")
    mgr.append("a", 45)
    mgr.release_behind_window("a")
    held = sorted(sum(p >= 0 for p in t) for t in mgr.requests["a"].block_tables)
    # the next query sits at 45: blocks of 7 start at 42 (page 5 of 0..5 stays), of 20 at 40 (page 5), of 33 at 33 (pages 4, 5)
    assert held == [1, 1, 2]
    mgr.check_invariants()


def test_plain_pieces_behave():
    x = torch.arange(12, dtype=torch.float64).view(6, 2) + 1
    w = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)
    y = P.short_conv(x, w)
    assert torch.equal(y[:, 0], x[:, 0]) and y[:2, 1].tolist() == [0.0, 0.0] and torch.equal(y[2:, 1], x[:-2, 1])
    s = P.token_shift(x, torch.tensor([0.0, 1.0]))
    assert torch.equal(s[:, 0], x[:, 0]) and s[0, 1] == 0.0 and torch.equal(s[1:, 1], x[:-1, 1])
    q = torch.randn(5, 2, 8, dtype=torch.float64)
    r = P.rotate_half(q, 4, 100.0)
    assert torch.allclose(r[0], q[0]) and torch.equal(r[:, :, 4:], q[:, :, 4:])
    assert torch.allclose(r[:, :, 0] ** 2 + r[:, :, 2] ** 2, q[:, :, 0] ** 2 + q[:, :, 2] ** 2)       # i turns with i + dims / 2
    assert [P.chunk_visible(8, j, 4) for j in (7, 8, 9)] == [False, True, False] and P.chunk_visible(7, 4, 4)
    n = P.scalar_norm(torch.tensor([[3.0, 4.0]], dtype=torch.float64), torch.tensor(2.0), 0.0)
    assert torch.allclose(n, torch.tensor([[3.0, 4.0]], dtype=torch.float64) * 2 / (12.5 ** 0.5))
    # weights are not summed to one: two equal keys weigh twice one key
    k = torch.ones(2, 1, 4, dtype=torch.float64)
    o = P.sigmoid_chunk_weights(k.clone(), k, k, torch.zeros(1), 0.0, 8)
    assert torch.allclose(o[0], torch.full((1, 4), 0.5, dtype=torch.float64)) and torch.allclose(o[1], torch.ones(1, 4, dtype=torch.float64))
    # top 2 of logits (1, 3, 2) + bias (0, 0, 5): experts 2 and 1, weights softmax(7, 3)
    h = torch.eye(4, dtype=torch.float64)[:1]
    p = {"router": torch.tensor([[1.0, 0, 0, 0], [3.0, 0, 0, 0], [2.0, 0, 0, 0]]), "router.b": torch.tensor([0.0, 0.0, 5.0])}
    for e in range(3):
        p[f"e{e}.up"] = torch.full((2, 4), float(e + 1))
        p[f"e{e}.down"] = torch.ones(4, 2)
    out = P.squared_relu_experts(h, p, dict(router=dict(experts=3, top=2)))
    sw = torch.softmax(torch.tensor([7.0, 3.0], dtype=torch.float64), 0)
    assert abs(float(out[0, 0]) - 2 * (float(sw[0]) * 9 + float(sw[1]) * 4)) < 1e-12
    p["e1.up"] = -p["e1.up"]                                                 # below zero: the square of max(v, 0) is 0
    out = P.squared_relu_experts(h, p, dict(router=dict(experts=3, top=2)))
    assert abs(float(out[0, 0]) - 2 * float(sw[0]) * 9) < 1e-12


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


# portions of two requests of 13 and 6 tokens: single tokens, portions shorter than any convolution, one request pausing
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


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pad", [3, 4])
@pytest.mark.parametrize("W", [5, 64, 300, 2048])
def test_token_shift_keeps_the_row_before(dtype, W, pad):
    """Two requests in portions, in swapped state rows of which one holds leftovers of an earlier request until it is
    cleared: every mixed row equals the whole sequence's, and a first token is mixed with zeros.  `pad` floats lie
    before the row in the state: with 4 of them the rows start on 16 bytes (the kernel's wide accesses), with 3 not."""
    n = [13, 6]
    x = [rand((n[b], W), 50 + b, scale=2.0) for b in (0, 1)]
    mu = rand((W,), 52, scale=0.5) + 0.5
    want = [P.token_shift(x[b].double().cpu(), mu.cpu()) for b in (0, 1)]
    state = torch.zeros((2, pad + W), device=DEV)

    def step(live, lens, starts):
        s = mini_step(lens, [1 - b for b in live], starts)
        xin = torch.cat([x[b][a:a + c] for b, a, c in zip(live, starts, lens)]).contiguous()
        out = torch.empty((xin.shape[0], W), dtype=dtype, device=DEV)
        ops().token_shift(xin, mu, state, pad, s.cu_seqlens, s.state_slots, s.req_index, s.positions, out)
        return out.float()

    got = in_portions(n, step)
    for b in (0, 1):
        close(got[b], want[b], dtype, "token shift", tol=1e-6 if dtype == torch.float32 else 8e-3)
        assert torch.equal(state[1 - b, pad:], x[b][-1])                      # the last row a request brought
    assert float(state[:, :pad].abs().max()) == 0.0
    close(got[0][0], (x[0][0].double() * (1 - mu.double())).cpu(), dtype, "a first token", tol=1e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("in_bias", [False, True])
@pytest.mark.parametrize("taps,C", [(1, 5), (2, 40), (4, 33), (6, 128)])
def test_convolution_without_bias_or_activation(taps, C, in_bias):
    """`in_bias`: the bias of the product that made the rows, added by the kernel as it reads them (zeros before a
    sequence's start stay zeros, the state keeps the rows with it)."""
    n = [13, 6]
    x = [rand((n[b], C + 3), 40 + b) for b in (0, 1)]
    w = rand((C, taps), 42)
    ib = rand((C,), 43) if in_bias else None
    want = [P.short_conv(x[b][:, 2:2 + C].double().cpu() + (ib.double().cpu() if in_bias else 0.0), w.cpu()) for b in (0, 1)]
    state = torch.zeros((2, 7 + max((taps - 1) * C, 1)), device=DEV)

    def step(live, lens, starts):
        s = mini_step(lens, [1 - b for b in live], starts)
        xin = torch.cat([x[b][a:a + c] for b, a, c in zip(live, starts, lens)]).contiguous()
        out = torch.empty((xin.shape[0], C), device=DEV)
        ops().short_conv(xin, 2, C, w, None, state, 7, s.cu_seqlens, s.state_slots, out, act=False, in_bias=ib)
        return out

    got = in_portions(n, step)
    for b in (0, 1):
        close(got[b], want[b], torch.float32, "short convolution")
    assert float(state[:, :7].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H_,G_,D_,rot,base", [(4, 2, 16, 8, 10000.0), (2, 1, 24, 24, 500.0), (3, 3, 20, 6, 50.0),
                                               (8, 2, 64, 32, 200000.0), (1, 1, 128, 2, 7.0), (40, 8, 64, 32, 10000.0)])
def test_whole_row_norm_rotation_and_cache_rows(dtype, H_, G_, D_, rot, base):
    """q and k are normed over the WHOLE row (a norm per head would be far off: the heads are given unequal sizes), the
    first `rot` features of every head turn by the position, the values are the keys as they came, and padded features
    are zeros.  (Angles of hundreds of radians made of float32 factors: 1e-4 of the largest number in float32.)"""
    T, page, eps = 11, 4, 1e-5
    Dp = -(-D_ // 16) * 16
    qk = rand((T, (H_ + G_) * D_ + 2), 60)
    qk[:, :D_] *= 5.0                                                       # one head far larger than the others
    qw, kw = rand((H_ * D_,), 61) + 1.5, rand((G_ * D_,), 62) + 1.5
    pos = [100 + 37 * t for t in range(T)]
    slots = [3 * page + t for t in range(T)]
    inv = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device=DEV)
    q_out = torch.full((T, H_ * Dp), 7.0, dtype=dtype, device=DEV)
    kc = torch.full((8, G_, page, Dp), 7.0, dtype=dtype, device=DEV)
    vc = torch.full((8, G_, page, Dp), 7.0, dtype=dtype, device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().rows_norm_rope_write(qk, ints(pos), ints(slots), qw, kw, eps, inv, rot, q_out, kc, vc, H_, G_, D_, e, padded_head_dim=Dp)
    assert int(e.item()) == 0
    q64, k64 = qk[:, :H_ * D_].double().cpu(), qk[:, H_ * D_:(H_ + G_) * D_].double().cpu()

    def turned(u, w, heads):
        full = torch.zeros(max(pos) + 1, heads, D_, dtype=torch.float64)
        full[pos] = P.whole_row_norm(u, w.cpu(), eps).view(T, heads, D_)
        return P.rotate_half(full, rot, base)[pos]

    close(q_out.view(T, H_, Dp)[:, :, :D_], turned(q64, qw, H_), dtype, "queries", tol=1e-4 if dtype == torch.float32 else 8e-3)
    rows = lambda c: torch.stack([c[s // page, :, s % page] for s in slots])            # [T, G, Dp]
    close(rows(kc)[:, :, :D_], turned(k64, kw, G_), dtype, "keys", tol=1e-4 if dtype == torch.float32 else 8e-3)
    close(rows(vc)[:, :, :D_], k64.view(T, G_, D_), dtype, "values", tol=1e-7 if dtype == torch.float32 else 8e-3)
    if Dp != D_:
        assert float(q_out.view(T, H_, Dp)[:, :, D_:].abs().max()) == 0.0 and float(rows(kc)[:, :, D_:].abs().max()) == 0.0 \
            and float(rows(vc)[:, :, D_:].abs().max()) == 0.0
    if H_ > 1:
        per_head = P.unit_rms(q64.view(T, H_, D_), eps).reshape(T, -1) * qw.double().cpu()
        assert float((per_head - P.whole_row_norm(q64, qw.cpu(), eps)).abs().max()) > 0.3


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H_,G_,D_,rot,taps", [(4, 2, 16, 8, 3), (2, 1, 24, 24, 1), (3, 3, 20, 6, 6), (8, 2, 64, 32, 4), (1, 1, 128, 2, 2),
                                                (36, 4, 64, 16, 3)])
def test_convolution_folded_into_the_row_kernel(dtype, H_, G_, D_, rot, taps):
    """The convolution, the whole-row norms, the rotation and the cache rows in one launch against the two kernels in
    turn, bit for bit: two requests in portions and single tokens (the launch renews the state itself when every request
    brings one token), in swapped state rows; queries, cache rows and the states after every step."""
    n, page, eps = [13, 6], 8, 1e-5
    Dp = -(-D_ // 16) * 16
    C = (H_ + G_) * D_
    x = [rand((n[b], C + H_ + 3), 140 + b, dtype) for b in (0, 1)]
    w, ib = rand((C, taps), 142), rand((C,), 143)
    qw, kw = rand((H_ * D_,), 144) + 1.5, rand((G_ * D_,), 145) + 1.5
    inv = torch.tensor([77.0 ** (-2.0 * i / rot) for i in range(rot // 2)], device=DEV)
    width = 5 + max((taps - 1) * C, 1)
    states = [torch.zeros((2, width), device=DEV) for _ in (0, 1)]
    caches = [[torch.zeros((6, G_, page, Dp), dtype=dtype, device=DEV) for _ in (0, 1)] for _ in (0, 1)]
    base = [0, 24]                                                          # cache slots of the two requests

    def step(live, lens, starts):
        s = mini_step(lens, [1 - b for b in live], starts)
        xin = torch.cat([x[b][a:a + c] for b, a, c in zip(live, starts, lens)]).contiguous()
        slots = ints([base[b] + a + i for b, a, c in zip(live, starts, lens) for i in range(c)])
        T = xin.shape[0]
        outs = []
        for fused in (0, 1):
            q = torch.empty((T, H_ * Dp), dtype=dtype, device=DEV)
            kc, vc = caches[fused]
            if fused:
                ops().conv_rows_norm_rope_write(xin, w, ib, states[1], 5, s.cu_seqlens, s.state_slots, s.req_index, max(lens),
                                                s.positions, slots, qw, kw, eps, inv, rot, q, kc, vc, H_, G_, D_, s.err,
                                                padded_head_dim=Dp)
            else:
                qk = torch.empty((T, C), device=DEV)
                ops().short_conv(xin, 0, C, w, None, states[0], 5, s.cu_seqlens, s.state_slots, qk, act=False, longest=max(lens),
                                 in_bias=ib)
                ops().rows_norm_rope_write(qk, s.positions, slots, qw, kw, eps, inv, rot, q, kc, vc, H_, G_, D_, s.err,
                                           padded_head_dim=Dp)
            outs.append(q)
        assert int(s.err.item()) == 0
        assert torch.equal(outs[0], outs[1]) and torch.equal(states[0], states[1])
        return outs[1]

    in_portions(n, step)
    assert torch.equal(caches[0][0], caches[1][0]) and torch.equal(caches[0][1], caches[1][1])
    assert float(caches[1][0].abs().max()) > 0 and float(states[1][:, :5].abs().max()) == 0.0


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


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H_,G_,D_,page,size", [(4, 2, 16, 8, 7), (6, 6, 32, 16, 1), (8, 2, 64, 64, 70), (3, 1, 48, 4, 33),
                                                (2, 2, 128, 16, 4096), (4, 1, 64, 64, 64)])
def test_sigmoid_weights_blocks_and_head_gate(dtype, H_, G_, D_, page, size):
    """Queries of two requests (a portion of a prompt and a single token, as a mixed step brings them) over shuffled
    pages: every visible key weighs sigmoid(score + bias) alone, keys of earlier blocks weigh nothing, and every head is
    multiplied by its gate."""
    lens, new = [150, 83], [61, 1]
    scale = 0.6 * D_ ** -0.5
    seqs = [(rand((n, G_, D_), 70 + b, dtype).cpu(), rand((n, G_, D_), 72 + b, dtype).cpu()) for b, n in enumerate(lens)]
    kc, vc, table = paged(seqs, page, G_, D_, dtype, 5)
    req = [b for b, c in enumerate(new) for _ in range(c)]
    pos = [p_ for n, c in zip(lens, new) for p_ in range(n - c, n)]
    T = len(req)
    q = rand((T, H_ * D_), 74, dtype)
    pb = rand((H_,), 75) - 1.0
    gate = rand((T, H_ + 3), 76, dtype, 2.0)
    out = torch.empty((T, H_ * D_), dtype=dtype, device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().paged_attention(q, out, kc, vc, table, ints(req), ints(pos), H_, G_, D_, scale, None, e, weighting="sigmoid",
                          chunk=size, head_bias=pb, gate=gate[:, 1:])
    assert int(e.item()) == 0
    for b, (n, c) in enumerate(zip(lens, new)):
        k, v = (t.double() for t in seqs[b])
        qfull = torch.zeros(n, H_, D_, dtype=torch.float64)
        mine = [t for t in range(T) if req[t] == b]
        qfull[n - c:] = q[mine].double().cpu().view(c, H_, D_)
        want = P.sigmoid_chunk_weights(qfull, k, v, pb.cpu(), scale, size)[n - c:]
        want = want * torch.sigmoid(gate[mine, 1:1 + H_].double().cpu())[:, :, None]
        close(out[mine].view(c, H_, D_), want, dtype, "sigmoid attention", tol=2e-5 if dtype == torch.float32 else 1.5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("weighting", ["sigmoid", "softmax"])
@pytest.mark.parametrize("H_,G_,D_,page,size", [(4, 2, 16, 8, 7), (6, 6, 32, 16, 1), (8, 2, 64, 64, 70), (3, 1, 48, 4, 33),
                                                (2, 2, 128, 16, 4096), (4, 1, 64, 64, 64), (40, 2, 32, 16, 300), (9, 1, 80, 32, 129)])
def test_tensor_core_kernels_take_the_weighting_the_blocks_and_the_gate(weighting, H_, G_, D_, page, size):
    """The bfloat16 kernels of a mixed step (tiles of a prompt's portion; single tokens, their keys split over blocks that
    merge as a cluster, through scratch, or not at all) against the plain sums, and against the kernel that serves float32."""
    dtype, sig = torch.bfloat16, weighting == "sigmoid"
    lens, new = [300, 83, 1200], [170, 1, 1]
    scale = 0.6 * D_ ** -0.5
    seqs = [(rand((n, G_, D_), 70 + b, dtype).cpu(), rand((n, G_, D_), 73 + b, dtype).cpu()) for b, n in enumerate(lens)]
    kc, vc, table = paged(seqs, page, G_, D_, dtype, 5)
    req = [b for b, c in enumerate(new) for _ in range(c)]
    pos = [p_ for n, c in zip(lens, new) for p_ in range(n - c, n)]
    T = len(req)
    q = rand((T, H_ * D_), 76, dtype)
    pb = (rand((H_,), 77) - 1.0) if sig else None
    gate = rand((T, H_ + 3), 78, dtype, 2.0)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    ref = torch.empty((T, H_ * D_), dtype=dtype, device=DEV)
    ops().paged_attention(q, ref, kc, vc, table, ints(req), ints(pos), H_, G_, D_, scale, None, e, weighting=weighting,
                          chunk=size, head_bias=pb, gate=gate[:, 1:])
    tiles = torch.tensor([[0, 0, 128, 130], [0, 128, 42, 258]], dtype=torch.int32, device=DEV)
    singles = ints([170, 171])
    for chunk in (64, 256, 1024):                                           # 19 chunks through scratch, 5 as a cluster, 2
        out = torch.full((T, H_ * D_), float("nan"), dtype=dtype, device=DEV)
        ops().flash_prefill(q, out, kc, vc, table, tiles, H_, G_, D_, scale, None, e, tile_rows=128, weighting=weighting,
                            mask_chunk=size, head_bias=pb, gate=gate[:, 1:])
        S, na, nm = ops().decode_attention_scratch(2, H_, D_, 1200, chunk)
        arrivals = torch.zeros(ops().flash_decode_arrivals(2, H_, G_), dtype=torch.int32, device=DEV)
        ops().flash_decode(q, out, kc, vc, table, ints(req), ints(pos), H_, G_, D_, scale, None, 1200,
                           torch.empty(na, device=DEV), torch.empty(nm, device=DEV), e, chunk=chunk, token_index=singles,
                           arrivals=arrivals, weighting=weighting, mask_chunk=size, head_bias=pb, gate=gate[:, 1:])
        assert int(e.item()) == 0 and int(arrivals.abs().max()) == 0
        close(out, ref, dtype, f"against the float32 kernel, chunks of {chunk}", tol=1.5e-2)
        if sig:
            for b, (n, c) in enumerate(zip(lens, new)):
                k, v = (t.double() for t in seqs[b])
                qfull = torch.zeros(n, H_, D_, dtype=torch.float64)
                mine = [t for t in range(T) if req[t] == b]
                qfull[n - c:] = q[mine].double().cpu().view(c, H_, D_)
                want = P.sigmoid_chunk_weights(qfull, k, v, pb.cpu(), scale, size)[n - c:]
                want = want * torch.sigmoid(gate[mine, 1:1 + H_].double().cpu())[:, :, None]
                close(out[mine].view(c, H_, D_), want, dtype, f"sigmoid attention, chunks of {chunk}", tol=1.5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("weighting", ["sigmoid", "softmax"])
@pytest.mark.parametrize("H_,G_,D_,page,size", [(4, 2, 64, 16, 70), (2, 1, 128, 64, 64), (2, 2, 128, 16, 300), (8, 2, 64, 32, 129),
                                                (6, 3, 64, 8, 1), (2, 1, 128, 128, 4096)])
def test_tcgen05_prompt_kernel_takes_the_weighting_the_blocks_and_the_gate(weighting, H_, G_, D_, page, size):
    """The kernel of long prompt portions (tcgen05, heads of 64 and 128): a portion of 170 tokens behind 130 cached ones,
    so that its tiles begin and end inside blocks of the mask, against the float32 kernel and the plain sums."""
    dtype, sig = torch.bfloat16, weighting == "sigmoid"
    if not ops().flash_tc5_supported(dtype, D_, page):
        pytest.skip("page size not taken by this kernel")
    n, c = 300, 170
    scale = 0.6 * D_ ** -0.5
    seqs = [(rand((n, G_, D_), 170, dtype).cpu(), rand((n, G_, D_), 173, dtype).cpu())]
    kc, vc, table = paged(seqs, page, G_, D_, dtype, 5)
    q = rand((c, H_ * D_), 176, dtype)
    pb = (rand((H_,), 177) - 1.0) if sig else None
    gate = rand((c, H_ + 3), 178, dtype, 2.0)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    ref = torch.empty((c, H_ * D_), dtype=dtype, device=DEV)
    ops().paged_attention(q, ref, kc, vc, table, ints([0] * c), ints(range(n - c, n)), H_, G_, D_, scale, None, e,
                          weighting=weighting, chunk=size, head_bias=pb, gate=gate[:, 1:])
    tiles = torch.tensor([[0, 0, 128, 130], [0, 128, 42, 258]], dtype=torch.int32, device=DEV)
    out = torch.full((c, H_ * D_), float("nan"), dtype=dtype, device=DEV)
    ops().flash_prefill_tc5(q, out, kc, vc, table, tiles, H_, G_, D_, scale, None, e, weighting=weighting, mask_chunk=size,
                            head_bias=pb, gate=gate[:, 1:])
    assert int(e.item()) == 0
    close(out, ref, dtype, "against the float32 kernel", tol=1.5e-2)
    if sig:
        k, v = (t.double() for t in seqs[0])
        qfull = torch.zeros(n, H_, D_, dtype=torch.float64)
        qfull[n - c:] = q.double().cpu().view(c, H_, D_)
        want = P.sigmoid_chunk_weights(qfull, k, v, pb.cpu(), scale, size)[n - c:]
        want = want * torch.sigmoid(gate[:, 1:1 + H_].double().cpu())[:, :, None]
        close(out.view(c, H_, D_), want, dtype, "sigmoid attention on tcgen05", tol=1.5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("size,far,seen", [(1024, 3, True), (512, 512, True), (512, 511, False), (300, 599, False), (300, 600, True),
                                           (150, 600, True), (150, 599, False), (64, 576, True), (64, 575, False), (128, 512, True),
                                           (128, 511, False)])
def test_tcgen05_prompt_kernel_sees_one_far_key_inside_the_block_only(size, far, seen):
    """As `test_one_far_key_among_hundreds`, for the kernel of long prompt portions: the query at position 600 is the
    last row of a portion of 100 tokens; every weight is near zero but for the key at `far`, whose value is a marker."""
    dtype, H_, G_, D_, page, n, T = torch.bfloat16, 2, 1, 64, 16, 601, 100
    k = rand((n, G_, D_), 180, dtype, 0.1).cpu()
    v = rand((n, G_, D_), 181, dtype, 0.1).cpu()
    q = rand((1, H_ * D_), 182, dtype, 0.1)
    k[far, 0] = 0.0
    k[far, 0, 5] = 8.0
    v[far, 0] = 100.0
    q[0, 5], q[0, D_ + 5] = 4.0, 4.0
    pb = torch.full((H_,), -12.0, device=DEV)
    kc, vc, table = paged([(k, v)], page, G_, D_, dtype, 6)
    qs = torch.cat([rand((T - 1, H_ * D_), 183, dtype, 0.1), q]).contiguous()
    out = torch.empty((T, H_ * D_), dtype=dtype, device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().flash_prefill_tc5(qs, out, kc, vc, table, ints([0, 0, T, n - T]).view(1, 4), H_, G_, D_, 1.0, None, e,
                            weighting="sigmoid", mask_chunk=size, head_bias=pb)
    assert int(e.item()) == 0
    got = out[-1].float().cpu()
    if seen:
        assert float((got - 100.0).abs().max()) < 1.0, got[:4]
    else:
        assert float(got.abs().max()) < 0.1, got[:4]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("size,far,seen", [(1024, 3, True), (1024, 0, True), (512, 512, True), (512, 511, False), (300, 599, False), (300, 600, True), (150, 600, True), (150, 599, False), (64, 576, True),
                                           (64, 575, False)])
def test_one_far_key_among_hundreds(dtype, size, far, seen):
    """A query at position 600 over 601 keys whose weights are all near zero (a bias of -12) but for the key at `far`,
    which is made to stand out (weight near 1) and whose value is a marker.  The marker shows in the output exactly when
    `far` lies in the query's block: at the block's first position, not one before it; in a prompt's portion and decoded."""
    H_, G_, D_, page, n = 2, 1, 32, 16, 601
    k = rand((n, G_, D_), 80, dtype, 0.1).cpu()
    v = rand((n, G_, D_), 81, dtype, 0.1).cpu()
    q = rand((1, H_ * D_), 82, dtype, 0.1)
    k[far, 0] = 0.0
    k[far, 0, 5] = 8.0
    v[far, 0] = 100.0
    q[0, 5], q[0, D_ + 5] = 4.0, 4.0                                        # score 32 at `far`, near zero elsewhere
    pb = torch.full((H_,), -12.0, device=DEV)
    kc, vc, table = paged([(k, v)], page, G_, D_, dtype, 6)
    for portion in (1, 40):                                                 # decoded alone, and as the last row of a portion
        T = portion
        qs = torch.cat([rand((T - 1, H_ * D_), 83, dtype, 0.1), q]) if T > 1 else q
        out = torch.empty((T, H_ * D_), dtype=dtype, device=DEV)
        e = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops().paged_attention(qs.contiguous(), out, kc, vc, table, ints([0] * T), ints(range(n - T, n)), H_, G_, D_, 1.0, None, e,
                              weighting="sigmoid", chunk=size, head_bias=pb)
        outs = [out]
        if dtype == torch.bfloat16:                                         # the tensor-core kernels of bfloat16 steps
            fast = torch.empty_like(out)
            if T == 1:
                S, na, nm = ops().decode_attention_scratch(1, H_, D_, n, 128)
                ops().flash_decode(qs.contiguous(), fast, kc, vc, table, ints([0]), ints([n - 1]), H_, G_, D_, 1.0, None, n,
                                   torch.empty(na, device=DEV), torch.empty(nm, device=DEV), e, chunk=128,
                                   arrivals=torch.zeros(ops().flash_decode_arrivals(1, H_, G_), dtype=torch.int32, device=DEV),
                                   weighting="sigmoid", mask_chunk=size, head_bias=pb)
            else:
                ops().flash_prefill(qs.contiguous(), fast, kc, vc, table, ints([0, 0, T, n - T]).view(1, 4), H_, G_, D_, 1.0,
                                    None, e, weighting="sigmoid", mask_chunk=size, head_bias=pb)
            outs.append(fast)
        assert int(e.item()) == 0
        for o_ in outs:
            got = o_[-1].float().cpu()
            if seen:
                assert float((got - 100.0).abs().max()) < 1.0, (portion, got[:4])
            else:
                assert float(got.abs().max()) < 0.1, (portion, got[:4])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,g,mult,bias", [(64, 1.7, 0.7, False), (72, 1.0, 1.0, True), (320, 0.3, 0.5, True), (1000, -2.0, 1.3, False),
                                          (1002, 0.5, 0.25, True), (4096, 1.1, 0.5, True)])
def test_norm_with_one_number_adds_into_the_stream(dtype, W, g, mult, bias):
    from vllm_lite_b200.parts import spec as S
    from vllm_lite_b200.parts.base import BuildContext
    from vllm_lite_b200.parts.registry import NORMS
    eps, T = 1e-3, 9
    spec = S.NormSpec(W, eps, kind="rms_norm", tensor="", scalar=True)
    part = NORMS.get("rms_norm")(spec, {"": torch.tensor(g, dtype=dtype)}, BuildContext(torch.device(DEV), dtype))
    y = rand((T, W), 90, dtype, 0.02)                                       # small rows: eps counts inside the root
    x = rand((T, W), 91)
    vec = rand((W,), 92, scale=0.02) if bias else None                      # left to the norm's kernel by the product before
    yb = y.double().cpu() + (vec.double().cpu() if bias else 0.0)
    want = x.double().cpu() + mult * P.scalar_norm(yb, torch.tensor(g, dtype=dtype), eps)
    assert float((P.scalar_norm(y.double().cpu(), torch.tensor(g), 0.0) - P.scalar_norm(y.double().cpu(), torch.tensor(g), eps)).abs().max()) > 0.05
    cast = torch.empty((T, W), dtype=dtype, device=DEV) if dtype != torch.float32 else None
    kw = {} if mult == 1.0 else {"mult": mult}
    if bias:
        kw["bias"] = vec
    part.add_normed(y, x, mini_step([T], [0]), cast, **kw)
    close(x, want, torch.float32, "stream", tol=3e-6)
    if cast is not None:
        assert torch.equal(cast, x.to(dtype))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_is_scaled_in_float32(dtype):
    table = rand((50, 24), 95, dtype)
    ids = ints([3, 49, 0, 3])
    out = torch.empty((4, 24), device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().embed(ids, table, out, e, 17.25)
    assert int(e.item()) == 0 and torch.equal(out, table[ids.long()].float() * 17.25)


def build_part(spec, dtype, seed, registry="MIXERS", edit=None):
    """(part, its tensors as the plain implementation reads them) with seeded random weights."""
    from vllm_lite_b200.parts import registry as R
    from vllm_lite_b200.parts.base import BuildContext
    from vllm_lite_b200.weights import random_tensors
    cls = getattr(R, registry).get(spec.kind)
    tensors = random_tensors(cls.declare(spec), seed, 0.15, 0.1, dtype=dtype)
    if edit:
        edit(tensors)
    part = cls(spec, {k: v.to(DEV) for k, v in tensors.items()}, BuildContext(torch.device(DEV), dtype))
    return part, tensors


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,ff,W,T", [(6, 2, 40, 64, 37), (8, 3, 24, 64, 5), (4, 1, 17, 72, 37), (5, 5, 48, 96, 20), (3, 2, 9, 72, 1),
                                          (16, 4, 64, 128, 300)])
def test_experts_without_a_gate(dtype, E, top, ff, W, T):
    """The square of max(v, 0) between two matrices, chosen by logits WITH the router's bias (which is made large
    enough to change the choice), weighted by the softmax over the chosen logits alone."""
    from vllm_lite_b200.parts import spec as S
    spec = S.RoutedExpertsSpec(W, ff, E, top, activation="relu2", gated=False, score="softmax", renormalize=True,
                               scale_input=False, router_bias=".b")

    def edit(t):
        t["router"] = (t["router"].float() * 40).to(dtype)                  # wide gaps between the experts' logits
        t["router.b"] = (t["router.b"].float() * 60).to(dtype)

    part, tensors = build_part(spec, dtype, 8, "FEED_FORWARDS", edit)
    h = rand((T, W), 9, dtype)
    got = part(h, mini_step([T], [0]))
    f = dict(router=dict(experts=E, top=top))
    want = P.squared_relu_experts(h.double().cpu(), tensors, f)
    close(got, want, dtype, "experts", tol=2e-5 if dtype == torch.float32 else 2.5e-2)
    if top < E and T > 1:
        bare = dict(tensors)
        bare["router.b"] = torch.zeros(E)
        assert float((P.squared_relu_experts(h.double().cpu(), bare, f) - want).abs().max()) > 0.05 * float(want.abs().max())


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
    """Most of a prompt in one step, then single tokens (replayed from a graph) across several edges of the mask's blocks;
    and a request fed one token at a time from its first (the shift and the convolutions start from zeros)."""
    toks, first = tokens_for(which, 140, 11), tokens_for(which, 12, 12)
    runner = make_runner(which, dtype, num_pages=pages_for(which, 140) + 2)
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
    reqs = {k: tokens_for(which, n, 60 + i) for i, (k, n) in enumerate([("a", 90), ("b", 41), ("c", 7), ("d", 66), ("e", 30)])}
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
def test_block_edges_show_in_the_logits(which):
    """Sharp scores: a block of the mask that is one position longer or shorter moves the logits by far more than the
    tolerance in the plain implementation, and the engine agrees with the right one, in prompts and in decoding."""
    sharp = 12.0
    toks = tokens_for(which, 150, 33)
    right = plain_run(which, toks, "float32", sharp)[0]
    for off in (-1, 1):
        wrong = plain_run(which, toks, "float32", sharp, block=off)[0]
        gap = float((wrong - right).abs().max()) / float(right.abs().max())
        assert gap > 100 * TOL["float32"], f"a block off by {off} would not show ({gap:.2e})"
    runner = make_runner(which, "float32", num_pages=pages_for(which, 150) + 1, sharp=sharp)
    schedule = [([("r", toks[:60], list(range(60)))], [])] + [([("r", [toks[p]], [0])], []) for p in range(60, 150)]
    # scores twelve times as large carry twelve times the rounding of q.k into the sigmoid: three times the tolerance,
    # which the gap shown above still exceeds thirty times over
    assert_rows(H.run_schedule(runner, schedule), which, {"r": toks}, "float32", "block edges", sharp, loosen=3.0)


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["B", "C"])
def test_long_prompt_whole_against_portions(which):
    """A prompt of 2,300 tokens in one step (the products, the experts and the attention of many rows run on their
    kernels for long steps, the convolution is cut among thread blocks) against the same prompt in portions of a few hundred
    tokens and of two: bfloat16 both, so they agree to rounding; float32 bit for bit.  Keys thousands of positions back
    weigh nothing once their block is over; the blocks of B's second layer and of C are crossed many times."""
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
        if which == "B":                                       # the last positions against the plain implementation
            tail = {k: v for k, v in whole.items() if k[1] >= n - 8}
            assert_rows(tail, which, {"w": toks}, dtype, "long prompt")
        del runner


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """420 tokens one by one in a pool of a third of that: pages of finished blocks are given back and used again."""
    which, length = "A", 420
    toks = tokens_for(which, length, 31)
    runner = make_runner(which, dtype, num_pages=pages_for(which, 140))
    schedule = [([("r", toks[:4], [3])], [])] + [([("r", [toks[p]], [0])], []) for p in range(4, length)]
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, {"r": toks}, dtype, "long decode")
    held = sorted(sum(p >= 0 for p in t) for t in runner.cache.requests["r"].block_tables)
    assert held[0] <= pages_for(which, 7) + 1 and held[2] <= pages_for(which, 33) + 1


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
