"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers 36]
    python bench.py --size 14b --context 8192 --continuous 32      (continuous batching, a line of its own)

Prints ONE JSON line.  `value` is decoded tokens per second of K decode steps at the
given batch, timed on the device with CUDA events (weights, 16 GB, are far larger than
L2, so every step reads them from HBM).  `e2e` is the same metric through the Python
entry point (`LLMEngine.step`): host token ids in through pinned memory, sampled ids
back to the host, every step.  `prefill` is one 2,048-token prompt, `points` are decode
at batch 1 and 64 and `prefill_default`, the same prompt through `LLMEngine` with the scheduler's default
limits (tokens per second to the first token, wall clock); `roofline` relates the decode step to the bytes
it must read.
Weights are random (seeded), prompts are seeded uniform token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=40960)
# the other dense sizes of the architecture (layers, hidden, heads, intermediate); kv heads 8, head_dim 128
SIZES = {"8b": (36, 4096, 32, 12288), "14b": (40, 5120, 40, 17408), "32b": (64, 5120, 64, 25600)}
METRIC = "decode tok/s at batch 8 (Qwen3-8B, bf16)"
PREFILL_TOKENS = 2048


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return self
        def pump():
            for line in self.proc.stdout:
                self.samples.append((time.time(), line.strip()))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        return self

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        rows = [l.split(", ") for t, l in self.samples if t0 <= t <= t1] or [l.split(", ") for _, l in self.samples]
        rows = [r for r in rows if len(r) == 6 and r[0].isdigit()]
        if not rows:
            return None
        mhz = sorted(int(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].strip().lower() == "active" for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def model_bytes_and_flops(cfg, layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * hd * H + H * nq * hd + 3 * H * I          # matrix elements of one layer
    norms = layers * (2 * H + 2 * hd) + H
    weight_bytes = 2 * (layers * per_layer + V * H) + 4 * norms            # bf16 matrices, every one read once
    kv_bytes_per_token = layers * 2 * nkv * hd * 2
    T = PREFILL_TOKENS
    prefill_flops = 2 * T * layers * per_layer + layers * 4 * nq * hd * (T * (T + 1) // 2) + 2 * V * H
    return weight_bytes, kv_bytes_per_token, prefill_flops


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "pplmx/vllm-lite is a Rust workspace (no setup.py or pyproject.toml; pip reports 'not "
                      "installable') and no cargo/rustc toolchain or crate registry exists offline"}))
    return 0


def decode_run(runner, sampler, batch, context, warmup, steps, fill, vocab, tag):
    """W + K decode steps of `batch` requests that end at `context` tokens each.
    Returns (ms per step, kernel launches per step, mean context over the timed steps)."""
    import torch
    from vllm_lite_b200.csrc import ops
    from vllm_lite_b200.engine import StepEntry
    from vllm_lite_b200.sampling import SamplingParams
    start_len = context - (warmup + steps)
    ids = [f"{tag}{i}" for i in range(batch)]
    gen = torch.Generator().manual_seed(1234)
    for rid in ids:
        if fill == "prefill":                           # the cache holds what a real prompt leaves
            prompt = torch.randint(0, vocab, (start_len,), generator=gen).tolist()
            for lo in range(0, start_len, PREFILL_TOKENS):
                runner.step([StepEntry(rid, prompt[lo:lo + PREFILL_TOKENS], [])])
        else:                                           # pages are taken; their contents are random numbers
            runner.cache.admit(rid)
            runner.cache.append(rid, start_len)
    greedy = [SamplingParams()] * batch
    def one(step):
        entries = [StepEntry(rid, [(7 * i + 13 * step) % vocab], [0]) for i, rid in enumerate(ids)]
        logits = runner.step(entries)
        sampler.sample(logits, greedy, [()] * batch)
    for s in range(warmup):
        one(s)
    torch.cuda.synchronize()
    n0 = ops.launch_count
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for s in range(steps):
        one(warmup + s)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    launches = (ops.launch_count - n0) / steps
    runner.check_device_errors()
    for rid in ids:
        runner.release(rid)
    return ms, launches, start_len + warmup + (steps - 1) / 2 + 1


def prefill_run(runner, vocab, repeats=3):
    import torch
    from vllm_lite_b200.engine import StepEntry
    gen = torch.Generator().manual_seed(99)
    times = []
    for r in range(repeats + 1):
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        runner.step([StepEntry("prefill", prompt, [PREFILL_TOKENS - 1])])
        t1.record()
        torch.cuda.synchronize()
        runner.release("prefill")
        if r:                                            # the first run warms up
            times.append(t0.elapsed_time(t1))
    times.sort()
    return times[len(times) // 2]


def prefill_default_run(engine, vocab, repeats=3):
    """What a user gets for one 2,048-token prompt: through LLMEngine with the scheduler's default limits
    (4,096 tokens a step, portions of 512 beside decoding requests), host ids in, the first token out.
    Returns tokens per second (median of `repeats` after one warm-up run)."""
    import torch
    cfg = engine.scheduler.config
    saved = (cfg.max_num_batched_tokens, cfg.prefill_chunk_size)
    cfg.max_num_batched_tokens, cfg.prefill_chunk_size = 4096, 512
    gen = torch.Generator().manual_seed(77)
    times = []
    try:
        for r in range(repeats + 1):
            prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            engine.add_request(prompt, max_tokens=1)
            out = []
            while engine.has_unfinished():
                out += engine.step()
            dt = time.perf_counter() - t0
            assert len(out) == 1 and out[0].finished
            if r:
                times.append(dt)
    finally:
        cfg.max_num_batched_tokens, cfg.prefill_chunk_size = saved
    times.sort()
    return PREFILL_TOKENS / times[len(times) // 2]


def e2e_run(engine, batch, context, warmup, steps, vocab):
    """The same decode steps through LLMEngine.step: host ids in, sampled ids out, every step."""
    import torch
    gen = torch.Generator().manual_seed(4321)
    # A request decodes while the prompts of the later ones are computed (a prompt takes `fill` steps): the
    # earlier a request comes, the shorter its prompt, so that all of them end the timed steps just below
    # `context` (and none crosses the context bound its decode graph was recorded for in mid-measurement).
    fill = -(-context // PREFILL_TOKENS) + 1
    for i in range(batch):
        prompt_len = max(16, context - (warmup + steps) - (batch - 1 - i) * fill - 4)
        engine.add_request(torch.randint(0, vocab, (prompt_len,), generator=gen).tolist(),
                           max_tokens=engine.scheduler.config.max_model_len - prompt_len)
        while any(s.remaining > 1 for s in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d0, t0 = engine.runner.uploaded_bytes, time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(engine.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (engine.runner.uploaded_bytes - h2d0) / steps
    for seq in list(engine.scheduler.running):
        engine.cancel_request(seq.seq_id)
    assert produced == batch * steps, (produced, batch, steps)
    if os.environ.get("VLLM_LITE_B200_BENCH_STEP_TIMES"):
        print("step times of the end-to-end run:", json.dumps(engine.stats()["step_times"]["decode"]), file=sys.stderr)
    return produced / dt, h2d, 4 * batch


def continuous_run(engine, requests, vocab, prompt_range, out_len):
    """Continuous batching through LLMEngine: all requests arrive at once with prompts of seeded
    uniform length, each generates `out_len` tokens.  Wall clock around the whole run, host token
    ids in and out.  Returns the figures of the JSON line."""
    import random
    import torch
    rng = random.Random(0)
    gen = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, vocab, (rng.randint(*prompt_range),), generator=gen).tolist() for _ in range(requests)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for p in prompts:
        engine.add_request(p, out_len)
    kinds = {"prompt": [0, 0.0], "mixed": [0, 0.0], "decode": [0, 0.0]}
    produced = 0
    before = dict(engine.scheduler.stats)
    while engine.has_unfinished():
        s0 = time.perf_counter()
        produced += len(engine.step())
        now = dict(engine.scheduler.stats)
        pre, dec = now["prefill_tokens"] - before["prefill_tokens"], now["decode_tokens"] - before["decode_tokens"]
        kind = "mixed" if pre and dec else "prompt" if pre else "decode"
        kinds[kind][0] += 1
        kinds[kind][1] += time.perf_counter() - s0
        before = now
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    engine.runner.check_device_errors()
    prompt_tokens = sum(len(p) for p in prompts)
    return {"value": round(produced / dt, 1), "unit": "generated tokens/s", "requests": requests,
            "prompt_tokens": prompt_tokens, "generated_tokens": produced, "seconds": round(dt, 3),
            "all_tokens_per_s": round((prompt_tokens + produced) / dt, 1),
            "steps": {k: v[0] for k, v in kinds.items()},
            "ms_per_step": {k: round(v[1] / v[0] * 1e3, 3) if v[0] else None for k, v in kinds.items()},
            "preemptions": engine.scheduler.stats["preemptions"],
            # host time of LLMEngine.step() and device time of every 16th step, by kind (median, 90th percentile)
            "step_times": engine.stats()["step_times"]}


def check_fp32(cfg, layers, tokens=1024):
    """The whole model in true float32 at full depth: a prompt run whole, the same prompt cut into
    portions of changing size beside another request's tokens, and its last tokens one by one must give
    the same bits at every compared position (the float32 kernels add in an order that depends on
    positions alone).  Prints one JSON line; exit code 0 only when every row is equal."""
    import torch
    from vllm_lite_b200.engine import ModelRunner, StepEntry, random_model
    vocab = cfg["vocab_size"]
    _, plan, weights = random_model(cfg, seed=0, dtype="float32", device="cuda:0", store_dtype=torch.float32)
    runner = ModelRunner(plan, weights, dtype=torch.float32, device="cuda:0", page_size=16,
                         num_pages=3 * (tokens // 16 + 2), max_requests=4, own_weights=True)
    del weights
    gen = torch.Generator().manual_seed(7)
    toks = torch.randint(0, vocab, (tokens,), generator=gen).tolist()
    other = torch.randint(0, vocab, (64,), generator=gen).tolist()
    places = sorted({0, 1, 15, 16, 17, tokens // 3, tokens // 2} | set(range(tokens - 9, tokens)))
    t0 = time.time()
    whole = runner.step([StepEntry("w", toks, places)]).clone()
    runner.release("w")
    rows, fed, k, o = {}, 0, 0, 0
    sizes = [299, 2, 17, 128, 1, 64, 3]
    while fed < tokens - 8:
        n = min(sizes[k % len(sizes)], tokens - 8 - fed)
        k += 1
        want = [p - fed for p in places if fed <= p < fed + n]
        entries = [StepEntry("c", toks[fed:fed + n], want)]
        if o < len(other):                              # another request's tokens share the step
            m = 1 if k % 2 else 5
            entries.insert(k % 2, StepEntry("o", other[o:o + m], []))
            o += m
        out = runner.step(entries)
        for r, w in enumerate(want):
            rows[fed + w] = out[r].clone()
        fed += n
    for p in range(tokens - 8, tokens):                 # the last tokens one by one (the decode path)
        rows[p] = runner.step([StepEntry("c", [toks[p]], [0])])[0].clone()
    runner.check_device_errors()
    torch.cuda.synchronize()
    unequal = [p for i, p in enumerate(places) if not torch.equal(rows[p], whole[i])]
    worst = max(float((rows[p] - whole[i]).abs().max()) for i, p in enumerate(places))
    print(json.dumps({"check": "float32, whole prompt against portions of changing size and single tokens",
                      "model": f"{layers} layers, hidden {cfg['hidden_size']}, vocabulary {vocab}", "tokens": tokens,
                      "rows_compared": len(places), "rows_equal_bit_for_bit": len(places) - len(unequal),
                      "max_abs_difference": worst, "seconds": round(time.time() - t0, 1)}))
    return 0 if not unequal else 1


def read_ceiling(cfg, batch, context):
    """What ONE launch that must read a given number of bytes can reach, at the sizes of a decode step's
    kernels: a kernel that only reads (csrc/memprobe.cu) beside the engine's own kernel for each of them.
    Every launch reads memory that L2 does not hold (8 copies of the operands in turn), launches follow one
    another inside a CUDA graph with programmatic dependent launch on, as in a decode step.  One JSON line."""
    import torch
    from vllm_lite_b200.csrc import ops
    dev = "cuda:0"
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    M, L = batch, 8
    ops.set_pdl(True)
    err = torch.zeros(1, dtype=torch.int32, device=dev)

    def in_graph(fn):                                   # microseconds per launch, L launches a replay
        fn(); torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(10):
            g.replay()
        t1.record(); torch.cuda.synchronize()
        return t0.elapsed_time(t1) / 10 / L * 1e3

    def weights(n, k):
        return [torch.randn(n, k, device=dev, dtype=torch.bfloat16) for _ in range(L)]

    nw = torch.ones(H, device=dev)
    x = torch.randn(M, H, device=dev)
    part = torch.zeros(ops.NORM_PARTIALS, 16, device=dev)
    rows = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
    out = {}

    def product(name, n, k, **kw):
        ws = weights(n, k)
        a = torch.randn(M, k, device=dev, dtype=torch.bfloat16)
        width = n // 2 if kw.get("swiglu") else n
        c = torch.empty(M, width, device=dev, dtype=kw.pop("out_dtype", torch.bfloat16))
        sink = kw.pop("sink", False)
        gu = torch.empty(M, n, device=dev, dtype=torch.bfloat16) if M > ops.SMALL_M else None
        def ours():
            for w in ws:
                if M > ops.SMALL_M:                   # more rows than the weight-streaming product takes: the library
                    if kw.get("swiglu"):
                        torch.mm(a, w.t(), out=gu)
                    else:
                        torch.mm(a, w.t(), out=c)
                elif sink:
                    ops.gemm_bf16_small_m(a, w, rows, err, sink=(x, nw, part))
                else:
                    ops.gemm_bf16_small_m(a, w, c, err, **kw)
        nbytes = n * k * 2
        def plain():
            for w in ws:
                ops.read_only(w, nbytes)
        out[name] = {"MB": round(nbytes / 1e6, 1), "engine_us": round(in_graph(ours), 1), "read_only_us": round(in_graph(plain), 1)}
        del ws

    product("qkv", (nq + 2 * nkv) * hd, H, scaled=(part, 1, 1e-6, H))
    product("o", H, nq * hd, sink=True)
    product("gate_up", 2 * I, H, swiglu=True, scaled=(part, 1, 1e-6, H))
    product("down", H, I, sink=True)
    if M <= ops.SMALL_M:
        product("head", V, H, out_dtype=torch.float32)
    # decode attention: `batch` requests of `context` keys, pages of 16 in a row
    page, nblk = 16, context // 16 + 1
    caches = [(torch.randn(batch * nblk, nkv, page, hd, device=dev, dtype=torch.bfloat16),
               torch.randn(batch * nblk, nkv, page, hd, device=dev, dtype=torch.bfloat16)) for _ in range(L)]
    table = torch.arange(batch * nblk, device=dev, dtype=torch.int32).view(batch, nblk)
    qkv = torch.randn(batch, (nq + 2 * nkv) * hd, device=dev, dtype=torch.bfloat16)
    o = torch.empty(batch, nq * hd, device=dev, dtype=torch.bfloat16)
    req = torch.arange(batch, dtype=torch.int32, device=dev)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
    chunk = ops.decode_chunk_for(batch, nkv, context, head_dim=hd)
    S, na, nm = ops.decode_attention_scratch(batch, nq, hd, context, chunk)
    pa, pm = torch.empty(na, device=dev), torch.empty(nm, device=dev)
    arr = torch.zeros(ops.flash_decode_arrivals(batch, nq, nkv), dtype=torch.int32, device=dev)
    def attention():
        for kc, vc in caches:
            ops.flash_decode(qkv, o, kc, vc, table, req, pos, nq, nkv, hd, hd ** -0.5, 0, context, pa, pm, err,
                             chunk=chunk, arrivals=arr)
    kv_bytes = batch * context * nkv * hd * 2 * 2
    def attention_plain():
        for kc, vc in caches:
            ops.read_only(kc, kv_bytes // 2 // 16 * 16)
            ops.read_only(vc, kv_bytes // 2 // 16 * 16)
    out["attention"] = {"MB": round(kv_bytes / 1e6, 1), "engine_us": round(in_graph(attention), 1),
                        "read_only_us": round(in_graph(attention_plain), 1), "read_only_launches": 2}
    assert int(err.item()) == 0
    pk = peaks()
    for v in out.values():
        v["at_copy_peak_us"] = round(v["MB"] * 1e6 / (pk["hbm_gbs"] * 1e9) * 1e6, 1)
    print(json.dumps({"read_ceiling": out, "batch": batch, "context": context, "copy_peak_gbs": pk["hbm_gbs"],
                      "how": "microseconds a launch, 8 launches over memory L2 does not hold, in a CUDA graph, dependent launches on"}))
    return 0


# ---------------------------------------------------------------------------------------------------
# --kikepel: the Kikepel decoder (latent attention with window and sink, routed experts, post-norm blocks)
# beside the Qwen3 decoder at equal width, depth, heads and active feed-forward width
# ---------------------------------------------------------------------------------------------------
# name: (width, heads, dim, vdim, q_rank, kv_rank, window, dense ff, expert ff, experts, top, vocab)
KIKEPEL_SIZES = {"2k": (2048, 16, 128, 128, 768, 128, 1024, 8192, 1024, 32, 4, 65536),
                 "4k": (4096, 32, 128, 128, 1536, 128, 4096, 12288, 1408, 64, 6, 65536),
                 "4k-r256": (4096, 32, 128, 128, 1536, 256, 4096, 12288, 1408, 64, 6, 65536)}
# kernels of the new design and the like kernels of the closest model, by the name of their entry in csrc/ops.py
TIMED_OPS = ("paged_attention", "flash_prefill", "flash_prefill_tc5", "flash_decode", "gemm_heads", "gemm_grouped",
             "gemm_grouped_fused", "gemm_grouped_tc5", "gemm_bf16_small_m", "gemm_bf16_tc5", "gemm_bf16_tc5_pair", "layernorm_add",
             "layernorm_rows", "add_rmsnorm", "latent_norm_write", "qk_norm_rope_write", "moe_route", "moe_align",
             "moe_gather", "moe_combine", "gated_act", "silu_mul", "scale_softcap", "embed", "cast", "add_bias",
             "hc_step", "dyt_rows", "short_conv", "ssd_scan", "mlstm_scan", "delta_scan", "gate_norm", "scaled_sum",
             "token_shift", "rows_norm_rope_write", "conv_rows_norm_rope_write", "rmsnorm_add", "unary_act",
             "head_norm_write", "rope_heads", "sigmoid_gate", "token_shift_multi", "decay_scan", "decay_from_raw")


def kikepel_config(size, layers):
    W, H, D, V, QR, KR, win, ff, eff, E, top, vocab = KIKEPEL_SIZES[size]
    mix = dict(heads=H, dim=D, vdim=V, q_rank=QR, kv_rank=KR, scale=D ** -0.5, mask=dict(size=win))
    moe = dict(kind="moe", expert=dict(ff=eff, limit=7.0), router=dict(experts=E, top=top))
    kinds = [("latent_attention", dict(kind="dense", ff=ff)), ("latent_attention", moe), ("latent_attention_2", moe),
             ("latent_attention", moe)]
    return dict(architecture="Kikepel", vocab=vocab, width=W, norm=dict(eps=1e-6), logit_scale=1.0, logit_softcap=30.0,
                max_position_embeddings=16384,
                layers=[dict(type=kinds[i % 4][0], mixer=mix, mlp=kinds[i % 4][1]) for i in range(layers)])


def timed_step(runner, entries):
    """One step with every kernel of csrc/ops.py between two CUDA events.  The launches queue up behind a
    kernel that only waits, so that the events see the kernels back to back and not the host's pace.
    Returns {op: [launches, microseconds]} (library products through torch.mm are 'library_mm')."""
    import torch
    from vllm_lite_b200.csrc import ops
    from vllm_lite_b200.parts import matmul
    records, saved = [], {}
    def wrap(name, fn):
        def inner(*a, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **k)
            e1.record()
            # an attention launch whose scores are capped or biased by the distance is listed apart
            shaped = k.get("softcap") or k.get("distance") is not None
            records.append((name + "+shape" if shaped else name, e0, e1))
            return r
        return inner
    for name in TIMED_OPS:
        saved[name] = getattr(ops, name)
        setattr(ops, name, wrap(name, saved[name]))
    mm = torch.mm
    torch.mm = wrap("library_mm", mm)
    graphs, runner.decode_graphs = runner.decode_graphs, False
    try:
        torch.cuda.synchronize()
        torch.cuda._sleep(60_000_000)
        runner.step(entries)
        torch.cuda.synchronize()
    finally:
        for name, fn in saved.items():
            setattr(ops, name, fn)
        torch.mm = mm
        runner.decode_graphs = graphs
    out = {}
    for name, e0, e1 in records:
        rec = out.setdefault(name, [0, 0.0])
        rec[0] += 1
        rec[1] += e0.elapsed_time(e1) * 1e3
    # the products count twice where an outer entry (gemm_bf16_tc5 ...) is itself an op: they are leaves here
    return {k: [v[0], round(v[1], 1)] for k, v in sorted(out.items())}


def kikepel_bench(args):
    import torch
    from vllm_lite_b200.engine import LLMEngine, StepEntry, random_model
    size, layers = args.kikepel, args.layers or 8
    W, H, D, V, QR, KR, win, ff, eff, E, top, vocab = KIKEPEL_SIZES[size]
    context, pk = args.context, peaks()
    warmup = max(args.warmup, 3)
    qwen = dict(QWEN3_8B, num_hidden_layers=layers, hidden_size=W, num_attention_heads=H, num_key_value_heads=max(1, H // 4),
                head_dim=128, intermediate_size=top * eff, vocab_size=vocab, max_position_embeddings=16384)
    results = {}
    for name, cfg in (("kikepel", kikepel_config(size, layers)), ("qwen3", qwen)):
        _, plan, weights = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
        slack = 256
        pages = 64 * (-(-(context + slack) // args.block_size) + 1) + PREFILL_TOKENS // args.block_size + 64
        engine = LLMEngine(plan=plan, weights=weights, dtype="bfloat16", kv_blocks=pages, block_size=args.block_size,
                           max_batch_size=64, max_num_batched_tokens=PREFILL_TOKENS, prefill_chunk_size=PREFILL_TOKENS,
                           max_model_len=context + slack)
        del weights
        runner, sampler = engine.runner, engine.sampler
        for t in runner.storage.paged:
            t.normal_()
        res = {}
        pms = prefill_run(runner, vocab)
        res["prefill"] = {"tokens": PREFILL_TOKENS, "ms": round(pms, 3), "tokens_per_s": round(PREFILL_TOKENS / pms * 1e3, 1)}
        for b in (8, 64):
            ms, launches, _ = decode_run(runner, sampler, b, context, warmup, args.steps, "random", vocab, f"d{b}.")
            res[f"decode_b{b}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(b * 1e3 / ms, 1), "launches": round(launches)}
        gen = torch.Generator().manual_seed(5)
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        res["kernels_prefill"] = timed_step(runner, [StepEntry("kp", prompt, [PREFILL_TOKENS - 1])])
        runner.release("kp")
        ids = [f"kd{i}" for i in range(64)]
        for rid in ids:
            runner.cache.admit(rid)
            runner.cache.append(rid, context - 1)
        res["kernels_decode_b64"] = timed_step(runner, [StepEntry(rid, [i], [0]) for i, rid in enumerate(ids)])
        for rid in ids:
            runner.release(rid)
        if name == "qwen3":
            # the same step with as many keys a token as the other design's mask leaves it: attention at equal reads
            reach = (context - 1) % block + 1
            for rid in ids:
                runner.cache.admit(rid)
                runner.cache.append(rid, reach - 1)
            runner.storage.zero_slots(runner.cache.take_fresh_slots())
            res["kernels_decode_b64_equal_keys"] = timed_step(runner, [StepEntry(rid, [i], [0]) for i, rid in enumerate(ids)])
            for rid in ids:
                runner.release(rid)
        runner.check_device_errors()
        res["weights_GB"] = round(sum(p.numel() * p.element_size() for p in _tensors_of(runner.model)) / 1e9, 2)
        results[name] = res
        del engine, runner, sampler
        torch.cuda.empty_cache()
    # ---- the new kernels against their rooflines, beside the like kernels of the closest model ---------
    T, B = PREFILL_TOKENS, 64
    keys = lambda w: sum(min(p + 1, w) for p in range(T))          # keys all queries of the prompt read
    nsink = sum(1 for i in range(layers) if i % 4 != 2)
    k, q = results["kikepel"], results["qwen3"]
    def us(res, step, names):
        return sum(res[step].get(n, [0, 0.0])[1] for n in names)
    roof = {}
    att = ("paged_attention", "flash_prefill", "flash_prefill_tc5", "flash_decode")
    tf = lambda flops, micro: round(flops / (micro * 1e-6) / 1e12, 1) if micro else None
    gb = lambda nbytes, micro: round(nbytes / (micro * 1e-6) / 1e9, 1) if micro else None
    roof["attention_prefill_tflops"] = {
        "kikepel": tf(layers * 4.0 * H * KR * keys(win), us(k, "kernels_prefill", att)),
        "qwen3": tf(layers * 4.0 * H * 128 * keys(T), us(q, "kernels_prefill", att))}
    roof["attention_decode_gbs"] = {
        "kikepel": gb(layers * B * min(context, win) * KR * 2.0, us(k, "kernels_decode_b64", att)),
        "qwen3": gb(layers * B * context * 2.0 * max(1, H // 4) * 128 * 2.0, us(q, "kernels_decode_b64", att))}
    head_flops = layers * 2.0 * T * H * KR * (D + V)
    roof["per_head_products_prefill_tflops"] = {"kikepel": tf(head_flops, us(k, "kernels_prefill", ("gemm_heads",)))}
    roof["per_head_products_decode_gbs"] = {"kikepel": gb(layers * H * KR * (D + V) * 2.0, us(k, "kernels_decode_b64", ("gemm_heads",)))}
    nmoe = sum(1 for i in range(layers) if i % 4 != 0)
    q_layer = (H + 2 * max(1, H // 4)) * 128 * W + W * H * 128 + 3 * W * top * eff      # matrix elements of a Qwen3 layer
    roof["expert_products_prefill_tflops"] = {
        "kikepel": tf(nmoe * 2.0 * T * top * 3 * W * eff, us(k, "kernels_prefill", ("gemm_grouped", "gemm_grouped_fused", "gemm_grouped_tc5"))),
        "qwen3 (all dense products of the layers)": tf(layers * 2.0 * T * q_layer,
                                                       us(q, "kernels_prefill", ("gemm_bf16_tc5", "gemm_bf16_tc5_pair", "library_mm")))}
    touched = min(E, B * top)
    roof["expert_products_decode_gbs"] = {
        "kikepel (experts that 64 tokens can reach)": gb(nmoe * touched * 3.0 * W * eff * 2, us(k, "kernels_decode_b64", ("gemm_grouped", "gemm_grouped_fused"))),
        "qwen3 (all products)": gb(q["weights_GB"] * 1e9 - 2.0 * vocab * W * 2, us(q, "kernels_decode_b64", ("library_mm", "gemm_bf16_small_m")))}
    roof["norm_prefill_gbs"] = {
        "kikepel layernorm_add (y in, x in and out, cast out)": gb(k["kernels_prefill"].get("layernorm_add", [0])[0] * T * W * 12.0,
                                                                  us(k, "kernels_prefill", ("layernorm_add",))),
        "qwen3 add_rmsnorm (delta in, x in and out, h out)": gb(q["kernels_prefill"].get("add_rmsnorm", [0])[0] * T * W * 12.0,
                                                               us(q, "kernels_prefill", ("add_rmsnorm",)))}
    roof["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk["source"]}
    print(json.dumps({"kikepel_bench": size, "layers": layers, "context": context, "steps": args.steps, "warmup": warmup,
                      "dtype": "bf16", "data": "synthetic (random weights, uniform token ids)",
                      "config": {"kikepel": dict(zip(("width", "heads", "dim", "vdim", "q_rank", "kv_rank", "window", "dense_ff",
                                                      "expert_ff", "experts", "top", "vocab"), KIKEPEL_SIZES[size])),
                                 "qwen3": {k_: qwen[k_] for k_ in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                                                    "head_dim", "intermediate_size", "vocab_size")}},
                      "results": results, "roofline": roof, "sinks_in": nsink}))
    return 0


# ---------------------------------------------------------------------------------------------------
# --tuzisun: the Tuzisun decoder (several residual streams, tanh norm, window attention beside a state space,
# matrix memory, channel-wise delta rule, grouped router) beside the Qwen3 decoder at equal width, depth and heads
# ---------------------------------------------------------------------------------------------------
# name: (width, streams, attention heads, kv heads, head size, window, state-space heads, their vdim, state, taps,
#        matrix-memory heads, dim, vdim, delta heads, dim, vdim, low rank, dense ff, expert ff, experts, top, groups, kept, vocab)
TUZISUN_SIZES = {"2k": (2048, 4, 16, 4, 128, 1024, 32, 64, 128, 4, 8, 128, 256, 16, 128, 128, 64, 8192, 1024, 32, 4, 4, 2, 65536),
                 "4k": (4096, 4, 32, 8, 128, 4096, 64, 64, 128, 4, 16, 128, 256, 32, 128, 128, 128, 12288, 1408, 64, 6, 8, 4, 65536)}


def tuzisun_config(size, layers):
    (W, S, H, KV, D, win, SH, SP, N, taps, MH, MD, MP, DH, DD, DP, rank, ff, eff, E, top, groups, keep, vocab) = TUZISUN_SIZES[size]
    par = dict(left=dict(heads=H, kv_heads=KV, dim=D, vdim=D, scale=D ** -0.5, mask=dict(size=win), rot=dict(dims=D, base=500000.0)),
               right=dict(heads=SH, vdim=SP, state=N, groups=1, conv=taps, norm_groups=8), left_scale=0.7, right_scale=1.1)
    moe = dict(kind="moe", expert=dict(ff=eff), router=dict(experts=E, top=top, groups=dict(count=groups, keep=keep)))
    dense = dict(kind="dense", ff=ff, limit=7.0)
    kinds = [("channel_delta", dict(heads=DH, kv_heads=DH, dim=DD, vdim=DP, conv=taps, decay_rank=rank, gate_rank=rank), dense),
             ("parallel", par, moe), ("mlstm", dict(heads=MH, dim=MD, vdim=MP, gate_cap=15.0), dense), ("parallel", par, moe)]
    return dict(architecture="Tuzisun", vocab=vocab, width=W, streams=S, norm=dict(eps=1e-6), max_position_embeddings=16384,
                layers=[dict(type=kinds[i % 4][0], mixer=kinds[i % 4][1], mlp=kinds[i % 4][2]) for i in range(layers)])


def tuzisun_bench(args):
    import torch
    from vllm_lite_b200.engine import LLMEngine, StepEntry, random_model
    size, layers = args.tuzisun, args.layers or 8
    (W, S, H, KV, D, win, SH, SP, N, taps, MH, MD, MP, DH, DD, DP, rank, ff, eff, E, top, groups, keep, vocab) = TUZISUN_SIZES[size]
    context, pk = args.context, peaks()
    warmup = max(args.warmup, 3)
    qwen = dict(QWEN3_8B, num_hidden_layers=layers, hidden_size=W, num_attention_heads=H, num_key_value_heads=KV,
                head_dim=D, intermediate_size=ff, vocab_size=vocab, max_position_embeddings=16384)
    results = {}
    for name, cfg in (("tuzisun", tuzisun_config(size, layers)), ("qwen3", qwen)):
        _, plan, weights = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
        slack = 256
        pages = 64 * (-(-(context + slack) // args.block_size) + 1) + PREFILL_TOKENS // args.block_size + 64
        engine = LLMEngine(plan=plan, weights=weights, dtype="bfloat16", kv_blocks=pages, block_size=args.block_size,
                           max_batch_size=64, max_num_batched_tokens=PREFILL_TOKENS, prefill_chunk_size=PREFILL_TOKENS,
                           max_model_len=context + slack)
        del weights
        runner, sampler = engine.runner, engine.sampler
        for t in runner.storage.paged:
            t.normal_()
        res = {}
        pms = prefill_run(runner, vocab)
        res["prefill"] = {"tokens": PREFILL_TOKENS, "ms": round(pms, 3), "tokens_per_s": round(PREFILL_TOKENS / pms * 1e3, 1)}
        for b in (8, 64):
            ms, launches, _ = decode_run(runner, sampler, b, context, warmup, args.steps, "random", vocab, f"d{b}.")
            res[f"decode_b{b}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(b * 1e3 / ms, 1), "launches": round(launches)}
        gen = torch.Generator().manual_seed(5)
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        res["kernels_prefill"] = timed_step(runner, [StepEntry("kp", prompt, [PREFILL_TOKENS - 1])])
        runner.release("kp")
        ids = [f"kd{i}" for i in range(64)]
        for rid in ids:
            runner.cache.admit(rid)
            runner.cache.append(rid, context - 1)
        runner.storage.zero_slots(runner.cache.take_fresh_slots())
        res["kernels_decode_b64"] = timed_step(runner, [StepEntry(rid, [i], [0]) for i, rid in enumerate(ids)])
        for rid in ids:
            runner.release(rid)
        if name == "qwen3":
            # the same step with as many keys a token as the other design's mask leaves it: attention at equal reads
            reach = (context - 1) % block + 1
            for rid in ids:
                runner.cache.admit(rid)
                runner.cache.append(rid, reach - 1)
            runner.storage.zero_slots(runner.cache.take_fresh_slots())
            res["kernels_decode_b64_equal_keys"] = timed_step(runner, [StepEntry(rid, [i], [0]) for i, rid in enumerate(ids)])
            for rid in ids:
                runner.release(rid)
        runner.check_device_errors()
        res["weights_GB"] = round(sum(p.numel() * p.element_size() for p in _tensors_of(runner.model)) / 1e9, 2)
        results[name] = res
        del engine, runner, sampler
        torch.cuda.empty_cache()
    # ---- the new kernels against their rooflines, beside the like kernels of the closest model ---------
    T, B = PREFILL_TOKENS, 64
    t, q = results["tuzisun"], results["qwen3"]
    def per(res, step, name):
        n, micro = res[step].get(name, [0, 0.0])
        return n, micro
    gb = lambda nbytes, micro: round(nbytes / (micro * 1e-6) / 1e9, 1) if micro else None
    n_par = sum(1 for i in range(layers) if i % 4 in (1, 3))
    n_delta = sum(1 for i in range(layers) if i % 4 == 0)
    n_mm = sum(1 for i in range(layers) if i % 4 == 2)
    conv_ch = {"ssm": SH * SP + 2 * N, "delta": 2 * DH * DD + DH * DP}
    roof = {}
    for step, rows in (("kernels_prefill", T), ("kernels_decode_b64", B)):
        r = {}
        n, micro = per(t, step, "hc_step")
        # a pass reads and writes S float32 copies, reads y and writes h (the first pass of a step reads one copy, the last writes a sum)
        r["hc_step_gbs"] = gb(n * rows * W * (8.0 * S + 4.0), micro)
        n, micro = per(q, step, "add_rmsnorm")
        r["qwen3_add_rmsnorm_gbs"] = gb(n * rows * W * 12.0, micro)
        n, micro = per(t, step, "short_conv")
        r["short_conv_gbs"] = gb(rows * 6.0 * (n_par * conv_ch["ssm"] + n_delta * conv_ch["delta"]), micro)
        n, micro = per(t, step, "gate_norm")
        r["gate_norm_gbs"] = gb(rows * 8.0 * (n_par * SH * SP + n_delta * DH * DP + n_mm * MH * MP), micro)
        for op, heads, rows_, cols, count in (("ssd_scan", SH, N, SP, n_par), ("mlstm_scan", MH, MD, MP, n_mm), ("delta_scan", DH, DD, DP, n_delta)):
            n, micro = per(t, step, op)
            flops = {"ssd_scan": 4.0, "mlstm_scan": 4.0, "delta_scan": 7.0}[op] * heads * rows_ * cols * rows * count
            state = 8.0 * heads * rows_ * cols * count * (B if step.endswith("b64") else 1)
            r[op] = {"us_a_layer": round(micro / max(n, 1), 1), "gflops": round(flops / (micro * 1e-6) / 1e9, 1) if micro else None,
                     "state_gbs": gb(state, micro)}
        roof[step] = r
    roof["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk["source"]}
    print(json.dumps({"tuzisun_bench": size, "layers": layers, "context": context, "steps": args.steps, "warmup": warmup,
                      "dtype": "bf16", "data": "synthetic (random weights, uniform token ids)",
                      "config": {"tuzisun": dict(zip(("width", "streams", "heads", "kv_heads", "dim", "window", "ssm_heads", "ssm_vdim",
                                                      "state", "taps", "mm_heads", "mm_dim", "mm_vdim", "delta_heads", "delta_dim",
                                                      "delta_vdim", "low_rank", "dense_ff", "expert_ff", "experts", "top", "groups",
                                                      "kept", "vocab"), TUZISUN_SIZES[size])),
                                 "qwen3": {k_: qwen[k_] for k_ in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                                                    "head_dim", "intermediate_size", "vocab_size")}},
                      "results": results, "roofline": roof}))
    return 0


# ---------------------------------------------------------------------------------------------------
# --sodonex: the Sodonex decoder (token shift, attention behind short convolutions with the keys as values, sigmoid
# weights in blocks of positions, a gate per head; experts without a gate; post-norm blocks with a factor) beside the
# Qwen3 decoder at equal width, depth, heads and active feed-forward width
# ---------------------------------------------------------------------------------------------------
# name: (width, heads, kv heads, head size, taps, positions per block of the mask, rotated features, expert ff, experts, top, vocab)
SODONEX_SIZES = {"2k": (2048, 16, 4, 128, 4, 1024, 64, 1024, 32, 4, 65536),
                 "4k": (4096, 32, 8, 128, 4, 2048, 64, 1408, 64, 6, 65536),
                 "4k-h64": (4096, 64, 8, 64, 3, 512, 32, 2048, 32, 4, 65536)}


def sodonex_config(size, layers):
    W, H, KV, D, taps, block, rot, eff, E, top, vocab = SODONEX_SIZES[size]
    mix = dict(heads=H, kv_heads=KV, dim=D, vdim=D, conv=taps, scale=D ** -0.5, mask=dict(size=block), rot=dict(dims=rot, base=500000.0))
    moe = dict(kind="moe", expert=dict(ff=eff), router=dict(experts=E, top=top))
    return dict(architecture="Sodonex", vocab=vocab, width=W, norm=dict(eps=1e-6), embedding=dict(scale=W ** 0.5), residual_mult=0.5,
                max_position_embeddings=16384, layers=[dict(type="attention", mixer=mix, mlp=moe) for _ in range(layers)])


def sodonex_bench(args):
    import torch
    from vllm_lite_b200.engine import LLMEngine, StepEntry, random_model
    size, layers = args.sodonex, args.layers or 8
    W, H, KV, D, taps, block, rot, eff, E, top, vocab = SODONEX_SIZES[size]
    context, pk = args.context, peaks()
    warmup = max(args.warmup, 3)
    qwen = dict(QWEN3_8B, num_hidden_layers=layers, hidden_size=W, num_attention_heads=H, num_key_value_heads=KV,
                head_dim=D, intermediate_size=top * eff, vocab_size=vocab, max_position_embeddings=16384)
    results = {}
    for name, cfg in (("sodonex", sodonex_config(size, layers)), ("qwen3", qwen)):
        _, plan, weights = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
        slack = 256
        pages = 64 * (-(-(context + slack) // args.block_size) + 1) + PREFILL_TOKENS // args.block_size + 64
        engine = LLMEngine(plan=plan, weights=weights, dtype="bfloat16", kv_blocks=pages, block_size=args.block_size,
                           max_batch_size=64, max_num_batched_tokens=PREFILL_TOKENS, prefill_chunk_size=PREFILL_TOKENS,
                           max_model_len=context + slack)
        del weights
        runner, sampler = engine.runner, engine.sampler
        for t in runner.storage.paged:
            t.normal_()
        res = {}
        pms = prefill_run(runner, vocab)
        res["prefill"] = {"tokens": PREFILL_TOKENS, "ms": round(pms, 3), "tokens_per_s": round(PREFILL_TOKENS / pms * 1e3, 1)}
        for b in (8, 64):
            ms, launches, _ = decode_run(runner, sampler, b, context, warmup, args.steps, "random", vocab, f"d{b}.")
            res[f"decode_b{b}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(b * 1e3 / ms, 1), "launches": round(launches)}
        gen = torch.Generator().manual_seed(5)
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        res["kernels_prefill"] = timed_step(runner, [StepEntry("kp", prompt, [PREFILL_TOKENS - 1])])
        runner.release("kp")
        ids = [f"kd{i}" for i in range(64)]
        for rid in ids:
            runner.cache.admit(rid)
            runner.cache.append(rid, context - 1)
        runner.storage.zero_slots(runner.cache.take_fresh_slots())
        res["kernels_decode_b64"] = timed_step(runner, [StepEntry(rid, [i], [0]) for i, rid in enumerate(ids)])
        for rid in ids:
            runner.release(rid)
        if name == "qwen3":
            # the same step with as many keys a token as the other design's mask leaves it: attention at equal reads
            reach = (context - 1) % block + 1
            for rid in ids:
                runner.cache.admit(rid)
                runner.cache.append(rid, reach - 1)
            runner.storage.zero_slots(runner.cache.take_fresh_slots())
            res["kernels_decode_b64_equal_keys"] = timed_step(runner, [StepEntry(rid, [i], [0]) for i, rid in enumerate(ids)])
            for rid in ids:
                runner.release(rid)
        runner.check_device_errors()
        res["weights_GB"] = round(sum(p.numel() * p.element_size() for p in _tensors_of(runner.model)) / 1e9, 2)
        results[name] = res
        del engine, runner, sampler
        torch.cuda.empty_cache()
    # ---- the new kernels against their rooflines, beside the like kernels of the closest model ---------
    T, B = PREFILL_TOKENS, 64
    sx, q = results["sodonex"], results["qwen3"]
    def us(res, step, names):
        return sum(res[step].get(n, [0, 0.0])[1] for n in names)
    def count(res, step, name):
        return res[step].get(name, [0, 0.0])[0]
    tf = lambda flops, micro: round(flops / (micro * 1e-6) / 1e12, 1) if micro else None
    gb = lambda nbytes, micro: round(nbytes / (micro * 1e-6) / 1e9, 1) if micro else None
    att = ("paged_attention", "flash_prefill", "flash_prefill_tc5", "flash_decode")
    keys_block = sum(p % block + 1 for p in range(T))              # keys all queries of the prompt read: their block up to themselves
    keys_all = T * (T + 1) // 2
    reach = (context - 1) % block + 1                              # keys a decoded token at the last position reads
    roof = {}
    roof["attention_prefill_tflops"] = {
        "sodonex": tf(layers * 4.0 * H * D * keys_block, us(sx, "kernels_prefill", att)),
        "qwen3": tf(layers * 4.0 * H * D * keys_all, us(q, "kernels_prefill", att)),
        "us_a_layer": {"sodonex": round(us(sx, "kernels_prefill", att) / layers, 1), "qwen3": round(us(q, "kernels_prefill", att) / layers, 1)}}
    roof["attention_decode_gbs"] = {
        "sodonex": gb(layers * B * reach * 2.0 * KV * D * 2.0, us(sx, "kernels_decode_b64", att)),
        "qwen3": gb(layers * B * context * 2.0 * KV * D * 2.0, us(q, "kernels_decode_b64", att)),
        "qwen3_at_equal_keys": gb(layers * B * reach * 2.0 * KV * D * 2.0, us(q, "kernels_decode_b64_equal_keys", att)),
        "keys_a_token": {"sodonex": reach, "qwen3": context, "qwen3_at_equal_keys": reach},
        "us_a_layer": {"sodonex": round(us(sx, "kernels_decode_b64", att) / layers, 1), "qwen3": round(us(q, "kernels_decode_b64", att) / layers, 1),
                       "qwen3_at_equal_keys": round(us(q, "kernels_decode_b64_equal_keys", att) / layers, 1)}}
    C = (H + KV) * D
    for step, rows in (("kernels_prefill", T), ("kernels_decode_b64", B)):
        r = {}
        # token shift: the float32 stream in, the activation out
        r["token_shift_gbs"] = gb(count(sx, step, "token_shift") * rows * W * 6.0, us(sx, step, ("token_shift",)))
        # convolution: the projection's q and k columns in (bfloat16), float32 out
        r["short_conv_gbs"] = gb(count(sx, step, "short_conv") * rows * C * 6.0, us(sx, step, ("short_conv",)))
        # whole-row norm, rotation, cache write: float32 q and k in; q, k and v out in bfloat16
        r["rows_norm_rope_write_gbs"] = gb(count(sx, step, "rows_norm_rope_write") * rows * (C * 4.0 + (H + 2 * KV) * D * 2.0),
                                           us(sx, step, ("rows_norm_rope_write",)))
        # the two in one launch: the product's q and k columns in (bfloat16); q, k and v out in bfloat16
        r["conv_rows_norm_rope_write_gbs"] = gb(count(sx, step, "conv_rows_norm_rope_write") * rows * (C * 2.0 + (H + 2 * KV) * D * 2.0),
                                                us(sx, step, ("conv_rows_norm_rope_write",)))
        r["qwen3_qk_norm_rope_write_gbs"] = gb(count(q, step, "qk_norm_rope_write") * rows * (H + 2 * KV) * D * 4.0,
                                               us(q, step, ("qk_norm_rope_write",)))
        # norm of a sublayer's output added into the stream: y in, x in and out, cast out
        r["rmsnorm_add_gbs"] = gb(count(sx, step, "rmsnorm_add") * rows * W * 12.0, us(sx, step, ("rmsnorm_add",)))
        r["qwen3_add_rmsnorm_gbs"] = gb(count(q, step, "add_rmsnorm") * rows * W * 12.0, us(q, step, ("add_rmsnorm",)))
        roof[step] = r
    grouped = ("gemm_grouped", "gemm_grouped_fused", "gemm_grouped_tc5")
    q_layer = (H + 2 * KV) * D * W + W * H * D + 3 * W * top * eff          # matrix elements of a Qwen3 layer
    roof["expert_products_prefill_tflops"] = {
        "sodonex": tf(layers * 2.0 * T * top * 2 * W * eff, us(sx, "kernels_prefill", grouped)),
        "qwen3 (all dense products of the layers)": tf(layers * 2.0 * T * q_layer,
                                                       us(q, "kernels_prefill", ("gemm_bf16_tc5", "gemm_bf16_tc5_pair", "library_mm")))}
    touched = min(E, B * top)
    roof["expert_products_decode_gbs"] = {
        "sodonex (experts that 64 tokens can reach)": gb(layers * touched * 2.0 * W * eff * 2, us(sx, "kernels_decode_b64", grouped)),
        "qwen3 (all products)": gb(q["weights_GB"] * 1e9 - 2.0 * vocab * W * 2, us(q, "kernels_decode_b64", ("library_mm", "gemm_bf16_small_m")))}
    roof["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk["source"]}
    print(json.dumps({"sodonex_bench": size, "layers": layers, "context": context, "steps": args.steps, "warmup": warmup,
                      "dtype": "bf16", "data": "synthetic (random weights, uniform token ids)",
                      "config": {"sodonex": dict(zip(("width", "heads", "kv_heads", "dim", "taps", "mask_block", "rotated", "expert_ff",
                                                      "experts", "top", "vocab"), SODONEX_SIZES[size])),
                                 "qwen3": {k_: qwen[k_] for k_ in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                                                    "head_dim", "intermediate_size", "vocab_size")}},
                      "results": results, "roofline": roof}))
    return 0


# ---------------------------------------------------------------------------------------------------
# --puturax: the Puturax decoder (norms before and after every sub-layer; latent attention with a rotated part; attention
# with capped, distance-biased scores beside a time mixing; grouped experts with a shared one) beside the Qwen3 decoder
# at equal width, depth, heads and active feed-forward width
# ---------------------------------------------------------------------------------------------------
# name: (width, heads, kv heads, head size, latent query rank, latent rank, rotated part, time-mixing heads, their size, decay rank,
#        dense ff, expert ff, experts, top, groups, kept, shared ff, vocab)
PUTURAX_SIZES = {"2k": (2048, 16, 4, 128, 768, 64, 64, 32, 64, 64, 8192, 1024, 32, 4, 4, 2, 1024, 65536),
                 "4k": (4096, 32, 8, 128, 1536, 64, 64, 64, 64, 128, 12288, 1408, 64, 6, 8, 4, 1408, 65536),
                 "4k-h64": (4096, 64, 8, 64, 1024, 96, 32, 32, 128, 64, 8192, 2048, 32, 4, 4, 3, 2048, 65536)}


def puturax_config(size, layers):
    W, H, KV, D, QR, KR, R, TH, TD, rank, ff, eff, E, top, groups, keep, sff, vocab = PUTURAX_SIZES[size]
    lat = dict(heads=H, dim=D, rot_dim=R, vdim=D, q_rank=QR, kv_rank=KR, scale=(D + R) ** -0.5, rot=dict(dims=R, base=500000.0))
    par = dict(left=dict(heads=H, kv_heads=KV, dim=D, vdim=D, scale=0.2, softcap=30.0,
                         q_temp=dict(coef=0.1, every=1024)),
               right=dict(heads=TH, dim=TD, decay_rank=rank), left_scale=0.7, right_scale=0.6)
    moe = dict(kind="moe", expert=dict(ff=eff), router=dict(experts=E, top=top, groups=dict(count=groups, keep=keep)), shared=dict(ff=sff))
    kinds = [("latent_attention", lat, dict(kind="dense", ff=ff)), ("parallel", par, moe), ("parallel", par, moe), ("parallel", par, moe)]
    return dict(architecture="Puturax", vocab=vocab, width=W, norm=dict(eps=1e-6), embedding=dict(scale=W ** 0.5),
                max_position_embeddings=16384,
                layers=[dict(type=kinds[i % 4][0], mixer=kinds[i % 4][1], mlp=kinds[i % 4][2]) for i in range(layers)])


def puturax_bench(args):
    import torch
    from vllm_lite_b200.engine import LLMEngine, StepEntry, random_model
    size, layers = args.puturax, args.layers or 8
    W, H, KV, D, QR, KR, R, TH, TD, rank, ff, eff, E, top, groups, keep, sff, vocab = PUTURAX_SIZES[size]
    context, pk = args.context, peaks()
    warmup = max(args.warmup, 3)
    qwen = dict(QWEN3_8B, num_hidden_layers=layers, hidden_size=W, num_attention_heads=H, num_key_value_heads=KV,
                head_dim=D, intermediate_size=top * eff + sff, vocab_size=vocab, max_position_embeddings=16384)
    results = {}
    for name, cfg in (("puturax", puturax_config(size, layers)), ("qwen3", qwen)):
        _, plan, weights = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
        slack = 256
        pages = 64 * (-(-(context + slack) // args.block_size) + 1) + PREFILL_TOKENS // args.block_size + 64
        engine = LLMEngine(plan=plan, weights=weights, dtype="bfloat16", kv_blocks=pages, block_size=args.block_size,
                           max_batch_size=64, max_num_batched_tokens=PREFILL_TOKENS, prefill_chunk_size=PREFILL_TOKENS,
                           max_model_len=context + slack)
        del weights
        runner, sampler = engine.runner, engine.sampler
        for t in runner.storage.paged:
            t.normal_()
        res = {}
        pms = prefill_run(runner, vocab)
        res["prefill"] = {"tokens": PREFILL_TOKENS, "ms": round(pms, 3), "tokens_per_s": round(PREFILL_TOKENS / pms * 1e3, 1)}
        for b in (8, 64):
            ms, launches, _ = decode_run(runner, sampler, b, context, warmup, args.steps, "random", vocab, f"d{b}.")
            res[f"decode_b{b}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(b * 1e3 / ms, 1), "launches": round(launches)}
        gen = torch.Generator().manual_seed(5)
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        res["kernels_prefill"] = timed_step(runner, [StepEntry("kp", prompt, [PREFILL_TOKENS - 1])])
        runner.release("kp")
        ids = [f"kd{i}" for i in range(64)]
        for rid in ids:
            runner.cache.admit(rid)
            runner.cache.append(rid, context - 1)
        runner.storage.zero_slots(runner.cache.take_fresh_slots())
        res["kernels_decode_b64"] = timed_step(runner, [StepEntry(rid, [i], [0]) for i, rid in enumerate(ids)])
        for rid in ids:
            runner.release(rid)
        runner.check_device_errors()
        res["weights_GB"] = round(sum(p.numel() * p.element_size() for p in _tensors_of(runner.model)) / 1e9, 2)
        results[name] = res
        del engine, runner, sampler
        torch.cuda.empty_cache()
    # ---- the new kernels against their rooflines, beside the like kernels of the closest model ---------
    T, B = PREFILL_TOKENS, 64
    px, q = results["puturax"], results["qwen3"]
    def us(res, step, names):
        return sum(res[step].get(n, [0, 0.0])[1] for n in names)
    def count(res, step, name):
        return res[step].get(name, [0, 0.0])[0]
    tf = lambda flops, micro: round(flops / (micro * 1e-6) / 1e12, 1) if micro else None
    gb = lambda nbytes, micro: round(nbytes / (micro * 1e-6) / 1e9, 1) if micro else None
    n_lat = sum(1 for i in range(layers) if i % 4 == 0)
    n_par = layers - n_lat
    att = ("paged_attention", "flash_prefill", "flash_prefill_tc5", "flash_decode")
    shaped = tuple(a + "+shape" for a in att)
    keys_all = T * (T + 1) // 2
    row = -(-(KR + R) // 16) * 16
    roof = {}
    roof["attention_prefill_tflops"] = {
        "puturax capped, distance bias, sink": tf(n_par * 4.0 * H * D * keys_all, us(px, "kernels_prefill", shaped)),
        "puturax latent row": tf(n_lat * 4.0 * H * row * keys_all, us(px, "kernels_prefill", att)),
        "qwen3": tf(layers * 4.0 * H * D * keys_all, us(q, "kernels_prefill", att)),
        "us_a_layer": {"puturax shaped": round(us(px, "kernels_prefill", shaped) / max(n_par, 1), 1),
                       "puturax latent": round(us(px, "kernels_prefill", att) / max(n_lat, 1), 1),
                       "qwen3": round(us(q, "kernels_prefill", att) / layers, 1)}}
    roof["attention_decode_gbs"] = {
        "puturax capped, distance bias, sink": gb(n_par * B * context * 2.0 * KV * D * 2.0, us(px, "kernels_decode_b64", shaped)),
        "puturax latent row": gb(n_lat * B * context * row * 2.0, us(px, "kernels_decode_b64", att)),
        "qwen3": gb(layers * B * context * 2.0 * KV * D * 2.0, us(q, "kernels_decode_b64", att)),
        "us_a_layer": {"puturax shaped": round(us(px, "kernels_decode_b64", shaped) / max(n_par, 1), 1),
                       "puturax latent": round(us(px, "kernels_decode_b64", att) / max(n_lat, 1), 1),
                       "qwen3": round(us(q, "kernels_decode_b64", att) / layers, 1)}}
    for step, rows in (("kernels_prefill", T), ("kernels_decode_b64", B)):
        r = {}
        # five mixes: the activation in, five rows out
        r["token_shift_multi_gbs"] = gb(count(px, step, "token_shift_multi") * rows * W * 12.0, us(px, step, ("token_shift_multi",)))
        # head work: q, k, v in; q, k, v out (bfloat16)
        r["head_norm_write_gbs"] = gb(count(px, step, "head_norm_write") * rows * (H + 2 * KV) * D * 4.0, us(px, step, ("head_norm_write",)))
        r["qwen3_qk_norm_rope_write_gbs"] = gb(count(q, step, "qk_norm_rope_write") * rows * (H + 2 * KV) * D * 4.0,
                                               us(q, step, ("qk_norm_rope_write",)))
        # the norm after a sub-layer: y in, x in and out; the norm before: x in, h out
        r["rmsnorm_add_gbs"] = gb(count(px, step, "rmsnorm_add") * rows * W * 10.0, us(px, step, ("rmsnorm_add",)))
        r["add_rmsnorm_gbs"] = gb(count(px, step, "add_rmsnorm") * rows * W * 6.0, us(px, step, ("add_rmsnorm",)))
        r["qwen3_add_rmsnorm_gbs"] = gb(count(q, step, "add_rmsnorm") * rows * W * 12.0, us(q, step, ("add_rmsnorm",)))
        # the output gate: heads in and out, gate in; the memory's norm and gate: float32 in, gate in, out
        r["sigmoid_gate_gbs"] = gb(rows * 6.0 * (n_par + n_lat) * H * D, us(px, step, ("sigmoid_gate",)))
        r["gate_norm_gbs"] = gb(count(px, step, "gate_norm") * rows * TH * TD * 8.0, us(px, step, ("gate_norm",)))
        n, micro = count(px, step, "decay_scan"), us(px, step, ("decay_scan",))
        state = 8.0 * TH * TD * TD * n * (B if step.endswith("b64") else 1)
        r["decay_scan"] = {"us_a_layer": round(micro / max(n, 1), 1), "us_a_token_and_layer": round(micro / max(n, 1) / (rows if step == "kernels_prefill" else 1), 3),
                           "gflops": round(6.0 * TH * TD * TD * rows * n / (micro * 1e-6) / 1e9, 1) if micro else None,
                           "state_gbs": gb(state, micro)}
        roof[step] = r
    grouped = ("gemm_grouped", "gemm_grouped_fused", "gemm_grouped_tc5")
    q_layer = (H + 2 * KV) * D * W + W * H * D + 3 * W * (top * eff + sff)          # matrix elements of a Qwen3 layer
    roof["expert_products_prefill_tflops"] = {
        "puturax": tf(n_par * 2.0 * T * top * 3 * W * eff, us(px, "kernels_prefill", grouped)),
        "qwen3 (all dense products of the layers)": tf(layers * 2.0 * T * q_layer,
                                                       us(q, "kernels_prefill", ("gemm_bf16_tc5", "gemm_bf16_tc5_pair", "library_mm")))}
    touched = min(E, B * top)
    roof["expert_products_decode_gbs"] = {
        "puturax (experts that 64 tokens can reach)": gb(n_par * touched * 3.0 * W * eff * 2, us(px, "kernels_decode_b64", grouped)),
        "qwen3 (all products)": gb(q["weights_GB"] * 1e9 - 2.0 * vocab * W * 2, us(q, "kernels_decode_b64", ("library_mm", "gemm_bf16_small_m")))}
    roof["peaks"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk["source"]}
    print(json.dumps({"puturax_bench": size, "layers": layers, "context": context, "steps": args.steps, "warmup": warmup,
                      "dtype": "bf16", "data": "synthetic (random weights, uniform token ids)",
                      "config": {"puturax": dict(zip(("width", "heads", "kv_heads", "dim", "q_rank", "kv_rank", "rot_dim", "mix_heads",
                                                      "mix_dim", "decay_rank", "dense_ff", "expert_ff", "experts", "top", "groups", "kept",
                                                      "shared_ff", "vocab"), PUTURAX_SIZES[size])),
                                 "qwen3": {k_: qwen[k_] for k_ in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                                                    "head_dim", "intermediate_size", "vocab_size")}},
                      "results": results, "roofline": roof}))
    return 0


def _tensors_of(model):
    """Every device tensor that the parts of a model hold (weights as they are resident)."""
    import torch
    seen, out, stack = set(), [], [model]
    while stack:
        obj = stack.pop()
        if id(obj) in seen:
            continue
        seen.add(id(obj))
        if isinstance(obj, torch.Tensor):
            out.append(obj)
        elif isinstance(obj, (list, tuple)):
            stack.extend(obj)
        elif hasattr(obj, "__dict__") and type(obj).__module__.startswith("vllm_lite_b200"):
            stack.extend(v for k_, v in vars(obj).items() if k_ not in ("plan", "ctx", "spec"))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--size", default="8b", choices=sorted(SIZES), help="layer sizes of Qwen3-8B (default), 14B or 32B")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the size has (both numbers are reported)")
    ap.add_argument("--block-size", type=int, default=64, help="positions per page of the cache")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--only-prefill", action="store_true", help="time the 2,048-token prefill alone (for profiling)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the run through the Python entry point (for profiling)")
    ap.add_argument("--kv-fill", default="prefill", choices=["prefill", "random"],
                    help="what the cache holds before decoding: what real prompts leave, or random numbers (for profiling)")
    ap.add_argument("--continuous", type=int, default=0, metavar="REQUESTS",
                    help="instead of the decode steps: continuous batching of this many requests through LLMEngine, prompts "
                         "uniform in [256, context/2], 512 generated tokens each (steps and warmup are not used)")
    ap.add_argument("--kv-blocks", default=None, metavar="N|auto",
                    help="pages of the cache: a count, or 'auto' = sized from the memory left after the weights (the "
                         "default for --size 32b); default otherwise: what the largest batch needs at --context")
    ap.add_argument("--read-ceiling", action="store_true",
                    help="instead of timing steps: every kernel of a decode step alone beside a kernel that only reads as many bytes")
    ap.add_argument("--tuzisun", default=None, choices=sorted(TUZISUN_SIZES), metavar="SIZE",
                    help="instead of the default workload: the Tuzisun decoder at layer sizes " + ", ".join(sorted(TUZISUN_SIZES))
                         + " beside the Qwen3 decoder at equal width, depth and heads: prefill of 2,048 tokens, decode at batch 8 "
                           "and 64, and every kernel of a step between CUDA events (--layers, default 8; --context, --steps)")
    ap.add_argument("--sodonex", default=None, choices=sorted(SODONEX_SIZES), metavar="SIZE",
                    help="instead of the default workload: the Sodonex decoder at layer sizes " + ", ".join(sorted(SODONEX_SIZES))
                         + " beside the Qwen3 decoder at equal width, depth, heads and active feed-forward width")
    ap.add_argument("--puturax", default=None, choices=sorted(PUTURAX_SIZES), metavar="SIZE",
                    help="instead of the default workload: the Puturax decoder at layer sizes " + ", ".join(sorted(PUTURAX_SIZES))
                         + " beside the Qwen3 decoder at equal width, depth, heads and active feed-forward width")
    ap.add_argument("--kikepel", default=None, choices=sorted(KIKEPEL_SIZES), metavar="SIZE",
                    help="instead of the default workload: the Kikepel decoder at layer sizes " + ", ".join(sorted(KIKEPEL_SIZES))
                         + " beside the Qwen3 decoder at equal width, depth and heads: prefill of 2,048 tokens, decode at batch 8 "
                           "and 64, and every kernel of a step between CUDA events (--layers, default 8; --context, --steps)")
    ap.add_argument("--check-fp32", action="store_true",
                    help="instead of timing: the model in true float32, whole prompt against cut prompt, bit for bit")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    warmup = max(args.warmup, 3)

    if args.kikepel:
        return kikepel_bench(args)
    if args.tuzisun:
        return tuzisun_bench(args)
    if args.sodonex:
        return sodonex_bench(args)
    if args.puturax:
        return puturax_bench(args)
    import torch
    from vllm_lite_b200.csrc import ops
    from vllm_lite_b200.engine import LLMEngine, random_model
    full_layers, hidden, heads, inter = SIZES[args.size]
    if args.layers is None:
        args.layers = full_layers
    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers, hidden_size=hidden, num_attention_heads=heads,
               intermediate_size=inter)
    vocab = cfg["vocab_size"]
    if args.check_fp32:
        return check_fp32(cfg, args.layers)
    if args.read_ceiling:
        return read_ceiling(cfg, args.batch, args.context)
    _, plan, weights = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    if args.continuous:
        R, out_len, prompt_range = args.continuous, 512, (256, args.context // 2)
        pages = R * (-(-(prompt_range[1] + out_len) // args.block_size) + 1) + 64
        engine = LLMEngine(plan=plan, weights=weights, dtype="bfloat16", kv_blocks=pages, block_size=args.block_size, max_batch_size=R,
                           max_num_batched_tokens=4096, prefill_chunk_size=512, max_model_len=args.context)
        del weights
        continuous_run(engine, min(R, 4), vocab, (256, 512), 16)          # warm-up: builds, graphs of the small buckets
        clocks = ClockSampler().start()
        w0 = time.time()
        out = continuous_run(engine, R, vocab, prompt_range, out_len)
        clocks.stop()
        out = {"metric": f"continuous batching, generated tok/s (Qwen3-{args.size.upper()}, bf16)", **out, "n_gpus": 1,
               "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform token ids)",
               "config": {"model": f"Qwen3-{args.size.upper()} layer sizes", "layers": args.layers, "layers_full": full_layers,
                          "context": args.context, "prompt_lengths": f"uniform in [{prompt_range[0]}, {prompt_range[1]}]",
                          "generated_each": out_len, "block_size": args.block_size, "max_num_batched_tokens": 4096,
                          "prefill_chunk_size": 512, "timing": "wall clock around the whole run, host ids in and out"},
               "clocks": clocks.summary(w0, time.time())}
        print(json.dumps(out))
        return 0
    big = args.batch if args.no_points else max(args.batch, 64)
    # In the end-to-end run the requests' prompts are computed one after the other while the earlier requests
    # already decode: every request needs room for the tokens it generates meanwhile.
    slack = 64 + args.batch * (args.context // PREFILL_TOKENS + 2)
    pages = big * (-(-(args.context + slack) // args.block_size) + 1) + PREFILL_TOKENS // args.block_size + 64
    if args.kv_blocks == "auto" or (args.kv_blocks is None and args.size == "32b"):
        pages = None                                      # the engine sizes the cache from what the weights leave
    elif args.kv_blocks is not None:
        pages = int(args.kv_blocks)
    engine = LLMEngine(plan=plan, weights=weights, dtype="bfloat16", kv_blocks=pages, block_size=args.block_size, max_batch_size=big,
                       max_num_batched_tokens=PREFILL_TOKENS, prefill_chunk_size=PREFILL_TOKENS,
                       max_model_len=args.context + slack)
    del weights
    runner, sampler = engine.runner, engine.sampler
    for t in runner.storage.paged:                        # pages that no prompt wrote hold random numbers
        t.normal_()
    weight_bytes, kv_per_token, prefill_flops = model_bytes_and_flops(cfg, args.layers)
    pk = peaks()

    if args.only_prefill:
        pms = prefill_run(runner, vocab, repeats=max(1, min(args.steps, 5)))
        print(json.dumps({"prefill": {"value": round(PREFILL_TOKENS / pms * 1000.0, 1), "tokens": PREFILL_TOKENS,
                                      "ms": round(pms, 3), "layers": args.layers,
                                      "frac": round(prefill_flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0
    clocks = ClockSampler().start()
    w0 = time.time()
    ms, launches, mean_ctx = decode_run(runner, sampler, args.batch, args.context, warmup, args.steps, args.kv_fill, vocab, "d")
    w1 = time.time()
    e2e_tps, h2d, d2h = (0.0, 0, 0) if args.no_e2e else e2e_run(engine, args.batch, args.context, warmup, args.steps, vocab)
    clocks.stop()
    value = args.batch * 1000.0 / ms
    step_bytes = weight_bytes + args.batch * mean_ctx * kv_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": METRIC.replace("8B", args.size.upper()).replace("batch 8", f"batch {args.batch}"), "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform token ids)",
        "config": {"model": f"Qwen3-{args.size.upper()} layer sizes", "layers": args.layers, "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": vocab,
                   "global_batch": args.batch, "seq_len": args.context, "block_size": args.block_size, "parallelism": "single GPU",
                   "kv_fill": "real prefill" if args.kv_fill == "prefill" else "random numbers", "l2": f"inputs (weights {weight_bytes / 1e9:.0f} GB) larger than L2, no flush",
                   "peaks": pk["source"], "kv_pages": sum(p.size for p in runner.cache.pools)},
        "clocks": clocks.summary(w0, w1),
        "e2e": None if args.no_e2e else {"value": round(e2e_tps, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                                         "d2h_bytes_per_step": d2h},
        "gpu_launches": int(round(launches * args.steps)),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if not args.no_points:
        pms = prefill_run(runner, vocab)
        # frac: of the burst peak of the library product (one launch timed alone); the step itself is a
        # long run of products under the power cap, for which the sustained figure is the fair one
        out["prefill"] = {"value": round(PREFILL_TOKENS / pms * 1000.0, 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                          "frac": round(prefill_flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                          "frac_of_sustained": round(prefill_flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}
        ms1, _, _ = decode_run(runner, sampler, 1, args.context, warmup, args.steps, "prefill", vocab, "s")
        ms64, _, _ = decode_run(runner, sampler, 64, args.context, warmup, args.steps, args.kv_fill, vocab, "l")
        out["points"] = {"decode_b1": round(1000.0 / ms1, 1), "decode_b64": round(64 * 1000.0 / ms64, 1),
                         "prefill_default": round(prefill_default_run(engine, vocab), 1)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
