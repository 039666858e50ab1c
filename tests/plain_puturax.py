"""A plain, slow statement of the Puturax decoder, one function per mechanism, in float64 on the CPU.

It shares no code with the engine: every function takes plain tensors and the numbers of its own section of
config.json and works on ONE sequence from its first token.  `forward` returns the logits of every position and
the residual stream after every layer.

Notation: T tokens, W the model width, x [T, W] the residual stream, h [T, W] a sub-layer's input.  Linear weights
are [out, in].
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def lin(w, h):
    return h @ w.to(F).t()


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight lies around zero: the factor is 1 + w."""
    return unit_rms(x, eps) * (1.0 + w.to(F))


def plain_norm(x, w, eps):
    return unit_rms(x, eps) * w.to(F)


def rotate_half(x, dims, base, positions=None):
    """x [T, ..., n]; feature i < dims/2 turns with feature i + dims/2 by position * base^(-2i/dims); features from
    `dims` on pass unchanged."""
    T = x.shape[0]
    pos = torch.arange(T, dtype=F) if positions is None else positions.to(F)
    out = x.clone()
    half = dims // 2
    shape = (T,) + (1,) * (x.dim() - 2)
    for i in range(half):
        a = pos * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a).reshape(shape), torch.sin(a).reshape(shape)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def sigmoid_gate(heads_out, h, wg):
    """The concatenated heads times sigmoid(W_g h), element by element."""
    return heads_out * torch.sigmoid(lin(wg, h))


def latent_attention(h, w, m, eps):
    """w: the mixer's tensors by their short names; m: the mixer's section of config.json."""
    T = h.shape[0]
    H, D, R, V, K = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = plain_norm(lin(w["dq"], h), w["dq.norm"], eps)
    q = lin(w["uq"], cq).reshape(T, H, D + R)
    low = lin(w["dkv"], h)
    c = plain_norm(low[:, :K], w["dkv.norm"], eps)
    k_rot = rotate_half(low[:, K:], m["rot"]["dims"], m["rot"]["base"])            # [T, R], one for all heads
    q_rot = rotate_half(q[:, :, D:], m["rot"]["dims"], m["rot"]["base"])
    k = lin(w["uk"], c).reshape(T, H, D)
    v = lin(w["uv"], c).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        for a in range(H):
            s = (k[:t + 1, a] @ q[t, a, :D] + k_rot[:t + 1] @ q_rot[t, a]) * m["scale"]
            p = torch.softmax(s, 0)
            out[t, a] = p @ v[:t + 1, a]
    return lin(w["o"], sigmoid_gate(out.reshape(T, H * V), h, w["g"]))


def query_temperature(T, coef, every):
    """The factor on the query at position p: 1 + coef ln(floor((p + 1) / every) + 1)."""
    return torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in range(T)], dtype=F)


def capped(s, cap):
    return cap * torch.tanh(s / cap)


def distance_bias(r1, r2, dist):
    """What is taken off a score whose key lies `dist` positions back."""
    return r1 * torch.log(1.0 + r2 * dist)


def softmax_plus_one(s):
    """exp(s_j) / (1 + sum exp(s)): the denominator holds one more term, e^0, that brings no value row."""
    mx = torch.clamp(s.max(), min=0.0)
    e = torch.exp(s - mx)
    return e / (torch.exp(-mx) + e.sum())


def biased_attention(h, w, m, eps):
    """The left side of a parallel mixer.  w: tensors q, k, v, r1, r2, g, o; m: its section of config.json."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms(lin(w["q"], h).reshape(T, H, D), eps)
    k = unit_rms(lin(w["k"], h).reshape(T, G, D), eps)
    v = unit_rms(lin(w["v"], h).reshape(T, G, V), eps)
    q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    r1, r2 = w["r1"].to(F), w["r2"].to(F)
    out = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        dist = torch.arange(t, -1, -1, dtype=F)                  # key j lies t - j back
        for a in range(H):
            g = a // (H // G)
            s = capped((k[:t + 1, g] @ q[t, a]) * m["scale"], m["softcap"]) - distance_bias(r1[a], r2[a], dist)
            out[t, a] = softmax_plus_one(s) @ v[:t + 1, g]
    return lin(w["o"], sigmoid_gate(out.reshape(T, H * V), h, w["g"]))


def shifted(h):
    """Row t holds h_(t-1); zeros for the first token."""
    return torch.cat([torch.zeros(1, h.shape[1], dtype=F), h[:-1]], 0)


def channel_decay(mix_w, w1, w2, w0):
    """exp(-exp(W_2 tanh(W_1 mix) + w0)), a number in (0, 1) per head and key channel."""
    return torch.exp(-torch.exp(lin(w2, torch.tanh(lin(w1, mix_w))) + w0.to(F)))


def decayed_memory(r, k, v, decay, u):
    """One head.  r, k, decay [T, D]; v [T, P]; u [D].  o_t = (S + diag(u) k_t v_t^T)^T r_t, then
    S <- diag(decay_t) S + k_t v_t^T, S starting at zero."""
    T, D = k.shape
    S = torch.zeros(D, v.shape[1], dtype=F)
    out = torch.zeros(T, v.shape[1], dtype=F)
    for t in range(T):
        kv = torch.outer(k[t], v[t])
        out[t] = (S + u[:, None] * kv).t() @ r[t]
        S = decay[t][:, None] * S + kv
    return out


def time_mixing(h, w, m, eps):
    """The right side of a parallel mixer.  w: tensors mu.r/k/v/g/w, r, k, v, g, w1, w2, w0, u, norm, o."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    before = shifted(h)
    mix = {s: h + (before - h) * w["mu." + s].to(F) for s in "rkvgw"}
    r = lin(w["r"], mix["r"]).reshape(T, H, D)
    k = lin(w["k"], mix["k"]).reshape(T, H, D)
    v = lin(w["v"], mix["v"]).reshape(T, H, D)
    gate = torch.nn.functional.silu(lin(w["g"], mix["g"]))
    decay = channel_decay(mix["w"], w["w1"], w["w2"], w["w0"]).reshape(T, H, D)
    u = w["u"].to(F).reshape(H, D)
    o = torch.stack([decayed_memory(r[:, a], k[:, a], v[:, a], decay[:, a], u[a]) for a in range(H)], 1)
    o = unit_rms(o, eps).reshape(T, H * D) * w["norm"].to(F) * gate
    return lin(w["o"], o)


def parallel_mixer(h, w, m, eps):
    sub = lambda side: {k[len(side) + 1:]: t for k, t in w.items() if k.startswith(side + ".")}
    return (m["left_scale"] * biased_attention(h, sub("left"), m["left"], eps)
            + m["right_scale"] * time_mixing(h, sub("right"), m["right"], eps))


def dense_ff(h, w):
    return lin(w["down"], torch.relu(lin(w["up"], h)) ** 2)


def gated_expert(h, gate, up, down):
    return lin(down, torch.nn.functional.silu(lin(gate, h)) * lin(up, h))


def route(h, router, correction, top, groups, keep):
    """Per token: the chosen experts and their weights.  Choice by sigmoid score + correction among the experts of
    the `keep` groups whose two best choice scores add up highest; weights from the scores without the correction."""
    s = torch.sigmoid(lin(router, h))
    choice = s + correction.to(F)
    T, E = s.shape
    per = E // groups
    ids, weights = [], []
    for t in range(T):
        gs = [choice[t, g * per:(g + 1) * per].topk(min(2, per)).values.sum() for g in range(groups)]
        kept = sorted(range(groups), key=lambda g: (-float(gs[g]), g))[:keep]
        masked = torch.full((E,), -math.inf, dtype=F)
        for g in kept:
            masked[g * per:(g + 1) * per] = choice[t, g * per:(g + 1) * per]
        pick = sorted(range(E), key=lambda e: (-float(masked[e]), e))[:top]
        sc = s[t, pick]
        ids.append(pick)
        weights.append(sc / (sc.sum() + 1e-20))
    return ids, weights


def expert_mixture(h, w, mlp):
    ro = mlp["router"]
    ids, weights = route(h, w["router"], w["correction"], ro["top"], ro["groups"]["count"], ro["groups"]["keep"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(ids[t], weights[t]):
            out[t] += p * gated_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    return out + gated_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])


MIXERS = {"latent_attention": latent_attention, "parallel": parallel_mixer}


def forward(config, weights, tokens):
    """logits [T, vocab] and the stream after every layer [layers, T, W]."""
    eps = config["norm"]["eps"]
    w = {k: v.to(F) for k, v in weights.items()}
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    streams = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        lw = {k[len(p):]: v for k, v in w.items() if k.startswith(p)}
        mw = {k[4:]: v for k, v in lw.items() if k.startswith("mix.")}
        y = MIXERS[layer["type"]](offset_norm(x, lw["norm1"], eps), mw, layer["mixer"], eps)
        x = x + offset_norm(y, lw["norm1b"], eps)
        if layer.get("mlp") is not None:
            fw = {k[4:]: v for k, v in lw.items() if k.startswith("mlp.")}
            h = offset_norm(x, lw["norm2"], eps)
            y = dense_ff(h, fw) if layer["mlp"]["kind"] == "dense" else expert_mixture(h, fw, layer["mlp"])
            x = x + offset_norm(y, lw["norm2b"], eps)
        streams.append(x)
    logits = lin(w["embed"], offset_norm(x, w["final.norm"], eps))
    return logits, torch.stack(streams)


def read_model_dir(folder):
    """(config.json as a dict, {name: tensor}) of a model folder; a reader of its own: 8 bytes of length, a JSON
    header name -> (dtype, shape, data_offsets), then the data."""
    import json
    import struct
    from pathlib import Path
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16}
    weights = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=kinds[info["dtype"]])
        weights[name] = t.reshape(info["shape"]).clone()
    return config, weights
