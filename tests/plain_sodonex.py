"""A plain, slow statement of the Sodonex decoder, one function per mechanism, in float64 on the CPU.

It shares no code with the engine: every function takes plain tensors and the numbers of its own section of
config.json and works on ONE sequence from its first token.  `forward` returns the logits of every position and
the residual stream after every layer.

Notation: T tokens, W the model width, x [T, W] the residual stream, h [T, W] a sub-layer's input.  Linear weights
are [out, in].
"""
from __future__ import annotations

import torch

F = torch.float64


def lin(w, h, b=None):
    y = h @ w.to(F).t()
    return y if b is None else y + b.to(F)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(y, g, eps):
    """RMS norm whose weight is one number for all coordinates."""
    return unit_rms(y, eps) * g.to(F)


def token_shift(h, mu):
    """h_t + (h_{t-1} - h_t) * mu, element by element; the first token's neighbour is zero."""
    before = torch.cat([torch.zeros(1, h.shape[1], dtype=F), h[:-1]], 0)
    return h + (before - h) * mu.to(F)


def short_conv(u, w):
    """u [T, C]; w [C, taps]; y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), u], 0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j].to(F)
    return y


def rotate_half(x, dims, base):
    """x [T, heads, dim]; feature i < dims/2 of every head turns with feature i + dims/2 by t * base^(-2i/dims)."""
    T = x.shape[0]
    out = x.clone()
    pos = torch.arange(T, dtype=F)
    half = dims // 2
    for i in range(half):
        a = pos * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def chunk_visible(i, j, size):
    """Whether query position i reads key position j: not later, and in the same block of `size` positions."""
    return j <= i and i // size == j // size


def whole_row_norm(u, w, eps):
    """u [T, C] divided by the root mean square of the WHOLE row (all heads at once), times a weight per channel."""
    return unit_rms(u, eps) * w.to(F)


def sigmoid_chunk_weights(q, k, v, pb, scale, size):
    """q [T, H, D], k and v [T, G, D], pb [H].  Every visible key weighs sigmoid(scale q.k + pb[head]) by itself;
    nothing is divided by a sum.  Returns [T, H, D]."""
    T, H, D = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for t in range(T):
        keys = [j for j in range(t + 1) if chunk_visible(t, j, size)]
        for hd in range(H):
            g = hd // (H // G)
            s = (k[keys, g] @ q[t, hd]) * scale
            w = torch.sigmoid(s + pb[hd].to(F))
            out[t, hd] = (w[:, None] * v[keys, g]).sum(0)
    return out


def head_gate(o, h, wg):
    """o [T, H, D] times sigmoid(W_g h), one number per head."""
    return o * torch.sigmoid(lin(wg, h))[:, :, None]


def sigmoid_attention(h, p, m, eps):
    """p: the mixer's tensors (q, q.b, k, k.b, q.conv, k.conv, q.norm, k.norm, pb, g, o, o.b); m: its sizes.
    The values are the keys as they leave the convolution, before the norm and the rotation."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = short_conv(lin(p["q"], h, p["q.b"]), p["q.conv"])
    k = short_conv(lin(p["k"], h, p["k.b"]), p["k.conv"])
    v = k.view(T, G, D)
    q = rotate_half(whole_row_norm(q, p["q.norm"], eps).view(T, H, D), m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half(whole_row_norm(k, p["k.norm"], eps).view(T, G, D), m["rot"]["dims"], m["rot"]["base"])
    out = sigmoid_chunk_weights(q, k, v, p["pb"], m["scale"], m["mask"]["size"])
    out = head_gate(out, h, p["g"])
    return lin(p["o"], out.reshape(T, H * D), p["o.b"])


def squared_relu_experts(h, p, f):
    """p: `router`, `router.b`, `e<i>.up`, `e<i>.down`; f: the feed-forward's section of config.json.  The `top`
    largest router logits choose; the weights are the softmax over the chosen logits alone."""
    top = f["router"]["top"]
    z = lin(p["router"], h, p["router.b"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        val, idx = torch.sort(z[t], descending=True, stable=True)
        w = torch.softmax(val[:top], 0)
        for c in range(top):
            e = int(idx[c])
            a = torch.relu(lin(p[f"e{e}.up"], h[t])) ** 2
            out[t] = out[t] + w[c] * lin(p[f"e{e}.down"], a)
    return out


def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens):
    """(logits [T, vocab], stream after every layer [layers, T, W]) of one sequence."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = weights["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        lw = sub(weights, f"l{i}.")
        if layer["type"] != "attention":
            raise ValueError(layer["type"])
        h = token_shift(x, lw["shift"])
        x = x + mult * scalar_norm(sigmoid_attention(h, sub(lw, "mix."), layer["mixer"], eps), lw["norm1"], eps)
        if layer["mlp"] is not None:
            x = x + mult * scalar_norm(squared_relu_experts(x, sub(lw, "mlp."), layer["mlp"]), lw["norm2"], eps)
        after.append(x)
    logits = lin(weights["head"], scalar_norm(x, weights["final.norm"], eps))
    return logits, torch.stack(after)


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
