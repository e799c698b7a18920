"""A plain, slow implementation of the Dufitar decoder: float64, whole sequences at once, one function per
mechanism, written from the design's equations.  It shares no code with the engine (it even reads model folders
itself) and serves as the oracle of the tests.

    x_0   = E[token] * s_embed
    x    <- x + m * N1b(mixer(N1(x)));   x <- x + m * N2b(ff(N2(x)))        every N: tanh(alpha x) * w + b
    logits = E . Nf(x)

``round_to`` emulates an engine that stores activations in a shorter type: the results of matrix products that an
engine keeps in that type, the cached rows, the queries and the attention outputs are rounded to it and widened
again; everything the design wants in 32-bit stays wide.
"""
import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64


# ---- model folders --------------------------------------------------------------------------------------------------
def load_folder(folder):
    """(config dict, {name: float64 tensor}) of a folder with config.json and model.safetensors."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        head = json.loads(f.read(n))
        data = f.read()
    w = {}
    for name, e in head.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        raw = np.frombuffer(data[a:b], dtype=np.uint8)
        if e["dtype"] == "BF16":
            t = torch.from_numpy(raw.copy()).view(torch.bfloat16).to(F64)
        elif e["dtype"] == "F32":
            t = torch.from_numpy(raw.copy()).view(torch.float32).to(F64)
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        w[name] = t.reshape(e["shape"])
    return cfg, w


def _r(t, round_to):
    return t if round_to is None else t.to(round_to).to(F64)


# ---- mechanisms ---------------------------------------------------------------------------------------------------------
def dynamic_tanh(x, alpha, weight, bias):
    return torch.tanh(alpha * x) * weight + bias


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot):
    """(frequency per pair, magnitude of cos and sin) of a ``rot`` dictionary {dims, base, scaling?}."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def pair_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, d]: the first rot['dims'] channels turn, channel 2i with 2i+1; the others pass."""
    f, mag = rotary_frequencies(rot)
    dims = rot["dims"]
    a = positions.to(F64)[:, None] * f[None, :]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T, size):
    """[T, T] mask: query i sees key j when 0 <= i - j < size (size None: every earlier key and itself)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = i >= j
    if size is not None:
        m = m & (i - j < size)
    return m


def softmax_rows(s, mask, sink=None):
    """Softmax over the visible keys of every row; with ``sink`` the denominator also holds exp(sink)."""
    s = s.masked_fill(~mask, -math.inf)
    top = s.max(dim=1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, torch.as_tensor(sink, dtype=F64))
    e = torch.exp(s - top)
    den = e.sum(dim=1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink - top)
    return e / den


def window_attention(h, w, p, m, round_to=None):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = _r(h @ w[p + "q"].T, round_to).reshape(T, H, d)
    k = _r(h @ w[p + "k"].T, round_to).reshape(T, G, d)
    v = _r(h @ w[p + "v"].T, round_to).reshape(T, G, dv)
    if m.get("rot"):
        q, k = _r(rotate(q, pos, m["rot"]), round_to), _r(rotate(k, pos, m["rot"]), round_to)
    mask = visible(T, (m.get("mask") or {}).get("size"))
    out = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        out[:, hh] = softmax_rows((q[:, hh] @ k[:, g].T) * m["scale"], mask) @ v[:, g]
    return _r(out, round_to).reshape(T, H * dv) @ w[p + "o"].T


def latent_rows(h, w, p, m, eps, round_to=None):
    """What a latent layer caches per token: (the normed latent [T, kv_rank], the rotated key part [T, rot_dim])."""
    T = h.shape[0]
    r = m["kv_rank"]
    dkv = _r(h @ w[p + "dkv"].T, round_to)
    c = dkv[:, :r]
    c = c / torch.sqrt((c * c).mean(dim=1, keepdim=True) + eps) * w[p + "dkv.norm"]
    kr = rotate(dkv[:, None, r:], torch.arange(T), m["rot"])[:, 0]
    return _r(c, round_to), _r(kr, round_to)


def latent_attention(h, w, p, m, rows, round_to=None):
    T = h.shape[0]
    H, d, rd, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = _r(h @ w[p + "q"].T, round_to).reshape(T, H, d + rd)
    q_plain, q_rot = q[..., :d], _r(rotate(q[..., d:], torch.arange(T), m["rot"]), round_to)
    c, kr = rows
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    mask = visible(T, (m.get("mask") or {}).get("size"))
    out = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        s = (q_plain[:, hh] @ k_plain[:, hh].T + q_rot[:, hh] @ kr.T) * m["scale"]
        out[:, hh] = softmax_rows(s, mask, sink=w[p + "sink"][hh]) @ v[:, hh]
    gate = torch.sigmoid(_r(h @ w[p + "g"].T, round_to))
    return _r(_r(out, round_to).reshape(T, H * dv) * gate, round_to) @ w[p + "o"].T


def dense_feed_forward(h, w, p, round_to=None):
    g, u = _r(h @ w[p + "gate"].T, round_to), _r(h @ w[p + "up"].T, round_to)
    return _r(gelu_tanh(g) * u, round_to) @ w[p + "down"].T


# ---- the model -------------------------------------------------------------------------------------------------------------
def forward(cfg, w, tokens, round_to=None, layers_out=None):
    """Logits [T, vocab] (float64) of a whole sequence; ``layers_out`` (a list) receives the stream after every layer."""
    def norm(x, name):
        return dynamic_tanh(x, w[name + ".alpha"], w[name], w[name + ".b"])

    table = w["embed"]
    x = table[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    mult, eps = cfg["residual_mult"], cfg["norm"]["eps"]
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}."
        h = _r(norm(x, L + "norm1"), round_to)
        m = layer["mixer"]
        if layer["type"] == "attention":
            a = window_attention(h, w, L + "mix.", m, round_to)
        else:
            src = m.get("kv_from")
            if src is None:
                cached[i] = latent_rows(h, w, L + "mix.", m, eps, round_to)
                src = i
            a = latent_attention(h, w, L + "mix.", m, cached[src], round_to)
        x = x + mult * norm(a, L + "norm1b")
        if layer.get("mlp") is not None:
            h = _r(norm(x, L + "norm2"), round_to)
            x = x + mult * norm(dense_feed_forward(h, w, L + "mlp.", round_to), L + "norm2b")
        if layers_out is not None:
            layers_out.append(x.clone())
    return _r(norm(x, "final.norm"), round_to) @ table.T


def generate(cfg, w, prompt, n):
    """Greedy continuation of ``prompt`` by ``n`` tokens (the whole sequence is run again for every token)."""
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(cfg, w, seq)[-1].argmax()))
    return seq[len(prompt):]
