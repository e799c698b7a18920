"""A plain, slow implementation of the Tidarax decoder, one function per mechanism, in float64
(or float32) torch on the CPU.  It is the oracle of the tests and shares no code with the engine.

Notation: a sequence is a matrix ``x[n, width]`` of n tokens at positions 0..n-1; linear weights
are ``[out, in]`` and act as ``x @ W.T``.  ``cfg`` is the model's config.json as a dict, ``w`` a dict
from tensor name to tensor.
"""
import math
from typing import Dict, List, Optional

import torch


# Where an engine that computes its matrix products in bfloat16 stores activations in that type, ``forward``
# with ``round_to=torch.bfloat16`` rounds them too: the difference to the unrounded run is the drift that
# rounding alone causes, which the tests take as their yardstick.
_ROUND = None


def _r(x: torch.Tensor) -> torch.Tensor:
    return x if _ROUND is None else x.to(_ROUND).to(x.dtype)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the distance of the gain from one."""
    return unit_rms(x, eps) * (1.0 + weight)


def rotary_frequencies(rot: dict) -> List[float]:
    """One frequency per rotated pair; long wavelengths are slowed down (the Llama 3.1 rule)."""
    dims, base = rot["dims"], rot["base"]
    sc = rot.get("scaling")
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            wavelength = 2.0 * math.pi / f
            orig, lo, hi, factor = sc["original"], sc["low"], sc["high"], sc["factor"]
            if wavelength < orig / hi:
                pass
            elif wavelength > orig / lo:
                f = f / factor
            else:
                s = (orig / wavelength - lo) / (hi - lo)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x[n, heads, dim]: the first rot['dims'] channels of every head turn by position * frequency,
    channel i together with channel i + dims/2; the others pass."""
    if not rot:
        return x
    dims = rot["dims"]
    half = dims // 2
    f = torch.tensor(rotary_frequencies(rot), dtype=x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]            # [n, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def talking_sink_attention(q, k, v, talk, scale: float) -> torch.Tensor:
    """q[n, H, d], k[n, G, d], v[n, G, dv], talk[H, H].  Scores of all heads for one (query, key)
    pair are mixed by ``talk`` before the softmax; the softmax has a silent extra entry of score 0.
    Causal.  Returns [n, H, dv]."""
    n, H, d = q.shape
    G = k.shape[1]
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)                     # head h reads kv head h // rep
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale           # [H, n, n]
    s = torch.einsum("hg,gij->hij", talk, s)
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    s = s.masked_fill(~mask[None], float("-inf"))
    m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    p = e / (torch.exp(-m) + e.sum(dim=-1, keepdim=True))
    return torch.einsum("hij,jhd->ihd", p, vv)


def attention_branch(h, positions, w: Dict[str, torch.Tensor], p: str, c: dict, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = _r(h @ w[p + "q"].T).view(n, H, d)
    k = _r(h @ w[p + "k"].T).view(n, G, d)
    v = _r(h @ w[p + "v"].T).view(n, G, dv)
    q = _r(unit_rms(rotate(q, positions, c.get("rot")), eps))
    k = _r(unit_rms(rotate(k, positions, c.get("rot")), eps))
    o = _r(talking_sink_attention(q, k, v, w[p + "talk"], c["scale"]))
    return o.reshape(n, H * dv) @ w[p + "o"].T


def mingru_candidate(u: torch.Tensor) -> torch.Tensor:
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def mingru_branch(h, w: Dict[str, torch.Tensor], p: str, state: Optional[torch.Tensor] = None):
    """Returns (output [n, width_model], states after each token [n, width])."""
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    cand = mingru_candidate(h @ w[p + "x"].T + w[p + "x.b"])
    s = torch.zeros(z.shape[1], dtype=h.dtype) if state is None else state
    states = []
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        states.append(s)
    S = torch.stack(states)
    g = h @ w[p + "g"].T
    return _r(S * (g * torch.sigmoid(g))) @ w[p + "o"].T, S


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    a, b, c, e = [float(x) for x in coef]
    return a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e


def dense_ff(h, w, p: str, eps: float) -> torch.Tensor:
    return _r(polynorm(h @ w[p + "up"].T, w[p + "act"], eps)) @ w[p + "down"].T


def table_moe(h, tokens, w, p: str) -> torch.Tensor:
    table = w[p + "table"]
    top = table.shape[1]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[int(tokens[t])].tolist():
            q = f"{p}e{int(e)}."
            g = h[t] @ w[q + "gate"].T
            out[t] += _r((g * torch.sigmoid(g)) * (h[t] @ w[q + "up"].T)) @ w[q + "down"].T / top
    return out


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[list] = None,
            round_to=None):
    """Logits [n, vocab] of one whole sequence; ``layers_out`` receives the stream after every layer."""
    global _ROUND
    _ROUND = round_to
    try:
        return _forward(cfg, w, tokens, dtype, layers_out)
    finally:
        _ROUND = None


def _forward(cfg, w, tokens, dtype, layers_out):
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tokens))
    x = w["embed"][tokens]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] != "parallel":
            raise ValueError(layer["type"])
        m = layer["mixer"]
        h = _r(norm_around_zero(x, w[p + "norm1"], eps))
        left = attention_branch(h, pos, w, p + "mix.left.", m["left"], eps)
        right, _ = mingru_branch(h, w, p + "mix.right.")
        x = x + m["left_scale"] * left + m["right_scale"] * right
        if layer.get("mlp"):
            h = _r(norm_around_zero(x, w[p + "norm2"], eps))
            if layer["mlp"]["kind"] == "dense":
                x = x + dense_ff(h, w, p + "mlp.", eps)
            else:
                x = x + table_moe(h, tokens, w, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    return _r(norm_around_zero(x, w["final.norm"], eps)) @ w["head"].T


def load_folder(folder: str):
    """(config dict, weights dict) of a model folder, read with the standard library and numpy only."""
    import json
    import os
    import struct
    import numpy as np
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    kinds = {"F32": (np.float32, torch.float32), "I32": (np.int32, torch.int32), "BF16": (np.uint16, torch.bfloat16)}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        npdt, tdt = kinds[info["dtype"]]
        arr = np.frombuffer(data[a:b], dtype=npdt).copy()
        t = torch.from_numpy(arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        w[name] = t.reshape(info["shape"])
    return cfg, w


def generate(cfg: dict, w: Dict[str, torch.Tensor], prompt, steps: int) -> List[int]:
    """Greedy continuation, the whole sequence recomputed for every token."""
    seq, out = list(prompt), []
    for _ in range(steps):
        tok = int(forward(cfg, w, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
