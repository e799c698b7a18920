"""Typed configuration of the Dufitar decoder, read from the keys of its own config.json, and its
arrangement of parts.

A Dufitar model lists its layers one by one (``layers``), each with its own sizes.  A layer norms a
sublayer's input *and* its output and adds the normed output times ``residual_mult``:

    x <- x + m * norm1b(mixer(norm1(x)));   x <- x + m * norm2b(ff(norm2(x)))       (the second half is optional)

Every norm is a Dynamic Tanh, ``tanh(alpha * x) * w + b``.  The mixer is grouped-query attention within a sliding
window, with rotary positions over the first channels of a head (pairs of neighbours, frequencies slowed by the
YaRN rule, cos and sin scaled by ``0.1 ln(factor) + 1``), or attention over a cached latent with a learned sink per
head and a sigmoid gate on the heads' outputs; a latent layer may read the rows an earlier latent layer cached
(``kv_from``).  The feed-forward is ``W_down(gelu_tanh(W_gate h) * (W_up h))``.  The embedding rows are scaled, the
head is the embedding table, the residual stream is float32 whatever the engine's dtype is.

Every size and every constant that config.json gives is read here and handed to the parts through their specs;
nothing is fixed in code but the tensor names, the arrangement and the constants of the YaRN magnitude.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError
from .plan import (AttentionSpec, BlockOp, BlockSpec, DynamicTanhSpec, FeedForwardSpec, LatentAttentionSpec, LayerRun,
                   ModelPlan, RopeSpec, YarnScaling)

ARCHITECTURE = "Dufitar"
# the engine's own bound on a sequence: this design has no position table and names no limit
MAX_POSITIONS = 1 << 20


def _get(raw, key: str, where: str):
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks '{where}{key}'")
    return raw[key]


def _int(raw, key: str, where: str, least: int = 1) -> int:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ConfigError(f"config key '{where}{key}' must be an integer >= {least}, got {v!r}")
    return v


def _num(raw, key: str, where: str, positive: bool = False) -> float:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"config key '{where}{key}' must be a{' positive' if positive else ''} number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class DufitarRot:
    dims: int
    base: float
    scaling: Optional[YarnScaling]


@dataclass(frozen=True)
class DufitarMixer:
    kind: str                 # "attention" or "latent_attention"
    heads: int
    dim: int                  # query/key channels of a head (latent attention: the channels that are not rotated)
    vdim: int
    scale: float
    window: Optional[int]
    rot: Optional[DufitarRot]
    kv_heads: int = 0         # attention
    kv_rank: int = 0          # latent attention
    rot_dim: int = 0          # latent attention
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class DufitarLayer:
    mixer: DufitarMixer
    ff: Optional[int]         # width of the dense feed-forward; None: the layer has none


def _rot(raw, where: str, most: int) -> DufitarRot:
    dims = _int(raw, "dims", where, least=2)
    if dims % 2 or dims > most:
        raise ConfigError(f"'{where}dims' {dims} must be even and at most {most}")
    scaling = None
    if raw.get("scaling") is not None:
        s, ws = raw["scaling"], where + "scaling."
        scaling = YarnScaling(factor=_num(s, "factor", ws, True), original=_num(s, "original", ws, True),
                              fast=_num(s, "fast", ws, True), slow=_num(s, "slow", ws, True))
    return DufitarRot(dims, _num(raw, "base", where, True), scaling)


def _window(mixer, where: str) -> Optional[int]:
    mask = mixer.get("mask")
    if mask is None:
        return None
    return _int(mask, "size", where + "mask.")


@dataclass(frozen=True)
class DufitarConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    residual_mult: float
    layers: Tuple[DufitarLayer, ...]

    ARCHITECTURE = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "DufitarConfig":
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        eps = _num(_get(raw, "norm", ""), "eps", "norm.", positive=True)
        embed_scale = _num(_get(raw, "embedding", ""), "scale", "embedding.")
        mult = _num(raw, "residual_mult", "")
        layers = _get(raw, "layers", "")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config key 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            w = f"layers[{i}]."
            kind = _get(layer, "type", w)
            m, wm = _get(layer, "mixer", w), w + "mixer."
            heads, dim, vdim = _int(m, "heads", wm), _int(m, "dim", wm), _int(m, "vdim", wm)
            scale, window = _num(m, "scale", wm), _window(m, wm)
            if kind == "attention":
                kv = _int(m, "kv_heads", wm)
                if heads % kv:
                    raise ConfigError(f"'{wm}heads' {heads} is not a multiple of '{wm}kv_heads' {kv}")
                rot = _rot(m["rot"], wm + "rot.", dim) if m.get("rot") is not None else None
                mixer = DufitarMixer("attention", heads, dim, vdim, scale, window, rot, kv_heads=kv)
            elif kind == "latent_attention":
                rot_dim = _int(m, "rot_dim", wm, least=2)
                rot = _rot(_get(m, "rot", wm), wm + "rot.", rot_dim)
                kv_from = None
                if m.get("kv_from") is not None:
                    kv_from = _int(m, "kv_from", wm, least=0)
                mixer = DufitarMixer("latent_attention", heads, dim, vdim, scale, window, rot,
                                     kv_rank=_int(m, "kv_rank", wm), rot_dim=rot_dim, kv_from=kv_from)
            else:
                raise ConfigError(f"config key '{w}type' is '{kind}'; known: attention, latent_attention")
            ff = None
            if layer.get("mlp") is not None:
                mlp, wf = layer["mlp"], w + "mlp."
                mk = _get(mlp, "kind", wf)
                if mk != "dense":
                    raise ConfigError(f"config key '{wf}kind' is '{mk}'; known: dense")
                ff = _int(mlp, "ff", wf)
            out.append(DufitarLayer(mixer, ff))
        for i, layer in enumerate(out):
            j = layer.mixer.kv_from
            if j is None:
                continue
            wm = f"layers[{i}].mixer."
            if not (0 <= j < i) or out[j].mixer.kind != "latent_attention" or out[j].mixer.kv_from is not None:
                raise ConfigError(f"'{wm}kv_from' {j} must name an earlier latent_attention layer with a latent projection "
                                  f"of its own")
            a, b = layer.mixer, out[j].mixer
            if (a.kv_rank, a.rot_dim, a.rot) != (b.kv_rank, b.rot_dim, b.rot):
                raise ConfigError(f"layer {i} reads the cached rows of layer {j}: their kv_rank, rot_dim and rot must be equal")
        return cls(vocab=vocab, width=width, eps=eps, embed_scale=embed_scale, residual_mult=mult, layers=tuple(out))

    # ---- the arrangement of parts ---------------------------------------------------------
    def plan(self) -> ModelPlan:
        def norm():
            return DynamicTanhSpec(kind="dynamic_tanh", dim=self.width, weight_name="", bias_name=".b", alpha_name=".alpha")

        def rope(rot: DufitarRot, head_dim: int) -> RopeSpec:
            # the YaRN magnitude: cos and sin grow with the logarithm of the stretch
            magnitude = 0.1 * math.log(rot.scaling.factor) + 1.0 if rot.scaling is not None else 1.0
            return RopeSpec(kind="rope", head_dim=head_dim, rotary_dim=rot.dims, theta=rot.base, max_positions=MAX_POSITIONS,
                            layout="interleaved", scaling=rot.scaling, tables=False, magnitude=magnitude)

        # rows cached by a latent layer are kept as long as the widest window among its readers asks
        keep = {}
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.kind == "latent_attention":
                owner = i if m.kv_from is None else m.kv_from
                keep.setdefault(owner, []).append(m.window)
        blocks, runs = [], []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.kind == "attention":
                mixer = AttentionSpec(kind="talking_attention", hidden=self.width, num_heads=m.heads, num_kv_heads=m.kv_heads,
                                      head_dim=m.dim, v_head_dim=m.vdim, scale=m.scale, qk_norm=False,
                                      rope=rope(m.rot, m.dim) if m.rot is not None else None, window=m.window,
                                      talking_heads=False, sink=False, names=("q", "k", "v", "o", "talk"))
            else:
                owner = i if m.kv_from is None else m.kv_from
                windows = keep[owner]
                mixer = LatentAttentionSpec(kind="latent_attention", hidden=self.width, num_heads=m.heads, head_dim=m.dim,
                                            rope_dim=m.rot_dim, v_head_dim=m.vdim, kv_rank=m.kv_rank, scale=m.scale,
                                            rope=rope(m.rot, m.rot_dim), window=m.window,
                                            cache_window=None if any(w is None for w in windows) else max(windows),
                                            norm_eps=self.eps, sink=True, gate=True, shares_cache=m.kv_from is not None)
            prog = [BlockOp("norm", "x", "h", norm(), "norm1"),
                    BlockOp("mixer", "h", "a", mixer, "mix."),
                    BlockOp("norm", "a", "a", norm(), "norm1b"),
                    BlockOp("add", "a", "x", scale=self.residual_mult)]
            if layer.ff is not None:
                ff = FeedForwardSpec(kind="swiglu", hidden=self.width, intermediate=layer.ff, activation="gelu_tanh",
                                     names=("gate", "up", "down"))
                prog += [BlockOp("norm", "x", "h", norm(), "norm2"),
                         BlockOp("feed_forward", "h", "f", ff, "mlp."),
                         BlockOp("norm", "f", "f", norm(), "norm2b"),
                         BlockOp("add", "f", "x", scale=self.residual_mult)]
            blocks.append(BlockSpec(f"l{i}.", tuple(prog)))
            runs.append(LayerRun(block=i, cache_from=m.kv_from))
        plan = ModelPlan(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden=self.width, embed_name="embed",
            blocks=tuple(blocks), runs=tuple(runs), final_norm=norm(), final_norm_name="final.norm", head_name=None,
            max_positions=MAX_POSITIONS, embed_scale=self.embed_scale, residual_dtype="float32")
        plan.validate()
        return plan
