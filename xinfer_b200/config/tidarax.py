"""Typed configuration of the Tidarax decoder, read from the keys of its own config.json, and its
arrangement of parts.

A Tidarax model lists its layers one by one (``layers``), each with its own sizes.  A layer is a
pre-norm block whose mixer runs two mixers side by side on the same normed input - grouped-query
attention with rotary positions, unit-norm queries and keys, scores mixed across heads and a
softmax with a silent extra entry; and a gated recurrence whose gates read only the current token
- and adds their scaled outputs; its feed-forward is a dense layer with a polynomial activation,
a mixture of small gated experts chosen by a table over token ids, or absent.  Norm weights are
stored around zero.  The residual stream is float32 whatever the engine's dtype is.

Every size and every constant that config.json gives is read here and handed to the parts through
their specs; nothing is fixed in code but the tensor names and the arrangement.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError
from .plan import (AttentionSpec, BlockOp, BlockSpec, ExpertTableSpec, FeedForwardSpec, GatedRecurrenceSpec, LayerRun,
                   ModelPlan, NormSpec, ParallelMixerSpec, RopeScaling, RopeSpec)

ARCHITECTURE = "Tidarax"
# the engine's own bound on a sequence: this design has no position table and names no limit
MAX_POSITIONS = 1 << 20


def _get(raw: Mapping[str, Any], key: str, where: str):
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
class TidaraxRot:
    dims: int
    base: float
    scaling: Optional[RopeScaling]


@dataclass(frozen=True)
class TidaraxLeft:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[TidaraxRot]


@dataclass(frozen=True)
class TidaraxFeedForward:
    kind: str            # "dense" or "moe"
    ff: int
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class TidaraxLayer:
    left: TidaraxLeft
    left_scale: float
    right_width: int
    right_scale: float
    mlp: Optional[TidaraxFeedForward]


@dataclass(frozen=True)
class TidaraxConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[TidaraxLayer, ...]

    ARCHITECTURE = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TidaraxConfig":
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        eps = _num(_get(raw, "norm", ""), "eps", "norm.", positive=True)
        layers = _get(raw, "layers", "")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config key 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            w = f"layers[{i}]."
            kind = _get(layer, "type", w)
            if kind != "parallel":
                raise ConfigError(f"config key '{w}type' is '{kind}'; this architecture has 'parallel' layers")
            mixer = _get(layer, "mixer", w)
            left = _get(mixer, "left", w + "mixer.")
            wl = w + "mixer.left."
            heads, kv = _int(left, "heads", wl), _int(left, "kv_heads", wl)
            if heads % kv:
                raise ConfigError(f"'{wl}heads' {heads} is not a multiple of '{wl}kv_heads' {kv}")
            dim = _int(left, "dim", wl)
            rot = None
            if left.get("rot") is not None:
                r = left["rot"]
                dims = _int(r, "dims", wl + "rot.", least=2)
                if dims % 2 or dims > dim:
                    raise ConfigError(f"'{wl}rot.dims' {dims} must be even and at most the head size {dim}")
                scaling = None
                if r.get("scaling") is not None:
                    s, ws = r["scaling"], wl + "rot.scaling."
                    scaling = RopeScaling(factor=_num(s, "factor", ws, True), low=_num(s, "low", ws, True),
                                          high=_num(s, "high", ws, True), original=_num(s, "original", ws, True))
                    if scaling.high == scaling.low:
                        raise ConfigError(f"'{ws}high' and '{ws}low' must differ")
                rot = TidaraxRot(dims, _num(r, "base", wl + "rot.", True), scaling)
            right = _get(mixer, "right", w + "mixer.")
            mlp = None
            if layer.get("mlp") is not None:
                m, wm = layer["mlp"], w + "mlp."
                mk = _get(m, "kind", wm)
                if mk == "dense":
                    mlp = TidaraxFeedForward("dense", _int(m, "ff", wm))
                elif mk == "moe":
                    router = _get(m, "router", wm)
                    experts, top = _int(router, "experts", wm + "router."), _int(router, "top", wm + "router.")
                    if top > experts:
                        raise ConfigError(f"'{wm}router.top' {top} exceeds '{wm}router.experts' {experts}")
                    mlp = TidaraxFeedForward("moe", _int(_get(m, "expert", wm), "ff", wm + "expert."), experts, top)
                else:
                    raise ConfigError(f"config key '{wm}kind' is '{mk}'; known: dense, moe")
            out.append(TidaraxLayer(
                left=TidaraxLeft(heads, kv, dim, _int(left, "vdim", wl), _num(left, "scale", wl), rot),
                left_scale=_num(mixer, "left_scale", w + "mixer."),
                right_width=_int(right, "width", w + "mixer.right."),
                right_scale=_num(mixer, "right_scale", w + "mixer."), mlp=mlp))
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(out))

    # ---- the arrangement of parts ---------------------------------------------------------
    def plan(self) -> ModelPlan:
        def norm():
            return NormSpec(kind="rmsnorm", dim=self.width, eps=self.eps, weight_offset=1.0, weight_name="",
                            init="around_zero")
        blocks = []
        for i, layer in enumerate(self.layers):
            lf = layer.left
            rope = None
            if lf.rot is not None:
                rope = RopeSpec(kind="rope", head_dim=lf.dim, rotary_dim=lf.rot.dims, theta=lf.rot.base,
                                max_positions=MAX_POSITIONS, layout="neox", scaling=lf.rot.scaling, tables=False)
            left = AttentionSpec(kind="talking_attention", hidden=self.width, num_heads=lf.heads, num_kv_heads=lf.kv_heads,
                                 head_dim=lf.dim, v_head_dim=lf.vdim, scale=lf.scale, qk_norm=True, qk_norm_eps=self.eps,
                                 qk_norm_weight=False, qk_norm_after_rope=True, rope=rope, talking_heads=True, sink=True,
                                 names=("q", "k", "v", "o", "talk"))
            right = GatedRecurrenceSpec(kind="min_gru", hidden=self.width, width=layer.right_width)
            mixer = ParallelMixerSpec(kind="parallel", hidden=self.width, left=left, right=right,
                                      left_scale=layer.left_scale, right_scale=layer.right_scale)
            prog = [BlockOp("norm", "x", "h", norm(), "norm1"),
                    BlockOp("mixer", "h", "a", mixer, "mix."),
                    BlockOp("add", "a", "x")]
            if layer.mlp is not None:
                if layer.mlp.kind == "dense":
                    ff = FeedForwardSpec(kind="polynorm_mlp", hidden=self.width, intermediate=layer.mlp.ff,
                                         activation="polynorm", eps=self.eps)
                else:
                    ff = ExpertTableSpec(kind="table_experts", hidden=self.width, intermediate=layer.mlp.ff,
                                         experts=layer.mlp.experts, top=layer.mlp.top, vocab=self.vocab)
                prog += [BlockOp("norm", "x", "h", norm(), "norm2"),
                         BlockOp("feed_forward", "h", "f", ff, "mlp."),
                         BlockOp("add", "f", "x")]
            blocks.append(BlockSpec(f"l{i}.", tuple(prog)))
        plan = ModelPlan(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden=self.width, embed_name="embed",
            blocks=tuple(blocks), runs=tuple(LayerRun(block=i) for i in range(len(blocks))),
            final_norm=norm(), final_norm_name="final.norm", head_name="head", max_positions=MAX_POSITIONS,
            residual_dtype="float32")
        plan.validate()
        return plan
