"""Tiny Tidarax configurations for the tests (config.json dictionaries) and their random model folders.

They differ from each other in every size and switch: heads and groups, key and value head sizes that
differ, rotation over part of a head or over all of it or none, frequency scaling present or absent,
recurrence widths, scales, the order of feed-forward kinds (dense, experts with one, two or three
choices, none), eps, vocabulary and page size."""
from typing import Dict, List, Sequence

import numpy as np
import torch


def _left(heads, kv, dim, vdim, scale, rot=None):
    out = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if rot is not None:
        out["rot"] = rot
    return out


def _layer(left, left_scale, width, right_scale, mlp):
    return dict(type="parallel", mixer=dict(left=left, left_scale=left_scale, right=dict(width=width), right_scale=right_scale),
                mlp=mlp)


def _moe(ff, experts, top):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


# name -> (config, seed, page size)
TINY_T: Dict[str, tuple] = {
    "T1": (dict(architecture="Tidarax", vocab=97, width=48, norm=dict(eps=1e-5), layers=[
        _layer(_left(4, 2, 16, 24, 0.55, dict(dims=8, base=1000.0, scaling=dict(factor=8.0, low=1.0, high=4.0, original=64))),
               0.7, 40, 1.3, _moe(24, 5, 2)),
        _layer(_left(4, 4, 16, 8, 0.5, dict(dims=16, base=500.0)), 1.0, 56, 0.8, dict(kind="dense", ff=56)),
        _layer(_left(2, 1, 32, 16, 0.4), 1.5, 24, 1.0, None),
    ]), 11, 8),
    "T2": (dict(architecture="Tidarax", vocab=211, width=80, norm=dict(eps=3e-6), layers=[
        _layer(_left(6, 2, 24, 40, 0.45, dict(dims=24, base=20000.0, scaling=dict(factor=2.0, low=2.0, high=8.0, original=48))),
               1.1, 72, 0.9, dict(kind="dense", ff=136)),
        _layer(_left(6, 2, 24, 40, 0.45, dict(dims=12, base=300.0, scaling=dict(factor=16.0, low=1.0, high=2.0, original=16))),
               0.9, 72, 1.2, _moe(40, 4, 3)),
    ]), 12, 16),
    "T3": (dict(architecture="Tidarax", vocab=150, width=64, norm=dict(eps=1e-6), layers=[
        _layer(_left(8, 1, 8, 8, 0.8, dict(dims=8, base=100.0)), 1.0, 64, 1.0, _moe(16, 7, 1)),
        _layer(_left(1, 1, 64, 48, 0.3, dict(dims=32, base=5000.0, scaling=dict(factor=4.0, low=1.0, high=4.0, original=128))),
               2.0, 8, 0.5, None),
        _layer(_left(8, 8, 8, 16, 0.8, dict(dims=2, base=10.0)), 0.6, 100, 1.4, dict(kind="dense", ff=200)),
        _layer(_left(4, 2, 16, 16, 0.6), 1.0, 64, 1.0, _moe(32, 2, 2)),
    ]), 13, 32),
    # sizes that fit no fast path: a width that is no multiple of 8, an odd recurrence width (the attention's rows
    # in the shared activation then start at odd offsets), odd feed-forward sizes
    "T4": (dict(architecture="Tidarax", vocab=61, width=52, norm=dict(eps=2e-6), layers=[
        _layer(_left(3, 1, 32, 16, 0.5, dict(dims=20, base=3000.0, scaling=dict(factor=5.0, low=1.0, high=3.0, original=40))),
               1.2, 37, 0.7, _moe(20, 3, 2)),
        _layer(_left(6, 3, 16, 16, 0.7, dict(dims=16, base=900.0)), 0.8, 44, 1.1, dict(kind="dense", ff=50)),
    ]), 14, 16),
}


def make_folder(path: str, name: str, store_dtype=torch.float32) -> str:
    """config.json and model.safetensors with random weights large enough that every layer matters."""
    from xinfer_b200.weights import write_random_model
    cfg, seed, _ = TINY_T[name]
    return write_random_model(path, cfg, seed, dtype=store_dtype, std=0.08, norm_std=0.2)


def prompts(name: str, lengths: Sequence[int], seed: int = 0) -> List[List[int]]:
    cfg = TINY_T[name][0]
    rng = np.random.default_rng(500 + seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
