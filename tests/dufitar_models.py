"""Tiny Dufitar configurations for the tests (config.json dictionaries) and their random model folders.

They differ from each other in every size and switch: heads and groups (one group, one head per group), key and
value head sizes that differ, rotation over part of a head or all of it, frequency scaling present or absent,
windows shorter and longer than a page and than the prompts, latent ranks that differ from the head sizes, latent
layers that read another layer's rows with a longer or a shorter window of their own, layers without a feed-forward,
residual factors, embedding scales, vocabulary and page size."""
from typing import Dict, List, Sequence

import numpy as np
import torch


def _attn(heads, kv, dim, vdim, scale, window, rot):
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale,
                                             mask=dict(size=window), rot=rot))


def _latent(heads, dim, rot_dim, vdim, rank, scale, window, base, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=scale, mask=dict(size=window),
             rot=dict(dims=rot_dim, base=base))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def _with(layer, ff):
    layer = dict(layer)
    layer["mlp"] = None if ff is None else dict(kind="dense", ff=ff)
    return layer


def _yarn(factor, original, fast, slow):
    return dict(factor=factor, original=original, fast=fast, slow=slow)


# name -> (config, seed, page size)
TINY_D: Dict[str, tuple] = {
    "D1": (dict(architecture="Dufitar", vocab=83, width=48, norm=dict(eps=1e-5), residual_mult=0.6, embedding=dict(scale=2.0),
                layers=[
        _with(_attn(4, 2, 16, 24, 1.1, 11, dict(dims=8, base=1000.0, scaling=_yarn(8.0, 64, 16.0, 2.0))), 56),
        _with(_latent(3, 8, 4, 12, 20, 1.3, 19, 300.0), 40),
        _with(_latent(2, 12, 4, 8, 20, 0.9, 27, 300.0, kv_from=1), None),
        _with(_attn(2, 1, 32, 16, 0.8, 64, dict(dims=32, base=500.0)), 72),
    ]), 21, 8),
    "D2": (dict(architecture="Dufitar", vocab=157, width=64, norm=dict(eps=3e-6), residual_mult=1.0, embedding=dict(scale=0.5),
                layers=[
        _with(_latent(5, 16, 8, 16, 24, 0.7, 33, 10000.0), 96),
        _with(_attn(6, 6, 8, 8, 1.5, 7, dict(dims=4, base=50.0, scaling=_yarn(2.0, 32, 8.0, 1.0))), None),
        _with(_latent(1, 24, 8, 40, 24, 1.0, 16, 10000.0, kv_from=0), 80),
    ]), 22, 16),
    # head sizes the tensor-core attention kernels take (multiples of 16, key and value sizes equal), a window of
    # several pages, a latent layer of its own beside one that is shared twice
    "D3": (dict(architecture="Dufitar", vocab=120, width=96, norm=dict(eps=1e-6), residual_mult=0.8, embedding=dict(scale=1.5),
                layers=[
        _with(_attn(4, 2, 32, 32, 0.6, 50, dict(dims=16, base=20000.0, scaling=_yarn(3.0, 128, 20.0, 1.0))), 160),
        _with(_latent(4, 32, 16, 32, 48, 0.5, 70, 5000.0), 128),
        _with(_attn(8, 1, 16, 16, 0.9, 23, dict(dims=16, base=100.0)), 64),
        _with(_latent(2, 16, 16, 24, 48, 0.6, 45, 5000.0, kv_from=1), 128),
        _with(_latent(6, 8, 16, 8, 48, 0.8, 120, 5000.0, kv_from=1), None),
        _with(_latent(3, 8, 2, 8, 10, 1.2, 9, 40.0), 32),
    ]), 23, 32),
    # sizes that fit no fast path: odd widths, head sizes that are no multiple of 4, a window of one
    "D4": (dict(architecture="Dufitar", vocab=61, width=52, norm=dict(eps=2e-6), residual_mult=1.3, embedding=dict(scale=3.5),
                layers=[
        _with(_attn(3, 1, 10, 6, 1.0, 1, dict(dims=6, base=3000.0, scaling=_yarn(5.0, 40, 10.0, 3.0))), 50),
        _with(_latent(3, 6, 2, 10, 14, 1.1, 13, 900.0), 37),
        _with(_attn(2, 2, 18, 22, 0.7, 200, dict(dims=2, base=10.0)), None),
    ]), 24, 16),
    # wide heads and a wide latent: the widest tiles of the tensor-core kernels (heads of 128 channels, a latent whose
    # value columns are shared out among eight warps), windows of several key tiles
    "D5": (dict(architecture="Dufitar", vocab=200, width=128, norm=dict(eps=1e-6), residual_mult=0.9, embedding=dict(scale=1.2),
                layers=[
        _with(_latent(3, 32, 16, 48, 128, 0.4, 150, 7000.0), 96),
        _with(_attn(2, 1, 128, 128, 0.3, 100, dict(dims=64, base=40000.0, scaling=_yarn(2.5, 96, 12.0, 1.0))), 192),
        _with(_latent(2, 16, 16, 16, 128, 0.5, 66, 7000.0, kv_from=0), None),
    ]), 25, 16),
}


def make_folder(path: str, name: str, store_dtype=torch.float32, override=None) -> str:
    """config.json and model.safetensors with random weights large enough that every layer matters."""
    from xinfer_b200.weights import write_random_model
    cfg, seed, _ = TINY_D[name]
    return write_random_model(path, cfg, seed, dtype=store_dtype, std=0.08, norm_std=0.2, override=override)


def prompts(name: str, lengths: Sequence[int], seed: int = 0) -> List[List[int]]:
    cfg = TINY_D[name][0]
    rng = np.random.default_rng(700 + seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
