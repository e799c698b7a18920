"""Dufitar on the CPU: its configuration reader, its plan, random model folders, the rotary frequencies and the
plain implementation's own properties."""
import copy
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_dufitar as plain
from dufitar_models import TINY_D, make_folder, prompts
from xinfer_b200.config import ConfigError, config_from_dict
from xinfer_b200.config.plan import YarnScaling
from xinfer_b200.models.decoder import model_weight_specs


def test_the_architecture_is_chosen_by_name_and_every_size_is_read():
    for name, (raw, _, _) in TINY_D.items():
        entry, cfg = config_from_dict(raw)
        assert entry.name == "Dufitar"
        plan = entry.plan_of(cfg)
        assert plan.vocab_size == raw["vocab"] and plan.hidden == raw["width"] and plan.residual_dtype == "float32"
        assert plan.embed_scale == raw["embedding"]["scale"] and plan.head_name is None
        assert len(plan.blocks) == len(raw["layers"]) == len(plan.runs)
        for i, (block, run, layer) in enumerate(zip(plan.blocks, plan.runs, raw["layers"])):
            mixer, m = block.mixer, layer["mixer"]
            assert run.block == i and run.cache_from == m.get("kv_from")
            assert (mixer.num_heads, mixer.head_dim, mixer.scale, mixer.window) == (m["heads"], m["dim"], m["scale"], m["mask"]["size"])
            assert mixer.rope.rotary_dim == m["rot"]["dims"] and mixer.rope.theta == m["rot"]["base"]
            assert mixer.rope.layout == "interleaved" and not mixer.rope.tables
            if layer["type"] == "attention":
                assert (mixer.num_kv_heads, mixer.value_dim) == (m["kv_heads"], m["vdim"])
                assert not mixer.talking_heads and not mixer.sink and not mixer.qk_norm
                sc = m["rot"].get("scaling")
                assert (mixer.rope.scaling is None) == (sc is None)
                if sc:
                    assert mixer.rope.scaling == YarnScaling(sc["factor"], sc["original"], sc["fast"], sc["slow"])
                    assert mixer.rope.magnitude == pytest.approx(0.1 * math.log(sc["factor"]) + 1.0)
            else:
                assert (mixer.rope_dim, mixer.v_head_dim, mixer.kv_rank) == (m["rot_dim"], m["vdim"], m["kv_rank"])
                assert mixer.sink and mixer.gate and mixer.shares_cache == ("kv_from" in m)
                assert mixer.norm_eps == raw["norm"]["eps"] and mixer.rope.magnitude == 1.0
            adds = block.ops_of("add")
            assert all(a.scale == raw["residual_mult"] for a in adds)
            assert len(adds) == (1 if layer["mlp"] is None else 2) and len(block.norms()) == 2 * len(adds)
            assert (block.feed_forward is None) == (layer["mlp"] is None)
            if layer["mlp"] is not None:
                assert block.feed_forward.intermediate == layer["mlp"]["ff"] and block.feed_forward.activation == "gelu_tanh"


def test_cached_rows_are_kept_for_the_widest_reader():
    raw, _, _ = TINY_D["D3"]
    entry, cfg = config_from_dict(raw)
    plan = entry.plan_of(cfg)
    # layer 1 is read by layers 3 and 4 with windows 45 and 120; its own is 70
    assert plan.blocks[1].mixer.cache_window == 120 and plan.blocks[1].mixer.window == 70
    assert plan.blocks[5].mixer.cache_window == 9
    raw2, _, _ = TINY_D["D2"]
    entry, cfg = config_from_dict(raw2)
    assert entry.plan_of(cfg).blocks[0].mixer.cache_window == 33      # the reader's window (16) is the shorter one


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), None, "vocab"), (("norm", "eps"), 0, "norm.eps"), (("layers", 0, "type"), "parallel", "type"),
    (("layers", 0, "mixer", "heads"), 3, "kv_heads"), (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mlp", "kind"), "moe", "kind"), (("layers", 1, "mixer", "kv_rank"), -4, "kv_rank"),
    (("residual_mult",), "big", "residual_mult"), (("embedding",), None, "embedding"),
    (("layers", 2, "mixer", "kv_from"), 0, "kv_from"), (("layers", 2, "mixer", "kv_from"), 2, "kv_from"),
    (("layers", 2, "mixer", "kv_rank"), 24, "kv_rank"), (("layers", 0, "mixer", "rot", "scaling", "factor"), 0, "factor"),
    (("layers", 1, "mixer", "rot_dim"), None, "rot_dim"),
])
def test_a_bad_key_is_named(path, value, word):
    raw = copy.deepcopy(TINY_D["D1"][0])
    at = raw
    for p in path[:-1]:
        at = at[p]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_random_folder_holds_the_declared_tensors(tmp_path):
    from xinfer_b200.weights.loader import WeightStore
    folder = make_folder(str(tmp_path / "m"), "D1", torch.bfloat16)
    raw = json.load(open(os.path.join(folder, "config.json")))
    entry, cfg = config_from_dict(raw)
    specs = model_weight_specs(entry.plan_of(cfg))
    store = WeightStore(folder)
    assert store.check(specs, strict=True) == []
    names = {s.name: tuple(s.shape) for s in specs}
    assert {"embed", "final.norm", "final.norm.b", "final.norm.alpha", "l0.norm1b.alpha", "l0.mix.k", "l1.mix.dkv",
            "l1.mix.dkv.norm", "l1.mix.sink", "l1.mix.g", "l2.mix.uk", "l3.mlp.gate"} <= set(names)
    assert "l2.mix.dkv" not in names and "l2.norm2" not in names and "head" not in names
    assert names["l0.norm1.alpha"] == () and names["l1.mix.dkv"] == (24, 48) and names["l2.mix.uv"] == (16, 20)
    cfg2, w = plain.load_folder(folder)
    assert plain.forward(cfg2, w, [1, 2, 3]).shape == (3, 83)


@pytest.mark.parametrize("rot", [
    dict(dims=8, base=1000.0, scaling=dict(factor=8.0, original=64, fast=16.0, slow=2.0)),
    dict(dims=40, base=80000.0, scaling=dict(factor=6.0, original=256, fast=24.0, slow=1.5)),
    dict(dims=6, base=3000.0, scaling=dict(factor=5.0, original=40, fast=10.0, slow=3.0)),
    dict(dims=2, base=10.0, scaling=dict(factor=3.0, original=8, fast=4.0, slow=1.0)),     # hi == lo: the 0.001 floor
    dict(dims=12, base=70000.0),
])
def test_scaled_frequencies_equal_the_plain_rule(rot):
    from xinfer_b200.parts.rope import inv_frequencies
    sc = rot.get("scaling")
    scaling = YarnScaling(sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None
    got = inv_frequencies(rot["base"], rot["dims"], scaling, True)
    want, _ = plain.rotary_frequencies(rot)
    assert np.allclose(got, want.numpy(), rtol=1e-6, atol=0)
    if sc:   # the fastest pair keeps its frequency, the slowest is slowed by the whole factor (if the ramp reaches it)
        assert got[0] == pytest.approx(1.0 if rot["dims"] > 2 else got[0])


def test_plain_softmax_with_a_sink_gives_less_than_one():
    s = torch.tensor([[0.5, -1.0, 2.0]], dtype=torch.float64)
    mask = torch.ones(1, 3, dtype=torch.bool)
    p = plain.softmax_rows(s, mask, sink=torch.tensor(1.0, dtype=torch.float64))
    assert float(p.sum()) == pytest.approx(float(torch.exp(s).sum() / (torch.exp(s).sum() + math.e)))
    very = plain.softmax_rows(s, mask, sink=torch.tensor(50.0, dtype=torch.float64))
    assert float(very.sum()) < 1e-18


def test_plain_window_keeps_exactly_size_keys():
    m = plain.visible(9, 3)
    assert m.sum(dim=1).tolist() == [1, 2, 3, 3, 3, 3, 3, 3, 3] and bool(m[5, 3]) and not bool(m[5, 2]) and not bool(m[5, 6])
    assert plain.visible(4, None).sum().item() == 10


def test_plain_rotation_pairs_neighbours_and_leaves_the_rest():
    x = torch.arange(12, dtype=torch.float64).reshape(1, 1, 12) + 1.0
    y = plain.rotate(x, torch.tensor([3]), dict(dims=4, base=100.0))
    assert torch.equal(y[..., 4:], x[..., 4:])
    a = 3.0 * 100.0 ** (-2.0 / 4.0)
    assert float(y[0, 0, 2]) == pytest.approx(3.0 * math.cos(a) - 4.0 * math.sin(a))
    assert float(y[0, 0, 3]) == pytest.approx(4.0 * math.cos(a) + 3.0 * math.sin(a))


def test_prompts_are_in_range():
    assert max(max(p) for p in prompts("D3", [50, 7])) < 120
