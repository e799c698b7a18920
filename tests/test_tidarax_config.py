"""Tidarax on the CPU: its configuration reader, its plan, random model folders and the plain
implementation's own properties."""
import copy
import json
import os

import pytest
import torch

import plain_tidarax as plain
from tidarax_models import TINY_T, make_folder, prompts
from xinfer_b200.config import ConfigError, config_from_dict
from xinfer_b200.models.decoder import model_weight_specs


def test_the_architecture_is_chosen_by_name_and_every_size_is_read():
    for name, (raw, _, _) in TINY_T.items():
        entry, cfg = config_from_dict(raw)
        assert entry.name == "Tidarax"
        plan = entry.plan_of(cfg)
        assert plan.vocab_size == raw["vocab"] and plan.hidden == raw["width"] and plan.residual_dtype == "float32"
        assert len(plan.blocks) == len(raw["layers"])
        for block, layer in zip(plan.blocks, raw["layers"]):
            mixer = block.mixer
            left, lf = mixer.left, layer["mixer"]["left"]
            assert (left.num_heads, left.num_kv_heads, left.head_dim, left.value_dim, left.scale) == (
                lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"], lf["scale"])
            assert left.talking_heads and left.sink and left.qk_norm_after_rope and not left.qk_norm_weight
            assert (left.rope is None) == ("rot" not in lf)
            if left.rope is not None:
                assert left.rope.rotary_dim == lf["rot"]["dims"] and left.rope.theta == lf["rot"]["base"]
                assert (left.rope.scaling is None) == ("scaling" not in lf["rot"]) and not left.rope.tables
            assert mixer.right.width == layer["mixer"]["right"]["width"]
            assert (mixer.left_scale, mixer.right_scale) == (layer["mixer"]["left_scale"], layer["mixer"]["right_scale"])
            assert (block.feed_forward is None) == (layer["mlp"] is None)
            for n in block.norms():
                assert n.eps == raw["norm"]["eps"] and n.weight_offset == 1.0


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), None, "vocab"), (("norm", "eps"), 0, "norm.eps"), (("layers", 0, "type"), "serial", "type"),
    (("layers", 0, "mixer", "left", "heads"), 3, "kv_heads"), (("layers", 0, "mixer", "left", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mlp", "kind"), "sparse", "kind"), (("layers", 0, "mlp", "router", "top"), 9, "top"),
    (("layers", 1, "mixer", "right", "width"), -4, "width"), (("layers", 0, "mixer", "left_scale"), "big", "left_scale"),
])
def test_a_bad_key_is_named(path, value, word):
    raw = copy.deepcopy(TINY_T["T1"][0])
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
    folder = make_folder(str(tmp_path / "m"), "T1", torch.bfloat16)
    raw = json.load(open(os.path.join(folder, "config.json")))
    entry, cfg = config_from_dict(raw)
    specs = model_weight_specs(entry.plan_of(cfg))
    store = WeightStore(folder)
    assert store.check(specs, strict=True) == []
    names = {s.name for s in specs}
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.mix.left.talk", "l0.mix.right.z.b", "l0.mlp.e4.down",
            "l0.mlp.table", "l1.mlp.act", "l2.norm1"} <= names and "l2.norm2" not in names
    table = store.raw("l0.mlp.table")
    assert table.dtype == torch.int32 and table.shape == (97, 2)
    assert int(table.min()) >= 0 and int(table.max()) < 5 and bool((table[:, 0] != table[:, 1]).all())
    cfg2, w = plain.load_folder(folder)
    assert plain.forward(cfg2, w, [1, 2, 3]).shape == (3, 97)


def test_plain_recurrence_in_portions_equals_the_whole():
    g = torch.Generator().manual_seed(0)
    W, hid = 12, 10
    w = {n: torch.randn(*s, generator=g, dtype=torch.float64) for n, s in
         [("z", (W, hid)), ("z.b", (W,)), ("x", (W, hid)), ("x.b", (W,)), ("g", (W, hid)), ("o", (hid, W))]}
    h = torch.randn(31, hid, generator=g, dtype=torch.float64)
    whole, S = plain.mingru_branch(h, w, "")
    a, Sa = plain.mingru_branch(h[:13], w, "")
    b, _ = plain.mingru_branch(h[13:], w, "", state=Sa[-1])
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12)


def test_plain_attention_with_an_identity_mix_and_strong_scores_is_a_softmax():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(6, 2, 4, generator=g, dtype=torch.float64)
    k = torch.randn(6, 1, 4, generator=g, dtype=torch.float64)
    v = torch.randn(6, 1, 3, generator=g, dtype=torch.float64)
    out = plain.talking_sink_attention(q, k, v, torch.eye(2, dtype=torch.float64), 1.0)
    s = torch.einsum("ihd,jd->hij", q, k[:, 0]).masked_fill(~torch.ones(6, 6, dtype=torch.bool).tril(), float("-inf"))
    e = torch.exp(s)
    ref = torch.einsum("hij,jd->ihd", e / (1 + e.sum(-1, keepdim=True)), v[:, 0])
    assert torch.allclose(out, ref, atol=1e-12)


def test_prompts_are_in_range():
    assert max(max(p) for p in prompts("T3", [50, 7])) < 150
