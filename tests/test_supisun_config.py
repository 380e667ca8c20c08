"""Configuration of the Supisun design: what is read, what is refused, what the parts are built from."""
import copy

import numpy as np
import pytest

from mynah_slm_b200.config.keys import ConfigError
from mynah_slm_b200.config.supisun import SupisunConfig
from mynah_slm_b200.registry import parse_config

CFG = {
    "architecture": "Supisun", "vocab": 120, "width": 32, "max_positions": 128, "norm": {"eps": 1e-5},
    "canon": {"taps": 3},
    "layers": [
        {"type": "mamba1", "mixer": {"inner": 48, "state": 4, "dt_rank": 2, "conv": 3}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 12, "vdim": 20, "scale": 0.3,
                                        "rot": {"dims": 4, "base": 100.0}, "mask": {"size": 24}, "v_mix": True},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "conv": 2}, "mlp": {"kind": "dense", "ff": 24}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 8, "vdim": 20, "scale": 0.5, "v_mix": True},
         "mlp": None},
    ],
}


def test_registry_reads_the_single_name_key():
    typed = parse_config(CFG)
    assert isinstance(typed, SupisunConfig)
    assert typed.to_dict() == CFG
    assert parse_config(typed.to_dict()).to_dict() == CFG


def test_spec_follows_the_configuration():
    spec = parse_config(CFG).model_spec()
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["mamba1", "projnorm_attention", "gated_delta", "projnorm_attention"]
    assert [l.ffn is None for l in spec.layers] == [True, False, False, True]
    a1, a3 = spec.layers[1].mixer, spec.layers[3].mixer
    assert (a1["value_mix"], a3["value_mix"]) == ("first", "mix")
    assert (a1["chunk"], a3["chunk"]) == (24, None)
    assert (a1["rot_dims"], a3["rot_dims"]) == (4, 0)
    assert a1["scale"] == 0.3 and a3["scale"] == 0.5
    assert all(l.block["input_conv_taps"] == 3 for l in spec.layers)
    assert spec.embedding.kind == "token_position_embedding" and spec.final_norm.kind == "layernorm"


def test_cache_plan_has_every_state():
    from mynah_slm_b200.engine.model import Model
    plan = Model(parse_config(CFG).model_spec()).cache_plan()
    assert [g.entries for g in plan.groups] == [[1], [3]]                    # heads of 12 and 8: two storage groups
    assert [(g.head_dim, g.v_head_dim) for g in plan.groups] == [(16, 24), (8, 24)]      # stored padded to multiples of 8
    assert sorted(plan.entries[0].state) == ["conv", "scan"] and plan.entries[0].state["scan"].shape == (48, 4)
    assert sorted(plan.entries[2].state) == ["S", "conv"] and plan.entries[2].state["S"].shape == (2, 8, 8)
    assert plan.entries[2].state["conv"].shape == (1, 2 * 2 * 8 + 2 * 8)
    assert all(e.block_state["input_conv"].shape == (2, 32) for e in plan.entries)


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "lstm", "type"),
    (("layers", 1, "mixer", "heads"), 3, "kv_heads"),              # 3 query heads on ... still a multiple of 1
    (("layers", 1, "mixer", "rot", "dims"), 5, "rot.dims"),
    (("layers", 1, "mlp", "kind"), "moe", "kind"),
    (("norm", "eps"), 0.0, "eps"),
    (("layers", 3, "mixer", "vdim"), 16, "vdim"),                   # cannot mix with the first layer's values
])
def test_refusals(path, value, word):
    cfg = copy.deepcopy(CFG)
    d = cfg
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    if path == ("layers", 1, "mixer", "heads"):
        cfg["layers"][1]["mixer"]["kv_heads"] = 2
    with pytest.raises(ConfigError) as e:
        parse_config(cfg).model_spec()
    assert word in str(e.value)


def test_missing_keys_are_named():
    for path in (("vocab",), ("canon",), ("layers", 0, "mixer", "state"), ("layers", 2, "mixer", "conv"),
                 ("layers", 1, "mixer", "scale")):
        cfg = copy.deepcopy(CFG)
        d = cfg
        for k in path[:-1]:
            d = d[k]
        del d[path[-1]]
        with pytest.raises(ConfigError) as e:
            parse_config(cfg)
        assert path[-1] in str(e.value)


def test_plain_controls():
    """The plain implementation would notice the readings that are easy to get wrong."""
    from plain import supisun as plain
    rng = np.random.default_rng(0)
    x = rng.normal(size=(6, 3))
    w = rng.normal(size=(3, 4))
    y = plain.causal_conv(x, w)
    assert np.allclose(y[0], w[:, 3] * x[0])                        # the last column weighs the current token
    assert np.allclose(y[2], w[:, 1] * x[0] + w[:, 2] * x[1] + w[:, 3] * x[2])
    q = rng.normal(size=(5, 2, 8))
    r = plain.rotate_half(q, 4, 10.0)
    assert np.allclose(r[0], q[0]) and np.allclose(r[..., 4:], q[..., 4:])      # position 0 and the unrotated rest
    assert np.allclose((r[..., :4] ** 2).sum(-1), (q[..., :4] ** 2).sum(-1))
    ang = 3 * 10.0 ** (-2 * 1 / 4)
    assert np.allclose(r[3, 0, 1], q[3, 0, 1] * np.cos(ang) - q[3, 0, 3] * np.sin(ang))
    vis = plain.visible(10, 4)
    assert vis[5].tolist() == [False] * 4 + [True, True] + [False] * 4
    assert vis[4].tolist() == [False] * 4 + [True] + [False] * 5
