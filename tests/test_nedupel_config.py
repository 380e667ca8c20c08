"""Configuration of the Nedupel design: what is read, what is refused, what the parts are built from; and controls
on the plain implementation (it would notice a wrong pairing, a missing scale, a wrong table column)."""
import copy

import numpy as np
import pytest

import nedupel_models as nm
from plain import nedupel as plain
from mynah_slm_b200.config.keys import ConfigError
from mynah_slm_b200.config.nedupel import NedupelConfig
from mynah_slm_b200.registry import parse_config

CFG = nm.HYBRID


def test_registry_reads_the_single_name_key():
    typed = parse_config(CFG)
    assert isinstance(typed, NedupelConfig)
    assert typed.to_dict() == CFG
    assert parse_config(typed.to_dict()).to_dict() == CFG
    with_limit = dict(CFG, max_positions=777)
    assert parse_config(with_limit).model_spec().max_positions == 777 and parse_config(with_limit).to_dict() == with_limit


def test_spec_follows_the_configuration():
    spec = parse_config(CFG).model_spec()
    assert [l.mixer.kind for l in spec.layers] == ["retention", "latent_attention", "latent_attention", "latent_attention",
                                                   "retention", "latent_attention"]
    assert [None if l.ffn is None else l.ffn.kind for l in spec.layers] == [
        "table_routed_experts", "dense_mlp", None, "table_routed_experts", "dense_mlp", "table_routed_experts"]
    assert [e.cache_from for e in spec.schedule] == [None, None, None, 1, None, 2]
    assert [l.mixer["own_kv"] for l in spec.layers if l.mixer.kind == "latent_attention"] == [True, True, False, False]
    assert spec.layers[1].mixer["rot"]["pairing"] == "interleaved" and spec.layers[0].mixer["rot"]["pairing"] == "half"
    assert spec.layers[1].mixer["rot"]["scaling"]["factor"] == 4.0 and "scaling" not in spec.layers[2].mixer["rot"]
    assert all(l.block["residual_mult"] == 0.8 for l in spec.layers)
    assert spec.embedding["scale"] == 3.0 and spec.head["logit_scale"] == 0.5 and spec.head["tied"] is False
    assert spec.layers[0].ffn["limit"] == 1.5 and spec.layers[3].ffn["top"] == 3 and spec.layers[1].ffn["activation"] == "relu2"
    assert spec.final_norm.kind == "rmsnorm_offset" and set(spec.layers[2].norms) == {"mixer"}


def test_cache_plan_shares_latent_caches_and_keeps_states():
    from mynah_slm_b200.engine.model import Model
    model = Model(parse_config(CFG).model_spec())
    plan = model.cache_plan()
    assert [(g.kv_heads, g.head_dim, g.v_head_dim, g.entries) for g in plan.groups] == [(1, 48, 0, [1]), (1, 40, 0, [2])]
    assert [e.source for e in plan.entries] == [None, None, None, 1, None, 2]
    assert plan.entries[0].state["S"].shape == (4, 16, 24) and plan.entries[4].state["S"].shape == (2, 32, 8)
    names = {ts.name: tuple(ts.shape) for _, ts in model.tensor_specs()}
    assert names == nm.tensor_shapes(CFG)
    for name, cfg in nm.CONFIGS.items():
        got = {ts.name: tuple(ts.shape) for _, ts in Model(parse_config(cfg).model_spec()).tensor_specs()}
        assert got == nm.tensor_shapes(cfg), name


def _set(cfg, path, value):
    cfg = copy.deepcopy(cfg)
    d = cfg
    for k in path[:-1]:
        d = d[k]
    if value is _DEL:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    return cfg


_DEL = object()


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "lstm", "type"),
    (("layers", 0, "mixer", "decay"), [0.9, 0.9], "decay"),
    (("layers", 0, "mixer", "rot", "dims"), 18, "rot.dims"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 1, "mixer", "kv_rank"), _DEL, "kv_rank"),
    (("layers", 1, "mixer", "scale"), "big", "scale"),
    (("layers", 1, "mixer", "rot", "scaling", "factor"), 0, "factor"),
    (("layers", 3, "mixer", "kv_from"), 4, "kv_from"),            # a retention layer keeps no latent cache
    (("layers", 3, "mixer", "kv_from"), 5, "kv_from"),            # a later layer
    (("layers", 5, "mixer", "kv_from"), 3, "kv_from"),            # a layer that itself reads another's cache
    (("layers", 3, "mixer", "kv_rank"), 24, "kv_rank"),           # differs from the layer whose cache it reads
    (("layers", 3, "mlp", "router", "top"), 6, "top"),
    (("layers", 1, "mlp", "kind"), "glu", "kind"),
    (("norm", "eps"), 0.0, "eps"),
    (("residual_mult",), _DEL, "residual_mult"),
    (("embedding",), _DEL, "embedding"),
    (("logit_scale",), None, "logit_scale"),
    (("vocab",), 12.5, "vocab"),
])
def test_refusals_name_the_key(path, value, word):
    with pytest.raises(ConfigError) as e:
        parse_config(_set(CFG, path, value)).model_spec()
    assert word in str(e.value)


def test_random_tables_hold_different_experts():
    from mynah_slm_b200.parts.base import TensorSpec
    from mynah_slm_b200.weights.random_init import table_tensor
    for rows, top, E in ((300, 2, 6), (50, 7, 7), (64, 1, 1), (1000, 3, 70)):
        t = table_tensor(TensorSpec("t", (rows, top), role="table", init=f"distinct:{E}"), seed=5).numpy()
        assert t.min() >= 0 and t.max() < E and all(len(set(r)) == top for r in t)
        if E > top:
            assert len(np.unique(t[:, 0])) > 1
    with pytest.raises(ValueError):
        table_tensor(TensorSpec("t", (4, 3), role="table", init="distinct:2"), seed=0)


def test_rotary_frequencies_match_the_plain_angles():
    from mynah_slm_b200.parts.position import rotary_frequencies
    for rot in ({"dims": 16, "base": 5000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}},
                {"dims": 6, "base": 20.0}, {"dims": 32, "base": 1e6, "scaling": {"factor": 8.0, "original": 32, "fast": 8.0, "slow": 2.0}}):
        f, mult = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        a, m = plain.rotary_angles([0, 1, 7, 1000], rot)
        assert m == pytest.approx(mult, rel=1e-15)
        np.testing.assert_allclose(np.outer([0, 1, 7, 1000], f), a, rtol=1e-14)
    # the interpolation leaves fast pairs alone, slows slow pairs by the factor and blends between
    f, _ = rotary_frequencies(32, 1e4, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0})
    g, _ = rotary_frequencies(32, 1e4, None)
    ratio = np.asarray(f) / np.asarray(g)
    assert ratio[0] == 1.0 and ratio[-1] == pytest.approx(1 / 8.0) and np.all(np.diff(ratio) <= 1e-12) and len(set(ratio)) > 2


# ------------------------------------------------------------------ controls on the plain implementation
def _logits(cfg, W, toks):
    return plain.forward(cfg, W, toks)


def _differs(a, b):
    return np.abs(a - b).max() > 1e-3 * np.abs(a).max()


@pytest.fixture(scope="module")
def hybrid(tmp_path_factory):
    W = nm.make_weights(CFG, 7)
    import torch
    return {n: (t.to(torch.float64) if t.dtype.is_floating_point else t.to(torch.int64)).numpy() for n, t in W.items()}


def test_plain_notices_wrong_readings(hybrid):
    toks = np.random.default_rng(3).integers(0, CFG["vocab"], size=40).tolist()
    ref = _logits(CFG, hybrid, toks)
    for path, value in [(("residual_mult",), 1.0), (("embedding", "scale"), 1.0), (("layers", 1, "mixer", "scale"), 0.31),
                        (("layers", 1, "mixer", "rot", "scaling", "factor"), 2.0), (("layers", 0, "mixer", "decay"), [0.9, 0.95, 0.99, 0.99]),
                        (("layers", 5, "mixer", "kv_from"), 1 if False else 2), (("norm", "eps"), 1e-2)]:
        other = _logits(_set(CFG, path, value), hybrid, toks)
        if path == ("layers", 5, "mixer", "kv_from"):
            assert not _differs(ref, other)             # the same value: the control of the control
        else:
            assert _differs(ref, other), path
    # pairing: the two layouts are different functions
    x = np.random.default_rng(0).normal(size=(5, 2, 8))
    rot = {"dims": 8, "base": 100.0}
    assert _differs(plain.rotate(x, np.arange(5), rot, "interleaved"), plain.rotate(x, np.arange(5), rot, "half"))
    # a table's second column counts
    swapped = dict(hybrid)
    t = hybrid["l0.mlp.table"].copy()
    t[:, 1] = (t[:, 1] + 1) % 6
    t[:, 1] = np.where(t[:, 1] == t[:, 0], (t[:, 1] + 1) % 6, t[:, 1])
    swapped["l0.mlp.table"] = t
    assert _differs(ref, _logits(CFG, swapped, toks))


def test_plain_latent_attention_equals_its_query_side_form(hybrid):
    """The identity the kernels rest on: q_u . (W_uk c) = (W_uk^T q_u) . c, and sum p (W_uv c) = W_uv (sum p c)."""
    m = CFG["layers"][1]["mixer"]
    rng = np.random.default_rng(1)
    T, H, dim, rd, vd, r = 30, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    h = rng.normal(size=(T, CFG["width"]))
    pos = np.arange(T)
    ref = plain.latent_attention(h, hybrid, "l1.mix.", m, 1e-5, pos)
    c, kr = plain.latent_kv(h, hybrid, "l1.mix.", m, 1e-5, pos)
    q = (h @ hybrid["l1.mix.q"].T).reshape(T, H, dim + rd)
    qr = plain.rotate(q[..., dim:], pos, m["rot"], "interleaved")
    Wuk, Wuv = hybrid["l1.mix.uk"].reshape(H, dim, r), hybrid["l1.mix.uv"].reshape(H, vd, r)
    rows = np.concatenate([c, kr], 1)
    out = np.zeros((T, H, vd))
    for hd in range(H):
        qa = np.concatenate([q[:, hd, :dim] @ Wuk[hd], qr[:, hd]], 1)
        s = np.where(np.tril(np.ones((T, T), bool)), qa @ rows.T * m["scale"], -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        out[:, hd] = (p @ rows)[:, :r] @ Wuv[hd].T
    np.testing.assert_allclose(out.reshape(T, -1) @ hybrid["l1.mix.o"].T, ref, rtol=1e-9, atol=1e-10)
