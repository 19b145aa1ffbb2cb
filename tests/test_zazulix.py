"""The Zazulix decoder on the CPU: its configuration, the model's description, and the plain implementation's own
mechanisms against closed forms."""
import numpy as np
import pytest

import plain_zazulix as P
import zazulix_models as M


@pytest.mark.parametrize("which", sorted(M.CONFIGS))
def test_configuration_round_trip_and_declared_tensors(which):
    from hk_b200.config import ZazulixConfig, config_from_dict, resolve_architecture
    raw = M.CONFIGS[which]
    cfg = config_from_dict(raw)
    assert isinstance(cfg, ZazulixConfig) and config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    _, build = resolve_architecture("Zazulix")
    model = build(cfg, 64)
    specs = model.param_specs()
    assert "embed" in specs and "final.norm" in specs and specs["head"].optional
    for i, layer in enumerate(raw["layers"]):
        m, mlp = layer["mixer"], layer["mlp"]
        d = raw["width"]
        if layer["type"] == "attention":
            assert specs[f"l{i}.mix.q"].shape == (m["heads"] * 2 * m["dim"], d)
            assert specs[f"l{i}.mix.k"].shape == (m["kv_heads"] * 2 * m["dim"], d)
            assert specs[f"l{i}.mix.v"].shape == (m["kv_heads"] * m["vdim"], d)
            assert specs[f"l{i}.mix.g"].shape == (m["heads"], d) and specs[f"l{i}.mix.lq2"].shape == (m["dim"],)
            assert (f"l{i}.mix.k.conv" in specs) == bool(m.get("conv"))
            if m.get("conv"):
                assert specs[f"l{i}.mix.v.conv"].shape == (m["kv_heads"] * m["vdim"], m["conv"])
        elif layer["type"] == "retention":
            assert specs[f"l{i}.mix.g"].shape == (m["heads"] * m["vdim"], d)
        else:
            assert specs[f"l{i}.mix.dkv"].shape == (m["kv_rank"], d) and specs[f"l{i}.mix.uk"].shape == (m["heads"] * m["dim"], m["kv_rank"])
        if mlp is None:
            assert f"l{i}.norm2" not in specs
        elif mlp["kind"] == "moe":
            E = mlp["router"]["experts"]
            assert specs[f"l{i}.mlp.router"].shape == (E, d) and specs[f"l{i}.mlp.correction"].shape == (E,)
            assert f"l{i}.mlp.e{E - 1}.down" in specs and f"l{i}.mlp.e{E}.down" not in specs
            assert (f"l{i}.mlp.shared.sg" in specs) == bool(mlp.get("shared"))
        else:
            assert specs[f"l{i}.mlp.gate"].shape == (mlp["ff"], d)
    caches = model.cache_specs()
    assert len(caches) == len(raw["layers"])


def test_configuration_errors_name_the_key():
    from hk_b200.config import ConfigError, config_from_dict
    import copy
    for path, value, word in ((("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 1, "mixer", "decay"), [0.5], "decay"),
                              (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"), (("layers", 0, "type"), "mamba", "type"),
                              (("layers", 1, "mlp", "limit"), -1.0, "limit")):
        raw = copy.deepcopy(M.CONFIGS["A"])
        at = raw
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(raw)


def test_plain_retention_is_its_closed_form():
    rng = np.random.default_rng(0)
    T, d, H, dk, dv = 12, 10, 2, 4, 3
    w = {"m." + k: rng.standard_normal(s) for k, s in (("q", (H * dk, d)), ("k", (H * dk, d)), ("v", (H * dv, d)), ("g", (H * dv, d)),
                                                       ("o", (d, H * dv)))}
    m = {"heads": H, "dim": dk, "vdim": dv, "decay": [0.9, 0.5]}
    h = rng.standard_normal((T, d))
    q, k, v = (h @ w["m.q"].T).reshape(T, H, dk), (h @ w["m.k"].T).reshape(T, H, dk) * dk ** -0.5, (h @ w["m.v"].T).reshape(T, H, dv)
    o = np.zeros((T, H, dv))
    for hh in range(H):
        for t in range(T):
            for j in range(t + 1):
                o[t, hh] += m["decay"][hh] ** (t - j) * (q[t, hh] @ k[j, hh]) * v[j, hh]
    want = (P.rms(o, 1e-6).reshape(T, -1) * P.silu(h @ w["m.g"].T)) @ w["m.o"].T
    np.testing.assert_allclose(P.retention(h, w, "m.", m, 1e-6), want, rtol=1e-9, atol=1e-9)


def test_plain_router_groups_weights_and_negative_scores():
    z = np.array([2.0, -1.0, 1.5, -0.4, 3.0, -4.0])
    s = P.sigmoid(z)
    # two groups of three; group scores are the sums of the two largest: the first group wins although the largest single
    # score (expert 4) lies in the second
    corr = np.zeros(6)
    chosen, weights, _ = P.route(z, corr, 2, {"count": 2, "keep": 1})
    assert sorted(chosen) == [0, 2] and np.isclose(weights.sum(), 1.0)
    np.testing.assert_allclose(weights, s[chosen] / s[chosen].sum())
    # the correction moves the choice, not the weights
    corr = np.array([0.0, 5.0, 0.0, 0.0, 0.0, 0.0])
    chosen, weights, _ = P.route(z, corr, 2, {"count": 2, "keep": 1})
    assert sorted(chosen) == [0, 1]
    np.testing.assert_allclose(weights, s[chosen] / s[chosen].sum())
    # all choice scores negative: the refused group's experts are never chosen
    chosen, _, _ = P.route(z, np.full(6, -3.0), 3, {"count": 2, "keep": 1})
    assert sorted(chosen) == [0, 1, 2]
    # without groups the three largest
    chosen, _, _ = P.route(z, np.zeros(6), 3, None)
    assert chosen == [4, 0, 2]


def test_plain_convolution_and_rotation():
    x = np.arange(12.0).reshape(6, 2)
    wt = np.array([[1.0, 0.0, 0.0], [0.0, 0.0, 2.0]])            # channel 0: the input two rows back; channel 1: twice the current one
    y = P.short_conv(x, wt)
    np.testing.assert_allclose(y[:, 0], [0, 0, 0, 2, 4, 6])
    np.testing.assert_allclose(y[:, 1], x[:, 1] * 2)
    rot = {"base": 100.0, "dims": 4}
    q = np.random.default_rng(1).standard_normal((5, 2, 6))
    r = P.rotate(q, np.arange(5), rot)
    np.testing.assert_allclose(r[..., 4:], q[..., 4:])                                   # the rest passes unchanged
    np.testing.assert_allclose(np.linalg.norm(r, axis=-1), np.linalg.norm(q, axis=-1))   # a rotation
    np.testing.assert_allclose(r[0], q[0])                                               # position 0: angle 0
    a = 3 * 100.0 ** (-2.0 / 4)
    np.testing.assert_allclose(r[3, 1, 1], q[3, 1, 1] * np.cos(a) - q[3, 1, 3] * np.sin(a))
