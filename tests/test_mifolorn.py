"""The Mifolorn decoder on the CPU: its configuration, the order in which its layers run, the tensors it declares,
and the plain implementation's own consistency."""
import math

import numpy as np
import pytest

import mifolorn_models as M
import plain_mifolorn as P


def test_configuration_round_trip_and_errors():
    from hk_b200.config import ConfigError, MifolornConfig, config_from_dict
    for raw in M.CONFIGS.values():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, MifolornConfig) and config_from_dict(cfg.to_dict()) == cfg
    cfg = config_from_dict(M.CONFIGS["U"])
    assert cfg.side_dim == 6 and cfg.embedding_scale == 3.0 and (cfg.loop.start, cfg.loop.stop, cfg.loop.times) == (1, 3, 3)
    left = cfg.layers[1].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.softcap, left.rot.dims) == (4, 2, 16, 16, 20.0, 8)
    assert cfg.layers[1].mixer.right.conv == 3 and cfg.layers[2].mlp is None and cfg.layers[2].mixer.gate_cap == 8.0
    plain = config_from_dict(M.CONFIGS["V"])
    assert plain.loop is None and plain.side_dim == 0 and plain.layers[1].mixer.left.softcap == 0.0

    def broken(change):
        import copy
        raw = copy.deepcopy(M.CONFIGS["U"])
        change(raw)
        with pytest.raises(ConfigError):
            config_from_dict(raw)
    broken(lambda r: r["layers"][0].__setitem__("type", "conv"))
    broken(lambda r: r["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3))
    broken(lambda r: r["layers"][0]["mixer"].__setitem__("conv", 0))
    broken(lambda r: r["layers"][2]["mixer"].__setitem__("gate_cap", 0))
    broken(lambda r: r["loop"].__setitem__("stop", 9))
    broken(lambda r: r["norm"].__setitem__("eps", 0))


@pytest.mark.parametrize("which", ["U", "V", "W", "X"])
def test_schedule_and_declared_tensors(which):
    from hk_b200.config import config_from_dict
    from hk_b200.models.mifolorn import build_mifolorn
    from hk_b200.parts import KVCacheSpec, StateSpec
    raw = M.CONFIGS[which]
    model = build_mifolorn(config_from_dict(raw), 64)
    assert [(c.layer, c.add_embedding) for c in model.schedule] == P.layer_runs(raw)
    specs = model.param_specs()
    n = len(raw["layers"])
    assert specs["embed"].shape == (raw["vocab"], raw["width"]) and specs["head"].optional
    if "token_side" in raw:
        assert specs["side.embed"].shape == (raw["vocab"], n * raw["token_side"]["dim"])
        assert specs["l0.side.gate"].shape == (raw["token_side"]["dim"], raw["width"])
    else:
        assert not any(".side." in k or k == "side.embed" for k in specs)
    for i, entry in enumerate(raw["layers"]):
        m = entry["mixer"]
        if entry["type"] == "parallel":
            lf, rt = m["left"], m["right"]
            assert specs[f"l{i}.mix.left.v.b"].shape == (lf["kv_heads"] * lf["vdim"],)
            assert specs[f"l{i}.mix.left.g"].shape == (lf["heads"] * lf["vdim"], raw["width"])
            assert specs[f"l{i}.mix.right.k.conv"].shape == (rt["kv_heads"] * rt["dim"], rt["conv"])
            assert specs[f"l{i}.mix.right.norm"].shape == (rt["vdim"],)
        elif entry["type"] == "mlstm":
            assert specs[f"l{i}.mix.i"].shape == (m["heads"], raw["width"]) and specs[f"l{i}.mix.f.b"].shape == (m["heads"],)
            assert specs[f"l{i}.mix.norm"].shape == (m["heads"] * m["vdim"],)
        else:
            assert specs[f"l{i}.mix.A_log"].shape == (m["heads"],) and specs[f"l{i}.mix.v.conv"].shape == (m["heads"] * m["vdim"], m["conv"])
        assert (f"l{i}.mlp.down" in specs) == (entry["mlp"] is not None)
    # every run of a layer keeps caches of its own: pages for an attention, two states for each recurrent mixer
    per_run = model.cache_specs()
    assert len(per_run) == len(model.schedule)
    for call, caches in zip(model.schedule, per_run):
        kind = raw["layers"][call.layer]["type"]
        assert [type(c) for c in caches] == ([KVCacheSpec, StateSpec, StateSpec] if kind == "parallel" else [StateSpec, StateSpec])


def test_a_loop_that_is_absent_or_empty_runs_every_layer_once():
    from hk_b200.config.mifolorn import MifolornLoop
    from hk_b200.models.mifolorn import layer_calls
    assert [c.layer for c in layer_calls(3, None)] == [0, 1, 2]
    assert [c.layer for c in layer_calls(3, MifolornLoop(1, 1, 4))] == [0, 1, 2]
    calls = layer_calls(4, MifolornLoop(2, 4, 2))
    assert [(c.layer, c.add_embedding) for c in calls] == [(0, False), (1, False), (2, False), (3, False), (2, True), (3, False)]


def test_plain_short_convolution_and_rotation():
    rng = np.random.default_rng(0)
    x, w = rng.normal(size=(9, 3)), rng.normal(size=(3, 4))
    y = P.short_conv(x, w)
    assert np.allclose(y[0], x[0] * w[:, 3]) and np.allclose(y[5], sum(x[5 - 3 + j] * w[:, j] for j in range(4)))
    # a cut anywhere gives the same rows when the tail of the first part is carried
    assert np.allclose(P.short_conv(np.concatenate([x[2:5], x[5:]]), w)[3:], P.short_conv(x[2:], w)[3:])
    rot = {"base": 100.0, "dims": 4}
    q = rng.normal(size=(6, 2, 6))
    r = P.rotate(q, np.arange(6), rot)
    assert np.allclose(r[..., 4:], q[..., 4:]) and np.allclose(r[0], q[0])
    assert np.allclose(np.sum(r * r, axis=-1), np.sum(q * q, axis=-1))
    f, mag = P.rotation_frequencies({"base": 100.0, "dims": 8, "scaling": M.YARN})
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0) and f[0] == pytest.approx(1.0) and f[-1] < 100.0 ** (-6 / 8) / 3.9


def test_plain_recurrences_in_closed_form():
    """The gated delta rule with beta = 1, no decay and orthonormal keys stores every value exactly: every
    token then reads its own value back."""
    d = 4
    w = {"m.q": np.eye(d), "m.k": np.eye(d), "m.v": np.eye(d), "m.g": np.ones((d, d)), "m.o": np.eye(d),
         "m.q.conv": np.tile([0.0, 1.0], (d, 1)), "m.k.conv": np.tile([0.0, 1.0], (d, 1)), "m.v.conv": np.tile([0.0, 1.0], (d, 1)),
         "m.b": np.full((1, d), 50.0), "m.a": np.zeros((1, d)), "m.A_log": np.array([-40.0]), "m.dt_bias": np.zeros(1),
         "m.norm": np.ones(d)}
    h = np.eye(d) * 30.0                      # silu(30) = 30: token t is the unit vector t
    out = P.gated_delta(h, w, "m.", {"heads": 1, "kv_heads": 1, "dim": d, "vdim": d, "conv": 2}, 1e-12)
    assert out.shape == (d, d) and np.all(np.argmax(np.abs(out), axis=1) == np.arange(d))
