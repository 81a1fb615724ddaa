"""Vipotar on the host: its typed configuration, the model it becomes (tensors, schedule, cache needs), and the
plain implementation's mechanisms one by one against closed forms."""
import copy
import math

import numpy as np
import pytest

from imparo_b200.config import ConfigError, load_config
from imparo_b200.parts.spec import PagedKV, SlotState
from imparo_b200.weights.random_init import model_on_cpu
from tests.plain import vipotar_plain as P
from tests.vipotar_configs import ALL, VIP_A, VIP_B, VIP_C


def test_config_is_typed_and_names_the_failing_key():
    arch, cfg = load_config(VIP_A)
    assert arch.name == "Vipotar" and cfg.width == 64 and cfg.loop_times == 3 and cfg.layers[0].left.window == 9
    assert cfg.layers[0].left.rot_scaling.factor == 4.0 and cfg.logit_softcap == 15.0
    _, c = load_config(VIP_C)
    assert not c.has_loop and c.layers[0].left.window is None and c.layers[0].left.rot_dims == 0
    bad = copy.deepcopy(VIP_A)
    del bad["layers"][0]["mixer"]["left"]["scale"]
    with pytest.raises(ConfigError, match="scale"):
        load_config(bad)
    bad = copy.deepcopy(VIP_A)
    bad["layers"][1]["mixer"]["right"]["decay"] = [0.5]
    with pytest.raises(ConfigError, match="decay"):
        load_config(bad)
    bad = copy.deepcopy(VIP_A)
    bad["loop"]["stop"] = 7
    with pytest.raises(ConfigError, match="loop"):
        load_config(bad)
    bad = copy.deepcopy(VIP_A)
    bad["layers"][0]["type"] = "serial"
    with pytest.raises(ConfigError, match="type"):
        load_config(bad)


@pytest.mark.parametrize("name", sorted(ALL))
def test_model_tensors_schedule_and_cache_needs(name):
    cfg = ALL[name]
    _, typed, model = model_on_cpu(cfg)
    names = {w.name: w for w in model.weight_specs()}
    runs = P.layer_runs(cfg)
    assert [e.layer for e in model.schedule] == [i for i, _, _ in runs]
    # a stream operation stands before the first layer of every pass, and nowhere else
    assert [e.before is not None for e in model.schedule] == [first for _, _, first in runs]
    assert ("loop.step" in names) == bool(cfg.get("loop"))
    for i, L in enumerate(cfg["layers"]):
        l, r = L["mixer"]["left"], L["mixer"]["right"]
        assert names[f"l{i}.mix.left.q"].shapes[0] == (l["heads"] * l["dim"], cfg["width"])
        assert names[f"l{i}.mix.left.v"].shapes[0] == (l["kv_heads"] * l["vdim"], cfg["width"])
        assert names[f"l{i}.mix.left.o"].shapes[0] == (cfg["width"], l["heads"] * l["vdim"])
        assert names[f"l{i}.mix.right.g"].shapes[0] == (r["heads"] * r["vdim"], cfg["width"])
        assert names[f"l{i}.mix.right.norm"].shapes[0] == (r["heads"] * r["vdim"],)
        assert (f"l{i}.mlp.up" in names) == (L["mlp"] is not None)
    # every run of a layer owns a paged cache and a state
    needs = model.cache_requirements()
    assert len(needs) == len(runs)
    for (entry, specs), (i, _, _) in zip(needs, runs):
        l, r = cfg["layers"][i]["mixer"]["left"], cfg["layers"][i]["mixer"]["right"]
        kv, st = specs
        assert isinstance(kv, PagedKV) and kv.window == (l.get("mask") or {}).get("size") and kv.v_width == l["kv_heads"] * l["vdim"]
        assert isinstance(st, SlotState) and st.shape == (r["heads"], r["dim"], r["vdim"])


def test_scaled_frequencies_plain_against_the_part():
    from imparo_b200.parts.position import RotaryInterleaved
    for rot in (VIP_A["layers"][0]["mixer"]["left"]["rot"], VIP_C["layers"][1]["mixer"]["left"]["rot"],
                {"dims": 6, "base": 50.0}, {"dims": 64, "base": 1e6, "scaling": {"factor": 16.0, "original": 4096, "fast": 32.0, "slow": 1.0}}):
        f, mag = P.rotation_table(rot)
        g, mag2 = RotaryInterleaved.table(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        assert np.allclose(f, g.numpy(), rtol=1e-12) and abs(mag - mag2) < 1e-12
        if rot.get("scaling"):
            plain = np.array([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)])
            assert np.all(f <= plain * (1 + 1e-12)) and np.all(f >= plain / rot["scaling"]["factor"] * (1 - 1e-12))
            assert mag == pytest.approx(0.1 * math.log(rot["scaling"]["factor"]) + 1.0)


def test_rotation_turns_pairs_and_leaves_the_rest():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 2, 10))
    f, _ = P.rotation_table({"dims": 6, "base": 100.0})
    y = P.rotate_interleaved(x, np.arange(5), f, 1.0)
    assert np.array_equal(y[..., 6:], x[..., 6:]) and np.array_equal(y[0], x[0])          # position 0: no turn
    assert np.allclose((y[..., :6] ** 2).sum(-1), (x[..., :6] ** 2).sum(-1))
    # relative: the product of a rotated query and key depends on the distance only
    q, k = rng.standard_normal((1, 1, 6)), rng.standard_normal((1, 1, 6))
    d = lambda a, b: float((P.rotate_interleaved(q, np.array([a]), f, 1.0) * P.rotate_interleaved(k, np.array([b]), f, 1.0)).sum())
    assert d(7, 3) == pytest.approx(d(104, 100))


def test_window_and_sink_of_the_plain_attention():
    """One key is made to stand out; it counts while it is inside the window and not one position later; with all
    scores far below zero the sink takes the weight and the output goes to zero."""
    rng = np.random.default_rng(1)
    W, T, size = 8, 12, 4
    cfg = {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 1.0, "mask": {"size": size}}
    w = {"q": np.eye(8), "k": np.eye(8), "v": np.eye(8), "o": np.eye(8)}
    h = rng.standard_normal((T, W)) * 0.01
    h[3] = 0.0
    h[3, 0] = 30.0                                           # the key (and value) that stands out
    for t in range(4, T):
        h[t, 0] = 1.0                                        # later queries look for it
    out = P.window_attention(h, w, "", cfg, np.float64)
    inside, outside = 3 + size - 1, 3 + size
    assert out[inside, 0] > 25.0 and abs(out[outside, 0]) < 2.0
    wq = dict(w, q=-100.0 * np.eye(8))
    cold = np.abs(rng.standard_normal((T, W))) + 1.0         # every score is far below zero; values are of size 1
    assert np.abs(P.window_attention(cold, wq, "", cfg, np.float64)).max() < 1e-6
    # and with all scores zero, n keys share the weight with the sink: each gets 1 / (n + 1)
    flat = P.window_attention(np.ones((3, W)), dict(w, q=np.zeros((8, 8))), "", cfg, np.float64)
    assert np.allclose(flat[:, 0], [1 / 2, 2 / 3, 3 / 4])


def test_recurrence_against_the_sum_it_unrolls_to():
    rng = np.random.default_rng(2)
    T, H, D, Dv, W = 9, 2, 3, 4, 6
    cfg = {"heads": H, "dim": D, "vdim": Dv, "decay": [0.5, 0.9]}
    w = {k: rng.standard_normal(s) for k, s in (("q", (H * D, W)), ("k", (H * D, W)), ("v", (H * Dv, W)), ("g", (H * Dv, W)),
                                                 ("o", (W, H * Dv)), ("norm", (H * Dv,)))}
    h = rng.standard_normal((T, W))
    got, S = P.decayed_linear_attention(h, w, "", cfg, 1e-6, np.float64)
    q, k, v = (P.silu(h @ w[n].T) for n in "qkv")
    o = np.zeros((T, H * Dv))
    for t in range(T):
        for hh in range(H):
            for j in range(t + 1):
                o[t, hh * Dv:(hh + 1) * Dv] += cfg["decay"][hh] ** (t - j) * (q[t, hh * D:(hh + 1) * D] @ k[j, hh * D:(hh + 1) * D]) \
                    * v[j, hh * Dv:(hh + 1) * Dv]
    want = (P.rms_norm(o, w["norm"], 1e-6) * P.sigmoid(h @ w["g"].T)) @ w["o"].T
    assert np.allclose(got, want)
    # carried state: the second half from the first half's state equals the whole
    a, Sa = P.decayed_linear_attention(h[:4], w, "", cfg, 1e-6, np.float64)
    b, Sb = P.decayed_linear_attention(h[4:], w, "", cfg, 1e-6, np.float64, state=Sa)
    assert np.allclose(np.concatenate([a, b]), got) and np.allclose(Sb, S)


def test_layer_runs_of_the_plain_model():
    assert P.layer_runs(VIP_B) == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (3, None, False)]
    assert P.layer_runs(VIP_C) == [(0, None, False), (1, None, False)]
    assert P.relu_squared(np.array([-2.0, 3.0])).tolist() == [0.0, 9.0]
    assert P.gelu_tanh(np.array([0.0]))[0] == 0.0 and P.gelu_tanh(np.array([10.0]))[0] == pytest.approx(10.0)
    assert P.soft_cap(np.array([1e9]), 30.0)[0] == pytest.approx(30.0)
