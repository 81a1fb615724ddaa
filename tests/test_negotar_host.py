"""Negotar on the host: its typed configuration, the model it becomes (tensors, schedule, cache needs), and the
plain implementation's mechanisms one by one against closed forms."""
import copy
import math

import numpy as np
import pytest

from imparo_b200.config import ConfigError, load_config
from imparo_b200.parts.spec import PagedKV, SlotState
from imparo_b200.weights.random_init import model_on_cpu
from tests.negotar_configs import ALL, NEG_A, NEG_B, NEG_C
from tests.plain import negotar_plain as P


def test_config_is_typed_and_names_the_failing_key():
    arch, cfg = load_config(NEG_A)
    assert arch.name == "Negotar" and cfg.width == 64 and cfg.logit_scale == 1.5 and len(cfg.layers) == 4
    a = cfg.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.softcap, a.v_mix, a.rot_dims) == (4, 2, 16, 24, 5.0, True, 8)
    assert a.rot_scaling.factor == 4.0 and a.rot_scaling.original == 32
    s = cfg.layers[1].mixer
    assert (s.heads, s.vdim, s.state, s.groups, s.conv, s.norm_groups) == (4, 8, 16, 2, 4, 2)
    assert cfg.layers[0].mlp.experts == 6 and cfg.layers[0].mlp.top == 2 and cfg.layers[0].mlp.ff == 40
    _, b = load_config(NEG_B)
    assert b.logit_scale == 1.0 and b.layers[2].mlp is None and b.layers[1].mixer.softcap is None and not b.layers[1].mixer.v_mix
    _, c = load_config(NEG_C)
    assert c.layers[0].mixer.rot_dims == 0 and c.layers[0].mixer.rot_scaling is None
    for path, key in ((("layers", 0, "mixer", "scale"), "scale"), (("layers", 1, "mixer", "state"), "state"),
                      (("layers", 0, "mlp", "router", "top"), "top"), (("norm", "eps"), "eps"), (("vocab",), "vocab")):
        bad = copy.deepcopy(NEG_A)
        d = bad
        for k in path[:-1]:
            d = d[k]
        del d[path[-1]]
        with pytest.raises(ConfigError, match=key):
            load_config(bad)
    bad = copy.deepcopy(NEG_A)
    bad["layers"][0]["type"] = "serial"
    with pytest.raises(ConfigError, match="type"):
        load_config(bad)
    bad = copy.deepcopy(NEG_A)
    bad["layers"][1]["mixer"]["groups"] = 3
    with pytest.raises(ConfigError, match="groups"):
        load_config(bad)
    bad = copy.deepcopy(NEG_A)
    bad["layers"][2]["mixer"]["vdim"] = 8                     # shared values of another width
    with pytest.raises(ConfigError, match="v_mix"):
        load_config(bad)
    bad = copy.deepcopy(NEG_A)
    bad["layers"][0]["mlp"]["router"]["top"] = 7
    with pytest.raises(ConfigError, match="top"):
        load_config(bad)


@pytest.mark.parametrize("name", sorted(ALL))
def test_model_tensors_schedule_and_cache_needs(name):
    cfg = ALL[name]
    _, typed, model = model_on_cpu(cfg)
    names = {w.name: w for w in model.weight_specs()}
    W = cfg["width"]
    assert [e.layer for e in model.schedule] == list(range(len(cfg["layers"])))
    assert names["embed"].shapes[0] == (cfg["vocab"], W) and "final.norm" in names and "head" not in names
    needs = dict(model.cache_requirements())
    first_shared = True
    for i, L in enumerate(cfg["layers"]):
        m = L["mixer"]
        if L["type"] == "attention":
            assert names[f"l{i}.mix.q"].shapes[0] == (m["heads"] * m["dim"], W)
            assert names[f"l{i}.mix.k.b"].shapes[0] == (m["kv_heads"] * m["dim"],)
            assert names[f"l{i}.mix.v"].shapes[0] == (m["kv_heads"] * m["vdim"], W)
            assert names[f"l{i}.mix.o"].shapes[0] == (W, m["heads"] * m["vdim"])
            assert (f"l{i}.mix.vmix" in names) == bool(m.get("v_mix"))
            if m.get("v_mix"):
                assert names[f"l{i}.mix.vmix"].shapes[0] == ()
                role = model.layers[i].mixer.v_share["role"]
                assert role == ("source" if first_shared else "blend")
                first_shared = False
            assert needs[i] == (PagedKV(m["kv_heads"], m["dim"], None, None if m["vdim"] == m["dim"] else m["vdim"]),)
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            assert names[f"l{i}.mix.in"].shapes[0] == (2 * inner + 2 * gn + m["heads"], W)
            assert names[f"l{i}.mix.conv"].shapes[0] == (inner + 2 * gn, m["conv"])
            assert names[f"l{i}.mix.conv.b"].shapes[0] == (inner + 2 * gn,)
            assert names[f"l{i}.mix.norm"].shapes[0] == (inner,) and names[f"l{i}.mix.A_log"].shapes[0] == (m["heads"],)
            assert needs[i] == (SlotState((m["heads"], m["state"], m["vdim"])), SlotState((max(m["conv"] - 1, 1), inner + 2 * gn)))
        if L["mlp"] is None:
            assert f"l{i}.norm2" not in names and f"l{i}.mlp.router" not in names
        else:
            E, ff = L["mlp"]["router"]["experts"], L["mlp"]["expert"]["ff"]
            assert names[f"l{i}.mlp.router"].shapes[0] == (E, W) and names[f"l{i}.mlp.router"].role == "vector"
            assert names[f"l{i}.mlp.e{E - 1}.down"].shapes[0] == (W, ff) and f"l{i}.mlp.e{E}.gate" not in names
            assert f"l{i}.norm2" in names


def test_frequencies_rescaled_by_wavelength():
    rot = {"dims": 64, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}}
    plain = P.rotation_frequencies({"dims": 64, "base": 10000.0})
    f = P.rotation_frequencies(rot)
    wl = 2 * math.pi / plain
    assert (f[wl < 64] == plain[wl < 64]).all() and np.allclose(f[wl > 256], plain[wl > 256] / 8.0)
    mid = (wl >= 64) & (wl <= 256)
    assert mid.any() and ((f[mid] <= plain[mid]) & (f[mid] >= plain[mid] / 8.0)).all()
    assert (np.diff(f) < 0).all()                              # still falling from pair to pair
    # the engine's table is the same rule in vector form
    import torch
    from imparo_b200.parts.base import Runtime, Workspace
    from imparo_b200.parts.position import RotaryNeox
    rt = Runtime(precision="float32", device=torch.device("cpu"), workspace=Workspace("cpu"))
    part = RotaryNeox({"head_dim": 96, "n_rot": 64, "theta": 10000.0, "wavelength_scaling": rot["scaling"]}, "", rt)
    assert np.allclose(part.rotary()[0].numpy(), f.astype(np.float32), rtol=1e-6) and part.rotary()[1] == 64


def test_rotation_is_a_function_of_distance_and_leaves_the_rest():
    rng = np.random.default_rng(0)
    f = P.rotation_frequencies({"dims": 8, "base": 100.0})
    q, k = rng.standard_normal((1, 1, 12)), rng.standard_normal((1, 1, 12))
    dots = [float(P.rotate_half_split(q, [p + 5], f, 8)[0, 0] @ P.rotate_half_split(k, [p], f, 8)[0, 0]) for p in (0, 7, 300)]
    assert np.allclose(dots, dots[0])
    assert np.array_equal(P.rotate_half_split(q, [9], f, 8)[0, 0, 8:], q[0, 0, 8:])
    assert np.allclose(P.rotate_half_split(q, [0], f, 8), q)


def test_attention_softcap_unit_norm_and_shared_values():
    rng = np.random.default_rng(1)
    T, width = 9, 16
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 100.0, "softcap": 3.0}
    W = {"q": rng.standard_normal((8, width)), "k": rng.standard_normal((4, width)), "v": rng.standard_normal((6, width)),
         "q.b": rng.standard_normal(8), "k.b": rng.standard_normal(4), "v.b": rng.standard_normal(6),
         "o": np.eye(12), "vmix": np.float64(0.25)}
    h = rng.standard_normal((T, width))
    out, v = P.attention_mixer(h, W, "", m, 1e-6)
    assert np.allclose(v.reshape(T, 6), h @ W["v"].T + W["v.b"])
    # scores are capped at 3: the softmax weights stay within e^6 of each other, so the output stays inside the values' hull
    assert np.allclose(out[0, :6], v[0, 0]) and (out[-1, :6] <= v[:, 0].max(0) + 1e-9).all()
    lo = np.exp(-3.0) / (np.exp(-3.0) + (T - 1) * np.exp(3.0))
    q = P.unit_rms((h @ W["q"].T + W["q.b"]).reshape(T, 2, 4), 1e-6)
    k = P.unit_rms((h @ W["k"].T + W["k.b"]).reshape(T, 1, 4), 1e-6)
    s = 3.0 * np.tanh(100.0 * (k[:, 0] @ q[-1, 0]) / 3.0)
    p = np.exp(s) / np.exp(s).sum()
    assert p.min() >= lo - 1e-12 and np.allclose(out[-1, :6], p @ v[:, 0])
    # biases do matter, and so does the scale of h not (q and k are unit vectors)
    out2, _ = P.attention_mixer(h, dict(W, **{"q.b": np.zeros(8)}), "", m, 1e-6)
    assert np.abs(out2 - out).max() > 1e-3
    first = rng.standard_normal((T, 1, 6))
    out3, v3 = P.attention_mixer(h, W, "", m, 1e-6, v_first=first)
    assert np.allclose(v3, 0.75 * v + 0.25 * first)


def test_conv_and_recurrence_against_closed_forms():
    rng = np.random.default_rng(2)
    T, C = 7, 3
    u, taps, bias = rng.standard_normal((T, C)), rng.standard_normal((C, 3)), rng.standard_normal(C)
    y = P.causal_conv_silu(u, taps, bias)
    z = bias + taps[:, 2] * u[4] + taps[:, 1] * u[3] + taps[:, 0] * u[2]
    assert np.allclose(y[4], z / (1 + np.exp(-z)))
    z0 = bias + taps[:, 2] * u[0]                                  # zeros before the start
    assert np.allclose(y[0], z0 / (1 + np.exp(-z0)))
    # recurrence unrolled: y_t = sum_s exp(a sum_{r=s+1..t} dt_r) dt_s (C_t . B_s) x_s + D x_t
    heads, vdim, N = 2, 3, 4
    x, B, Cm = rng.standard_normal((T, heads, vdim)), rng.standard_normal((T, 1, N)), rng.standard_normal((T, 1, N))
    dt, A_log, D = rng.uniform(0.1, 1.0, (T, heads)), np.array([-0.5, 0.7]), np.array([0.3, 1.1])
    got = P.selective_scan(x, B, Cm, dt, A_log, D, 1)
    for h in range(heads):
        a = -math.exp(A_log[h])
        t = T - 1
        want = D[h] * x[t, h]
        for s in range(t + 1):
            want = want + math.exp(a * dt[s + 1:t + 1, h].sum()) * dt[s, h] * float(Cm[t, 0] @ B[s, 0]) * x[s, h]
        assert np.allclose(got[t, h], want)
    # heads share B and C by group: head h uses group h // (heads / groups)
    B2, C2 = rng.standard_normal((T, 2, N)), rng.standard_normal((T, 2, N))
    both = P.selective_scan(x, B2, C2, dt, A_log, D, 2)
    assert np.allclose(both[:, 1], P.selective_scan(x[:, 1:], B2[:, 1:], C2[:, 1:], dt[:, 1:], A_log[1:], D[1:], 1)[:, 0])
    g = P.grouped_unit_rms(np.arange(1.0, 9.0).reshape(1, 8), 2, 0.0)
    assert np.allclose(g[0, :4], np.arange(1.0, 5.0) / math.sqrt(np.mean(np.arange(1.0, 5.0) ** 2)))


def test_routed_experts_weight_the_input_and_do_not_renormalise():
    rng = np.random.default_rng(3)
    width, ff, E = 6, 5, 4
    W = {"router": rng.standard_normal((E, width))}
    for e in range(E):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = rng.standard_normal((ff, width)), rng.standard_normal((ff, width)), rng.standard_normal((width, ff))
    h = rng.standard_normal((3, width))
    s = 1 / (1 + np.exp(-(h @ W["router"].T)))
    out = P.routed_experts(h, W, "", {"router": {"experts": E, "top": 2}})
    for t in range(3):
        want = 0
        for e in np.argsort(-s[t])[:2]:
            u = s[t, e] * h[t]
            g = W[f"e{e}.gate"] @ u
            want = want + W[f"e{e}.down"] @ (g / (1 + np.exp(-g)) * (W[f"e{e}.up"] @ u))
        assert np.allclose(out[t], want)
    # the expert is not linear in its input, so a weight on the output would differ
    e = int(np.argmax(s[0]))
    g = W[f"e{e}.gate"] @ h[0]
    on_output = s[0, e] * (W[f"e{e}.down"] @ (g / (1 + np.exp(-g)) * (W[f"e{e}.up"] @ h[0])))
    assert np.abs(P.routed_experts(h[:1], W, "", {"router": {"experts": E, "top": 1}})[0] - on_output).max() > 1e-3


def test_layer_norms_sit_on_the_outputs():
    cfg = copy.deepcopy(NEG_B)
    _, _, model = model_on_cpu(cfg)
    rng = np.random.default_rng(4)
    W = {w.name: rng.standard_normal(w.shapes[0]) * 0.2 for w in model.weight_specs()}
    toks = [3, 7, 1, 250]
    streams = []
    logits = P.forward(cfg, W, toks, streams=streams)
    assert len(streams) == 4 and logits.shape == (4, cfg["vocab"])
    # layer 2 has no feed-forward: its update is one normed vector per token, of root mean square |1 + norm1| on average
    delta = streams[2] - streams[1]
    want = np.sqrt(np.mean((1 + W["l2.norm1"]) ** 2))
    assert np.allclose(np.sqrt(np.mean(delta ** 2, axis=1)), want, rtol=0.35)
    # the first token's logits do not depend on later tokens
    assert np.allclose(P.forward(cfg, W, toks[:1])[0], logits[0])
