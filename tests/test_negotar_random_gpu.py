"""Negotar configurations drawn from a seeded generator — widths, the order and number of attention and state-space
layers, head counts and sizes (also 64 and 128, which the tensor-core kernels take, next to sizes they decline), value
sizes equal to the key size or not, rotation over part of a head, all of it or none, with or without rescaled
frequencies, caps, shared values on some layers, state sizes, groups, taps and norm stretches, experts and how many a
token uses, layers without feed-forward, a logit scale, page sizes, ways of cutting — each replayed as a mixed trace in
32-bit (every position) and bfloat16 (positions away from a router's near tie) against the plain implementation."""
import os
import tempfile

import numpy as np
import pytest

from tests import traces
from tests.plain import negotar_plain as P
from tests.plain.lfm2_plain import read_safetensors

pytestmark = pytest.mark.gpu
_tmp = tempfile.TemporaryDirectory(prefix="imparo_b200_negotar_random_")


def draw_config(seed, fast=False):
    """fast: heads of 64 or 128 with values of the same size and at most 8 query heads per kv head, widths and expert
    sizes in multiples of 8 (what the tensor-core attention and the tensor-memory experts take)."""
    rng = np.random.default_rng(2000 + seed + (5000 if fast else 0))
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    width = pick([64, 128, 192, 256]) if fast else pick([44, 48, 64, 96, 100, 120, 128, 160])
    n_layers = int(rng.integers(2, 6))
    shared = None                 # (kv_heads, vdim) of the layers that share values: they must agree

    def attention():
        nonlocal shared
        heads = pick([1, 2, 3, 4, 6, 8, 12])
        kv = pick([k for k in (1, 2, 3, 4, 6, 8, 12) if heads % k == 0])
        dim = pick([8, 12, 16, 24, 32, 48, 64, 80, 96, 128])
        vdim = dim if rng.random() < 0.4 else pick([8, 12, 16, 24, 40, 64, 96, 128])
        if fast:
            heads = pick([1, 2, 4, 8])
            kv = pick([k for k in (1, 2, 4, 8) if heads % k == 0])
            dim = vdim = pick([64, 128])
        v_mix = rng.random() < 0.6
        if v_mix:
            if shared is None:
                shared = (kv, vdim)
            else:
                kv, vdim = shared
                heads = kv * pick([1, 2, 4])
                if fast:
                    dim = vdim
        d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": float(rng.uniform(0.05, 0.5))}
        if v_mix:
            d["v_mix"] = True
        if rng.random() < 0.7:
            d["softcap"] = float(pick([2.0, 8.0, 25.0, 60.0]))
        if rng.random() < 0.85:
            rot = {"dims": 2 * int(rng.integers(1, dim // 2 + 1)), "base": float(pick([50.0, 10000.0, 500000.0]))}
            if rng.random() < 0.6:
                low = float(pick([0.5, 1.0, 2.0]))
                rot["scaling"] = {"factor": float(pick([2.0, 4.0, 16.0])), "original": pick([16, 64, 1024]), "low": low,
                                  "high": low * float(pick([2.0, 4.0, 8.0]))}
            d["rot"] = rot
        return {"type": "attention", "mixer": d}

    def state_space():
        heads = pick([1, 2, 3, 4, 6, 8])
        groups = pick([g for g in (1, 2, 3, 4, 6, 8) if heads % g == 0])
        vdim = pick([8, 16, 20, 32, 48, 64]) if not fast else pick([32, 64])
        inner = heads * vdim
        return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": pick([4, 8, 16, 24, 32, 64, 100, 128]),
                                            "groups": groups, "conv": int(rng.integers(1, 6)),
                                            "norm_groups": pick([g for g in (1, 2, 3, 4, heads) if inner % g == 0])}}

    def layer():
        L = attention() if rng.random() < 0.55 else state_space()
        if rng.random() < 0.2:
            L["mlp"] = None
        else:
            experts = int(pick([1, 2, 3, 5, 8, 12, 33]))
            L["mlp"] = {"kind": "moe", "router": {"experts": experts, "top": int(rng.integers(1, min(experts, 4) + 1))},
                        "expert": {"ff": int(pick([16, 40, 64, 72, 128])) if fast else int(pick([10, 16, 30, 64, 100]))}}
        return L
    cfg = {"architecture": "Negotar", "vocab": int(rng.integers(100, 700)), "width": width,
           "norm": {"eps": float(pick([1e-6, 1e-5, 3e-6]))}, "layers": [layer() for _ in range(n_layers)]}
    if rng.random() < 0.6:
        cfg["logit_scale"] = float(pick([0.25, 1.5, 3.0]))
    return cfg, rng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(14)) + [f"fast{i}" for i in range(8)])
def test_drawn_configuration_mixed_trace(seed, dtype):
    from imparo_b200.engine import Engine
    from imparo_b200.weights import write_random_model
    from tests.gpu_helpers import run_trace
    from tests.test_negotar_gpu import CLOSE, TOL, WORST, all_errors, rescale
    fast = isinstance(seed, str)
    seed = int(seed[4:]) if fast else seed
    cfg, rng = draw_config(seed, fast)
    folder = os.path.join(_tmp.name, f"m{seed}{'f' if fast else ''}")
    if not os.path.isdir(folder):
        write_random_model(folder, cfg, seed=seed, dtype="bfloat16", norm_jitter=0.3)
        rescale(os.path.join(folder, "model.safetensors"))
    w = read_safetensors(os.path.join(folder, "model.safetensors"))
    lengths = [int(x) for x in rng.integers(3, 200, 3)] + ([int(rng.integers(300, 520))] if fast else [int(rng.integers(3, 200))]) + [1]
    reqs = {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(lengths)}
    steps = traces.mixed(reqs, seed=seed, max_portion=int(rng.choice([3, 17, 70, 200])))
    page = int(rng.choice([4, 8, 16, 16, 32, 64]))
    max_tokens = traces.max_live_tokens(steps, max(64, page))
    eng = Engine(folder, dtype=dtype, ctx=max_tokens, parallel=4, page_size=page, num_pages=(max_tokens + page - 1) // page,
                 max_step_tokens=max(256, max_tokens))
    ref, tie = {}, {}
    for k, t in reqs.items():
        gaps = []
        ref[k] = P.forward(cfg, w, t, gaps=gaps)
        near = np.min(np.stack(gaps), axis=0) < CLOSE if gaps else np.zeros(len(t), dtype=bool)
        tie[k] = near.copy()
        tie[k][1:] |= near[:-1]
    want = traces.expected(steps, ref)
    got = run_trace(eng, steps)
    scale = max(float(np.abs(v).max()) for v in ref.values())
    errs = all_errors(steps, got, want)
    if dtype == "bfloat16":
        errs = [e for e in errs if not tie[e[1]][e[2]]]
        if len(errs) < 20:
            pytest.skip("too few positions away from a router's near tie")
    worst = max(errs, key=lambda e: e[3])
    if dtype == "float32":
        assert worst[3] <= WORST[dtype] * scale, (cfg, page, worst, scale)
    else:
        # drawn models of a few dozen columns amplify 8-bit rounding through their output norms and carry one token's
        # deviation on through the state: the middle of the distribution is what bfloat16 is held to here (the 32-bit run
        # of the same configuration holds every position, the kernel tests hold each bfloat16 kernel to 2e-2)
        assert float(np.median([e[3] for e in errs])) <= 2 * TOL[dtype] * scale, (cfg, page, worst, scale)
        assert sum(e[3] > 2 * TOL[dtype] * scale for e in errs) <= 0.4 * len(errs), (cfg, page, worst, scale)
    assert eng.cache.n_requests() == 0
