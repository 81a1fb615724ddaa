"""Vipotar configurations drawn from a seeded generator — widths, head counts and sizes (also 64 and 128, which the
tensor-core kernels take, next to sizes they decline), value sizes equal to the key size or not, windows from 1 to
beyond the prompts, rotation over part of a head or all of it with or without scaled frequencies, decays, layers with
and without feed-forward and with sizes of their own, a repeated stretch anywhere, page sizes, ways of cutting — each
replayed as a mixed trace in 32-bit and bfloat16 against the plain implementation."""
import os
import tempfile

import numpy as np
import pytest

from tests import traces
from tests.plain import vipotar_plain as P
from tests.plain.lfm2_plain import read_safetensors

pytestmark = pytest.mark.gpu
_tmp = tempfile.TemporaryDirectory(prefix="imparo_b200_vipotar_random_")


def draw_config(seed, fast=False):
    """fast: heads of 64 or 128 with values of the same size and at most 8 query heads per kv head (what the tensor-core
    attention kernels take), linear attention sizes that are multiples of 16 up to 128 (the tensor-core chunks)."""
    rng = np.random.default_rng(1000 + seed + (5000 if fast else 0))
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    width = pick([48, 64, 96, 120, 128, 160, 256])
    n_layers = int(rng.integers(2, 6))

    def left():
        heads = pick([1, 2, 3, 4, 6, 8, 12, 16])
        kv = pick([k for k in (1, 2, 3, 4, 6, 8, 12, 16) if heads % k == 0])
        dim = pick([8, 16, 24, 32, 48, 64, 64, 96, 128, 128])
        vdim = dim if rng.random() < 0.5 else pick([8, 16, 24, 40, 64, 96, 128])
        if fast:
            heads = pick([1, 2, 4, 8])
            kv = pick([k for k in (1, 2, 4, 8) if heads % k == 0])
            dim = vdim = pick([64, 128])
        d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": float(rng.uniform(0.05, 0.4))}
        if rng.random() < 0.85:
            d["mask"] = {"size": pick([1, 2, 5, 17, 33, 64, 72, 130, 300])}
        if rng.random() < 0.85:
            rot = {"dims": 2 * int(rng.integers(1, dim // 2 + 1)), "base": float(pick([50.0, 10000.0, 500000.0]))}
            if rng.random() < 0.5:
                rot["scaling"] = {"factor": float(pick([2.0, 4.0, 8.0, 32.0])), "original": pick([16, 64, 1024]),
                                  "fast": float(pick([4.0, 32.0])), "slow": float(pick([0.5, 1.0, 2.0]))}
            d["rot"] = rot
        return d

    def right():
        heads = pick([1, 2, 3, 4, 8])
        if fast:
            return {"heads": heads, "dim": pick([16, 32, 64, 128]), "vdim": pick([16, 32, 64, 96, 128]),
                    "decay": [float(x) for x in 1.0 - rng.uniform(0.0, 0.7, heads) ** 2]}
        return {"heads": heads, "dim": pick([4, 8, 16, 32, 64, 128]), "vdim": pick([8, 16, 32, 64, 72, 128, 160]),
                "decay": [float(x) for x in 1.0 - rng.uniform(0.0, 0.7, heads) ** 2]}

    def layer():
        ff = None if rng.random() < 0.2 else int(pick([32, 100, 256, 384]))
        return {"type": "parallel", "mixer": {"left": left(), "right": right()}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    same = rng.random() < 0.5
    first = layer()
    cfg = {"architecture": "Vipotar", "vocab": int(rng.integers(100, 700)), "width": width,
           "norm": {"eps": float(pick([1e-6, 1e-5, 3e-6]))}, "residual_mult": float(pick([1.0, 0.3, 0.5, 0.8])),
           "layers": [first if same else layer() for _ in range(n_layers)]}
    if rng.random() < 0.6:
        cfg["logit_softcap"] = float(pick([8.0, 30.0, 50.0]))
    if rng.random() < 0.7:
        start = int(rng.integers(0, n_layers))
        stop = int(rng.integers(start + 1, n_layers + 1))
        cfg["loop"] = {"start": start, "stop": stop, "times": int(rng.integers(1, 4))}
    return cfg, rng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(12)) + [f"fast{i}" for i in range(8)])
def test_drawn_configuration_mixed_trace(seed, dtype):
    from imparo_b200.engine import Engine
    from imparo_b200.weights import write_random_model
    from tests.gpu_helpers import run_trace
    from tests.test_vipotar_gpu import TOL, WORST, all_errors
    fast = isinstance(seed, str)
    seed = int(seed[4:]) if fast else seed
    cfg, rng = draw_config(seed, fast)
    folder = os.path.join(_tmp.name, f"m{seed}{'f' if fast else ''}")
    if not os.path.isdir(folder):
        write_random_model(folder, cfg, seed=seed, dtype="bfloat16", matrix_std=1.0 / np.sqrt(cfg["width"]), norm_jitter=0.3)
    w = read_safetensors(os.path.join(folder, "model.safetensors"))
    lengths = [int(x) for x in rng.integers(3, 260, 3)] + ([int(rng.integers(300, 520))] if fast else [int(rng.integers(3, 260))]) + [1]
    reqs = {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(lengths)}
    steps = traces.mixed(reqs, seed=seed, max_portion=int(rng.choice([3, 17, 70, 200])))
    page = int(rng.choice([4, 8, 16, 16, 32, 64]))
    max_tokens = traces.max_live_tokens(steps, max(64, page))
    eng = Engine(folder, dtype=dtype, ctx=max_tokens, parallel=4, page_size=page, num_pages=(max_tokens + page - 1) // page,
                 max_step_tokens=max(256, max_tokens))
    ref = {k: P.forward(cfg, w, t) for k, t in reqs.items()}
    want = traces.expected(steps, ref)
    got = run_trace(eng, steps)
    scale = max(float(np.abs(v).max()) for v in ref.values())
    errs = all_errors(steps, got, want)
    worst = max(errs, key=lambda e: e[3])
    assert worst[3] <= WORST[dtype] * scale, (cfg, page, worst, scale)
    assert sum(e[3] > TOL[dtype] * scale for e in errs) <= 0.1 * len(errs), (cfg, page, worst, scale)
    assert eng.cache.n_requests() == 0
