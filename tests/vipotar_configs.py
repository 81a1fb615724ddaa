"""Tiny Vipotar configurations for tests.  They differ in every size and option: heads and groups, key and value
sizes (equal or not, multiples of 16 or not), rotated dimensions (part of a head, all of it, none), scaled or plain
frequencies, window (small, larger than the prompts, none), decays, a layer without feed-forward, a repeated
stretch (at the start, in the middle, none, a single pass), soft cap or none, residual factor (also 1), widths and
vocabularies that are no power of two."""


def _left(heads, kv, dim, vdim, scale, window=None, rot=None):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        d["mask"] = {"size": window}
    if rot is not None:
        d["rot"] = rot
    return d


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _layer(left, right, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


_ROT_SCALED = {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}

VIP_A = {
    "architecture": "Vipotar", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.5, "logit_softcap": 15.0,
    "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [_layer(_left(4, 2, 16, 24, 0.3, window=9, rot=_ROT_SCALED), _right(2, 8, 16, (0.9, 0.99)), 96)] * 3,
}

VIP_B = {
    "architecture": "Vipotar", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _layer(_left(3, 3, 32, 32, 0.2, window=33, rot={"dims": 32, "base": 500.0}), _right(3, 16, 40, (0.5, 0.95, 1.0)), 128),
        _layer(_left(3, 3, 32, 32, 0.2, window=33, rot={"dims": 32, "base": 500.0}), _right(3, 16, 40, (0.5, 0.95, 1.0)), 128),
        _layer(_left(3, 3, 32, 32, 0.2, window=33, rot={"dims": 32, "base": 500.0}), _right(3, 16, 40, (0.5, 0.95, 1.0)), None),
        _layer(_left(3, 1, 32, 16, 0.25, window=2, rot={"dims": 2, "base": 7.0}), _right(1, 48, 8, (0.97,)), 40),
    ],
}

VIP_C = {
    "architecture": "Vipotar", "vocab": 257, "width": 72, "norm": {"eps": 3e-6}, "residual_mult": 0.3, "logit_softcap": 8.0,
    "layers": [
        _layer(_left(6, 1, 24, 8, 0.4), _right(1, 40, 72, (0.999,)), 100),
        _layer(_left(6, 2, 24, 8, 0.4, window=5, rot={"dims": 12, "base": 100.0,
                                                     "scaling": {"factor": 8.0, "original": 16, "fast": 4.0, "slow": 0.5}}),
               _right(4, 4, 12, (0.3, 0.6, 0.9, 0.99)), 100),
    ],
}

# a width that is no multiple of 8 (no 16-byte rows), as many kv heads as heads, a single pass of a repeated stretch
VIP_D = {
    "architecture": "Vipotar", "vocab": 199, "width": 100, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
    "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [_layer(_left(5, 5, 20, 12, 0.22, window=17, rot={"dims": 20, "base": 10000.0}), _right(2, 20, 50, (0.8, 0.9)), 150)] * 2,
}

# sizes the tensor-core kernels take: heads of 64 with values of 64 (two query heads per kv head), a linear attention
# of 64 x 64; and heads of 128 with one kv head for eight heads, 128 x 128
VIP_E = {
    "architecture": "Vipotar", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.4, "logit_softcap": 20.0,
    "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [_layer(_left(4, 2, 64, 64, 0.125, window=40, rot={"dims": 32, "base": 10000.0,
                                                               "scaling": {"factor": 2.0, "original": 64, "fast": 16.0, "slow": 1.0}}),
                      _right(2, 64, 64, (0.9, 0.995)), 256)] * 2,
}

VIP_F = {
    "architecture": "Vipotar", "vocab": 270, "width": 256, "norm": {"eps": 2e-6}, "residual_mult": 0.3,
    "layers": [_layer(_left(8, 1, 128, 128, 0.09, window=70, rot={"dims": 64, "base": 500000.0}),
                      _right(2, 128, 128, (0.98, 0.999)), 384)] * 2,
}

# windows wider than a query tile of the tensor-core kernels (128 rows), not multiples of a page or a tile
VIP_G = {
    "architecture": "Vipotar", "vocab": 280, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
    "layers": [_layer(_left(4, 1, 64, 64, 0.125, window=130, rot={"dims": 64, "base": 10000.0}), _right(2, 32, 64, (0.9, 0.99)), 192),
               _layer(_left(4, 4, 64, 64, 0.125, window=72, rot={"dims": 16, "base": 10000.0}), _right(1, 64, 128, (0.999,)), 192)],
}

VIP_H = {
    "architecture": "Vipotar", "vocab": 290, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.6, "logit_softcap": 25.0,
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [_layer(_left(4, 1, 128, 128, 0.09, window=257, rot={"dims": 32, "base": 500000.0,
                                                                "scaling": {"factor": 2.0, "original": 128, "fast": 32.0, "slow": 1.0}}),
                      _right(2, 64, 64, (0.95, 0.999)), 160),
               _layer(_left(8, 2, 128, 128, 0.09, rot={"dims": 128, "base": 1000.0}), _right(4, 16, 32, (0.5, 0.9, 0.99, 0.999)), None)],
}

ALL = {"A": VIP_A, "B": VIP_B, "C": VIP_C, "D": VIP_D, "E": VIP_E, "F": VIP_F, "G": VIP_G, "H": VIP_H}
PAGE = {"A": 4, "B": 8, "C": 16, "D": 32, "E": 16, "F": 64, "G": 32, "H": 16}
