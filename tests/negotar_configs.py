"""Tiny Negotar configurations for tests.  They differ in every size and option: the order of layer types, heads and
groups, key and value sizes (equal or not, multiples of 16 or not), rotated dimensions (part of a head, all of it, none),
scaled or plain frequencies, soft cap or none, shared values on all, some or no attention layers, experts and how many
of them a token uses (one, some, all), a layer without feed-forward, state sizes and taps of the state-space mixer,
groups equal to heads or 1, norm stretches, a logit scale or none, widths and vocabularies that are no power of two."""


def _attn(heads, kv, dim, vdim, scale, rot=None, softcap=None, v_mix=None):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        d["rot"] = rot
    if softcap is not None:
        d["softcap"] = softcap
    if v_mix is not None:
        d["v_mix"] = v_mix
    return {"type": "attention", "mixer": d}


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def _with(layer, experts=None, top=None, ff=None):
    layer = dict(layer)
    layer["mlp"] = None if experts is None else {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    return layer


_SCALED = {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}

NEG_A = {
    "architecture": "Negotar", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 1.5,
    "layers": [
        _with(_attn(4, 2, 16, 24, 0.3, rot=_SCALED, softcap=5.0, v_mix=True), 6, 2, 40),
        _with(_ssm(4, 8, 16, 2, 4, 2), 6, 2, 40),
        _with(_attn(4, 2, 16, 24, 0.3, rot=_SCALED, softcap=5.0, v_mix=True), 6, 2, 40),
        _with(_attn(4, 2, 16, 24, 0.3, rot=_SCALED, softcap=5.0, v_mix=True), 6, 2, 40),
    ],
}

# the state-space mixer first, groups == heads, one norm stretch, two taps; attention without shared values or cap,
# the whole head rotated with plain frequencies; a layer without feed-forward; no logit scale
NEG_B = {
    "architecture": "Negotar", "vocab": 300, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        _with(_ssm(3, 32, 8, 3, 2, 1), 5, 2, 64),
        _with(_attn(3, 3, 32, 32, 0.2, rot={"dims": 32, "base": 500.0}), 5, 2, 64),
        _with(_ssm(3, 32, 8, 3, 2, 1)),
        _with(_attn(6, 1, 16, 48, 0.25, rot={"dims": 2, "base": 7.0}, softcap=50.0), 4, 3, 24),
    ],
}

# a width that is no multiple of 8; sizes that are no multiples of 16 or 32; no rotation; every expert used by every
# token; shared values on the second and fourth layer only (the first attention layer has none); five taps, one group; one expert
# per token in the last layer
NEG_C = {
    "architecture": "Negotar", "vocab": 257, "width": 100, "norm": {"eps": 3e-6}, "logit_scale": 0.5,
    "layers": [
        _with(_attn(5, 5, 20, 12, 0.22, softcap=8.0), 3, 3, 30),
        _with(_attn(5, 5, 20, 12, 0.22, rot={"dims": 12, "base": 100.0, "scaling": {"factor": 8.0, "low": 0.5, "high": 4.0, "original": 16}},
                    v_mix=True), 3, 3, 30),
        _with(_ssm(5, 12, 20, 1, 5, 5), 7, 2, 50),
        _with(_attn(10, 5, 24, 12, 0.4, v_mix=True), 3, 1, 30),
    ],
}

# sizes the tensor-core kernels take: heads of 64 with a cap, state 64, value columns 64, features in multiples of 64
NEG_D = {
    "architecture": "Negotar", "vocab": 512, "width": 128, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
    "layers": [
        _with(_attn(4, 2, 64, 64, 0.1, rot={"dims": 64, "base": 10000.0}, softcap=20.0, v_mix=True), 8, 2, 64),
        _with(_ssm(4, 64, 64, 2, 4, 4), 8, 2, 64),
        _with(_attn(4, 2, 64, 64, 0.1, rot={"dims": 64, "base": 10000.0}, softcap=20.0, v_mix=True), 8, 2, 64),
    ],
}

# heads of 128 without a cap, eight query heads per key head, partial rotation, state 128
NEG_E = {
    "architecture": "Negotar", "vocab": 400, "width": 256, "norm": {"eps": 1e-5},
    "layers": [
        _with(_ssm(2, 64, 128, 1, 3, 2), 4, 2, 128),
        _with(_attn(8, 1, 128, 128, 0.09, rot={"dims": 64, "base": 1000.0}, v_mix=True), 4, 2, 128),
        _with(_attn(8, 1, 128, 128, 0.09, rot={"dims": 64, "base": 1000.0}, v_mix=True), 4, 2, 128),
    ],
}

ALL = {"A": NEG_A, "B": NEG_B, "C": NEG_C, "D": NEG_D, "E": NEG_E}
PAGE = {"A": 16, "B": 8, "C": 4, "D": 16, "E": 16}
