"""Typed configuration of Negotar, read from its config.json keys.

A decoder-only design whose layers put their norm on each sublayer's output: x += norm(mixer(x)), then
x += norm(feed_forward(x)), both norms with a weight kept as its distance from one.  `layers` lists the layers in order; each entry
names its mixer type ("attention": grouped-query attention with biases, a half-split rotation whose frequencies may be
rescaled by wavelength, a norm without a weight on q and k after the rotation, a soft cap on the scores and values that
may be blended with those of the first such layer; "mamba2": a selective state-space mixer), the mixer's sizes, and its
feed-forward ("moe": sigmoid-routed experts that are fed the input times their score; null: none).  Every size and
constant below comes from config.json; a key that is absent switches its mechanism off (no `rot`: no rotation; no
`rot.scaling`: plain frequencies; no `softcap`: plain scores; no `v_mix`: the layer's own values; no `logit_scale`: 1).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .base import ConfigError, KeyReader

LAYER_TYPES = ("attention", "mamba2")
MLP_KINDS = ("moe",)


@dataclass(frozen=True)
class WavelengthScaling:
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    v_mix: bool
    rot_dims: int                     # 0: no rotation
    rot_base: float
    rot_scaling: Optional[WavelengthScaling]


@dataclass(frozen=True)
class Mamba2Sizes:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class ExpertSizes:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class NegotarLayer:
    type: str
    mixer: Union[AttentionSizes, Mamba2Sizes]
    mlp: Optional[ExpertSizes]        # None: the layer has no feed-forward


@dataclass(frozen=True)
class NegotarConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: Tuple[NegotarLayer, ...]


def _sub(reader: KeyReader, key: str, required: bool = True) -> Optional[KeyReader]:
    v = reader.raw(key)
    if v is None:
        if required:
            raise ConfigError(f"{reader.where}: missing required key '{key}'")
        return None
    return KeyReader(v, f"{reader.where}: {key}")


def _attention(r: KeyReader) -> AttentionSizes:
    heads, kv = r.integer("heads", minimum=1), r.integer("kv_heads", minimum=1)
    if heads % kv:
        raise ConfigError(f"{r.where}: kv_heads {kv} must divide heads {heads}")
    dim = r.integer("dim", minimum=1)
    rot = _sub(r, "rot", required=False)
    rot_dims, rot_base, scaling = 0, 10000.0, None
    if rot is not None:
        rot_dims, rot_base = rot.integer("dims", minimum=0), rot.number("base")
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"{rot.where}: dims {rot_dims} must be even and at most dim {dim}")
        sc = _sub(rot, "scaling", required=False)
        if sc is not None:
            scaling = WavelengthScaling(sc.number("factor"), sc.number("low"), sc.number("high"), sc.number("original"))
            if scaling.high == scaling.low:
                raise ConfigError(f"{sc.where}: high and low must differ")
    cap = r.number("softcap", default=None)
    return AttentionSizes(heads=heads, kv_heads=kv, dim=dim, vdim=r.integer("vdim", minimum=1), scale=r.number("scale"),
                          softcap=cap if cap else None, v_mix=bool(r.boolean("v_mix", default=False)),
                          rot_dims=rot_dims, rot_base=rot_base, rot_scaling=scaling)


def _mamba2(r: KeyReader) -> Mamba2Sizes:
    heads, groups = r.integer("heads", minimum=1), r.integer("groups", minimum=1)
    if heads % groups:
        raise ConfigError(f"{r.where}: groups {groups} must divide heads {heads}")
    vdim, norm_groups = r.integer("vdim", minimum=1), r.integer("norm_groups", default=1, minimum=1)
    if (heads * vdim) % norm_groups:
        raise ConfigError(f"{r.where}: norm_groups {norm_groups} must divide heads * vdim = {heads * vdim}")
    return Mamba2Sizes(heads=heads, vdim=vdim, state=r.integer("state", minimum=1), groups=groups,
                       conv=r.integer("conv", minimum=1), norm_groups=norm_groups)


def _mlp(r: Optional[KeyReader]) -> Optional[ExpertSizes]:
    if r is None:
        return None
    kind = r.raw("kind")
    if kind not in MLP_KINDS:
        raise ConfigError(f"{r.where}: unknown kind {kind!r}; known: {', '.join(MLP_KINDS)}")
    router, expert = _sub(r, "router"), _sub(r, "expert")
    experts, top = router.integer("experts", minimum=1), router.integer("top", minimum=1)
    if top > experts:
        raise ConfigError(f"{router.where}: top {top} exceeds experts {experts}")
    return ExpertSizes(experts=experts, top=top, ff=expert.integer("ff", minimum=1))


def parse_negotar_config(values: dict) -> NegotarConfig:
    r = KeyReader(values)
    layers_raw = r.raw("layers")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: key 'layers' must be a non-empty list")
    layers = []
    shared_width = None
    for i, entry in enumerate(layers_raw):
        lr = KeyReader(entry, f"config.json: layers[{i}]")
        kind = lr.raw("type")
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{lr.where}: unknown type {kind!r}; known: {', '.join(LAYER_TYPES)}")
        mixer = _attention(_sub(lr, "mixer")) if kind == "attention" else _mamba2(_sub(lr, "mixer"))
        if kind == "attention" and mixer.v_mix:
            w = mixer.kv_heads * mixer.vdim
            if shared_width is not None and w != shared_width:
                raise ConfigError(f"{lr.where}: layers with v_mix must have the same kv_heads * vdim (found {w} and {shared_width})")
            shared_width = w
        layers.append(NegotarLayer(type=kind, mixer=mixer, mlp=_mlp(_sub(lr, "mlp", required=False))))
    norm = _sub(r, "norm")
    return NegotarConfig(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), eps=norm.number("eps"),
                         logit_scale=r.number("logit_scale", default=1.0), layers=tuple(layers))
