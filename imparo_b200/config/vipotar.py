"""Typed configuration of Vipotar, read from its config.json keys.

A decoder-only design: every layer has one RMS norm whose output feeds a mixer and (optionally) a dense
feed-forward, both added into the stream times `residual_mult`.  The mixer of layer type "parallel" is two
mixers side by side: "left", a windowed grouped-query attention with a partial interleaved rotation (optionally
with scaled frequencies) and a softmax whose denominator counts one extra term; "right", a linear attention
with a per-head decay.  A stretch of layers (`loop`: start, stop, times) may run several times in a row with the
same weights.  Every size and constant below comes from config.json; a key that is absent switches its
mechanism off (no `loop`: every layer once; no `mask`: all earlier positions; no `rot`: no rotation; no
`rot.scaling`: plain frequencies; no `logit_softcap`: plain logits; `mlp` null: no feed-forward).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, KeyReader

LAYER_TYPES = ("parallel",)
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class RotationScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LeftMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot_dims: int                     # 0: no rotation
    rot_base: float
    rot_scaling: Optional[RotationScaling]


@dataclass(frozen=True)
class RightMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class VipotarLayer:
    type: str
    left: LeftMixer
    right: RightMixer
    ff: Optional[int]                 # None: the layer has no feed-forward


@dataclass(frozen=True)
class VipotarConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_softcap: Optional[float]
    layers: Tuple[VipotarLayer, ...]
    loop_start: int
    loop_stop: int
    loop_times: int                   # 0: no repeated stretch

    @property
    def has_loop(self) -> bool:
        return self.loop_times > 0


def _sub(reader: KeyReader, key: str, required: bool = True) -> Optional[KeyReader]:
    v = reader.raw(key)
    if v is None:
        if required:
            raise ConfigError(f"{reader.where}: missing required key '{key}'")
        return None
    return KeyReader(v, f"{reader.where}: {key}")


def _left(r: KeyReader) -> LeftMixer:
    heads, kv = r.integer("heads", minimum=1), r.integer("kv_heads", minimum=1)
    if heads % kv:
        raise ConfigError(f"{r.where}: kv_heads {kv} must divide heads {heads}")
    dim = r.integer("dim", minimum=1)
    mask = _sub(r, "mask", required=False)
    rot = _sub(r, "rot", required=False)
    rot_dims, rot_base, scaling = 0, 10000.0, None
    if rot is not None:
        rot_dims, rot_base = rot.integer("dims", minimum=0), rot.number("base")
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"{rot.where}: dims {rot_dims} must be even and at most dim {dim}")
        sc = _sub(rot, "scaling", required=False)
        if sc is not None:
            scaling = RotationScaling(sc.number("factor"), sc.number("original"), sc.number("fast"), sc.number("slow"))
    return LeftMixer(heads=heads, kv_heads=kv, dim=dim, vdim=r.integer("vdim", minimum=1), scale=r.number("scale"),
                     window=mask.integer("size", minimum=1) if mask is not None else None,
                     rot_dims=rot_dims, rot_base=rot_base, rot_scaling=scaling)


def _right(r: KeyReader) -> RightMixer:
    heads = r.integer("heads", minimum=1)
    decay = r.raw("decay")
    if not isinstance(decay, (list, tuple)) or len(decay) != heads or not all(isinstance(d, (int, float)) for d in decay):
        raise ConfigError(f"{r.where}: decay must be a list of {heads} numbers (one per head)")
    return RightMixer(heads=heads, dim=r.integer("dim", minimum=1), vdim=r.integer("vdim", minimum=1),
                      decay=tuple(float(d) for d in decay))


def parse_vipotar_config(values: dict) -> VipotarConfig:
    r = KeyReader(values)
    layers_raw = r.raw("layers")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: key 'layers' must be a non-empty list")
    layers = []
    for i, entry in enumerate(layers_raw):
        lr = KeyReader(entry, f"config.json: layers[{i}]")
        kind = lr.raw("type")
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{lr.where}: unknown type {kind!r}; known: {', '.join(LAYER_TYPES)}")
        mixer = _sub(lr, "mixer")
        mlp = _sub(lr, "mlp", required=False)
        ff = None
        if mlp is not None:
            mk = mlp.raw("kind")
            if mk not in MLP_KINDS:
                raise ConfigError(f"{mlp.where}: unknown kind {mk!r}; known: {', '.join(MLP_KINDS)}")
            ff = mlp.integer("ff", minimum=1)
        layers.append(VipotarLayer(type=kind, left=_left(_sub(mixer, "left")), right=_right(_sub(mixer, "right")), ff=ff))
    loop = _sub(r, "loop", required=False)
    start = stop = times = 0
    if loop is not None:
        start, stop, times = loop.integer("start", minimum=0), loop.integer("stop", minimum=0), loop.integer("times", minimum=1)
        if not start < stop <= len(layers):
            raise ConfigError(f"config.json: loop: start {start} < stop {stop} <= {len(layers)} layers does not hold")
    norm = _sub(r, "norm")
    cap = r.number("logit_softcap", default=None)
    return VipotarConfig(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), eps=norm.number("eps"),
                         residual_mult=r.number("residual_mult", default=1.0), logit_softcap=cap if cap else None,
                         layers=tuple(layers), loop_start=start, loop_stop=stop, loop_times=times)
