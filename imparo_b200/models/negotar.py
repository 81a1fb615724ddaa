"""Negotar: which parts each layer has, from its typed config.

Layer i (tensors "l<i>."): the output-norm arrangement (x += norm1(mixer(x)); x += norm2(feed_forward(x)), norms whose
stored tensor is the weight minus one) around a mixer "mix." — an attention with q/k/v biases ("q.b", ...), a half-split rotation
with wavelength-scaled frequencies, a norm without a weight on q and k, a soft cap on the scores and values blended with
the first such layer's ("vmix"), or a Mamba-2 mixer ("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o") — and
a routed feed-forward "mlp." ("router", "e<j>.gate" / "up" / "down") whose experts are fed the input times their sigmoid score.
Embedding "embed" unscaled, final norm "final.norm", head tied to the embedding, logits times logit_scale.
"""
from __future__ import annotations

from ..config.negotar import NegotarConfig, parse_negotar_config
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20         # the design states no limit; rotation angles are 32-bit products


def negotar_model_spec(cfg: NegotarConfig) -> ModelSpec:
    W = cfg.width
    layers = []
    source_seen = False
    for i, L in enumerate(cfg.layers):
        prefix = f"l{i}."
        m = L.mixer
        if L.type == "attention":
            position = PartSpec("none")
            if m.rot_dims:
                sc = m.rot_scaling
                position = PartSpec("rope_neox", {
                    "head_dim": m.dim, "n_rot": m.rot_dims, "theta": m.rot_base,
                    "wavelength_scaling": None if sc is None else {"factor": sc.factor, "low": sc.low, "high": sc.high,
                                                                   "original": sc.original}})
            share = None
            if m.v_mix:
                share = {"role": "blend" if source_seen else "source", "lambda": "mix.vmix"}
                source_seen = True
            mixer = PartSpec("attention", {
                "hidden": W, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "scale": m.scale, "softcap": m.softcap, "qk_norm": False, "unit_norm": True, "eps": cfg.eps, "bias": "required",
                "v_share": share, "position": position,
                "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_bias": "mix.q.b", "k_bias": "mix.k.b",
                          "v_bias": "mix.v.b"}})
        else:
            mixer = PartSpec("mamba2", {
                "hidden": W, "heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups, "conv": m.conv,
                "norm_groups": m.norm_groups, "eps": cfg.eps,
                "names": {k: "mix." + v for k, v in {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias",
                                                     "A_log": "A_log", "D": "D", "norm": "norm", "o": "o"}.items()}})
        ff = ff_norm = None
        if L.mlp is not None:
            ff = PartSpec("routed_experts", {
                "hidden": W, "ff": L.mlp.ff, "experts": L.mlp.experts, "top": L.mlp.top, "score": "sigmoid",
                "renormalise": False, "weight_on": "input",
                "names": {"router": "mlp.router", "gate": "mlp.e{e}.gate", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down"}})
            ff_norm = PartSpec("rmsnorm", {"width": W, "eps": cfg.eps, "name": "norm2", "offset": 1.0})
        layers.append(LayerSpec(prefix=prefix, mixer=mixer, feed_forward=ff,
                                mixer_norm=PartSpec("rmsnorm", {"width": W, "eps": cfg.eps, "name": "norm1", "offset": 1.0}),
                                feed_forward_norm=ff_norm, block="outnorm_residual"))
    return ModelSpec(
        architecture="Negotar", vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab, "width": W, "name": "embed"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"width": W, "eps": cfg.eps, "name": "final.norm", "offset": 1.0}),
        head=PartSpec("linear", {"vocab": cfg.vocab, "width": W, "name": "embed", "scale": cfg.logit_scale}),
        max_positions=MAX_POSITIONS, eos_token_ids=())


register_architecture(Architecture(name="Negotar", model_types=("negotar",),
                                   parse_config=parse_negotar_config, model_spec=negotar_model_spec), replace=True)
