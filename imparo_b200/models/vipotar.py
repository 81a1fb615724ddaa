"""Vipotar: which parts each layer has, from its typed config.

Layer i (tensors "l<i>."): the parallel arrangement (one norm "norm1"; x += m * (mixer + feed-forward)) around a
side-by-side mixer ("mix.": "left" a windowed attention with a sink and an interleaved, optionally scaled,
partial rotation; "right" a decayed linear attention; each output RMS-normed with "mix.left.out" /
"mix.right.out" and the two averaged) and a dense feed-forward with a squared ReLU ("mlp.up", "mlp.down").
Embedding "embed" unscaled, final norm "final.norm", own head "head" with an optional soft cap.  A repeated
stretch of layers becomes schedule entries that name the same layers again (each run owns its cache); the first
entry of every pass is preceded by a stream operation that adds "loop.step"[pass] and, from the second pass on,
the tokens' embedding rows."""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.vipotar import VipotarConfig, parse_vipotar_config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20         # the design states no limit; rotation angles are 32-bit products


def vipotar_model_spec(cfg: VipotarConfig) -> ModelSpec:
    W = cfg.width
    layers = []
    for i, L in enumerate(cfg.layers):
        prefix = f"l{i}."
        left, right = L.left, L.right
        position = PartSpec("none")
        if left.rot_dims:
            sc = left.rot_scaling
            position = PartSpec("rope_interleaved", {
                "head_dim": left.dim, "n_rot": left.rot_dims, "theta": left.rot_base,
                "scaling": None if sc is None else {"factor": sc.factor, "original": sc.original, "fast": sc.fast, "slow": sc.slow}})
        attention = PartSpec("attention", {
            "hidden": W, "n_heads": left.heads, "n_kv_heads": left.kv_heads, "head_dim": left.dim, "v_head_dim": left.vdim,
            "scale": left.scale, "window": left.window, "sink": True, "qk_norm": False, "position": position,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o"}})
        linear = PartSpec("decay_linear_attention", {
            "hidden": W, "heads": right.heads, "dim": right.dim, "vdim": right.vdim, "decay": right.decay, "eps": cfg.eps,
            "act": "silu"})
        mixer = PartSpec("side_by_side", {"hidden": W, "eps": cfg.eps, "branches": (
            ("mix.left.", attention, "mix.left.out"), ("mix.right.", linear, "mix.right.out"))})
        ff = None if L.ff is None else PartSpec("dense", {"hidden": W, "ff": L.ff, "act": "relu2",
                                                          "names": {"up": "mlp.up", "down": "mlp.down"}})
        layers.append(LayerSpec(prefix=prefix, mixer=mixer, feed_forward=ff,
                                mixer_norm=PartSpec("rmsnorm", {"width": W, "eps": cfg.eps, "name": "norm1"}),
                                feed_forward_norm=None, block="parallel_residual",
                                params={"residual_scale": cfg.residual_mult}))
    n = len(cfg.layers)
    if cfg.has_loop:
        schedule = [ScheduleEntry(i) for i in range(cfg.loop_start)]
        for t in range(cfg.loop_times):
            for i in range(cfg.loop_start, cfg.loop_stop):
                before = None
                if i == cfg.loop_start:
                    before = PartSpec("stretch_entry", {"width": W, "passes": cfg.loop_times, "index": t, "vector": "loop.step",
                                                        "embedding": "embed" if t > 0 else None, "vocab": cfg.vocab})
                schedule.append(ScheduleEntry(i, before=before))
        schedule += [ScheduleEntry(i) for i in range(cfg.loop_stop, n)]
    else:
        schedule = [ScheduleEntry(i) for i in range(n)]
    return ModelSpec(
        architecture="Vipotar", vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab, "width": W, "name": "embed"}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", {"width": W, "eps": cfg.eps, "name": "final.norm"}),
        head=PartSpec("linear", {"vocab": cfg.vocab, "width": W, "name": "head", "softcap": cfg.logit_softcap}),
        max_positions=MAX_POSITIONS, eos_token_ids=())


register_architecture(Architecture(name="Vipotar", model_types=("vipotar",),
                                   parse_config=parse_vipotar_config, model_spec=vipotar_model_spec), replace=True)
