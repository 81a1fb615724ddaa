"""Plain Vipotar forward: whole sequences, no cache, one function per mechanism.

Written from the design's equations alone; it shares no code with the engine (own
config reading, plain numpy arithmetic, a loop per token where the engine has kernels).
All arithmetic runs in the numpy dtype given (float64 by default: a ground truth for
judging rounding).

The design in this file's notation (x: the residual stream [T, width], one sequence):

  x = embed[tokens]                                     e0 = x (kept for the looped passes)
  layers: the list of the config; layers start..stop-1 run `times` times in a row (same
          weights, every pass a cache of its own), then the rest.  Right before the first
          layer of pass t:  x += e0 (t > 0);  x += loop.step[t].
  layer:  h = rms(x) * norm1;  x += m * (mixer(h) + ff(h))         (ff absent: 0)
  mixer:  0.5 * (rms(L(h)) * left.out + rms(R(h)) * right.out)
  L:      windowed grouped-query attention; interleaved partial rotation with scaled
          frequencies; probabilities exp(s_j) / (1 + sum_j exp(s_j))
  R:      linear attention with a per-head decay: S_t = d S_(t-1) + k_t v_t^T, o_t = S_t^T q_t,
          q, k, v = silu(projections); then rms over all heads * norm * sigmoid(W_g h), W_o
  ff:     W_down relu(W_up h)^2
  out:    logits = head (rms(x) * final.norm), then cap * tanh(logits / cap)
"""
from __future__ import annotations

import math

import numpy as np


# ----------------------------------------------------------------------------
# small pieces
# ----------------------------------------------------------------------------

def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w None: no weight)."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def relu_squared(z):
    r = np.maximum(z, 0.0)
    return r * r


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def soft_cap(z, cap):
    return cap * np.tanh(z / cap)


# ----------------------------------------------------------------------------
# rotation
# ----------------------------------------------------------------------------

def rotation_table(rot):
    """(frequency per pair [dims/2], magnitude) from the config's 'rot' entry."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    i = np.arange(dims // 2, dtype=np.float64)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, freq, magnitude):
    """x [T, heads, dim]: dimension 2i turns with 2i+1 by positions * freq[i]; the rest passes."""
    out = x.copy()
    n = 2 * len(freq)
    a = positions[:, None].astype(x.dtype) * freq[None, :].astype(x.dtype)        # [T, n/2]
    c, s = np.cos(a)[:, None, :] * magnitude, np.sin(a)[:, None, :] * magnitude
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------
# the two mixers
# ----------------------------------------------------------------------------

def window_attention(h, w, prefix, cfg, dtype):
    """The left mixer on one whole sequence.  h [T, width] -> [T, width]."""
    T = h.shape[0]
    H, G, D, Dv = int(cfg["heads"]), int(cfg["kv_heads"]), int(cfg["dim"]), int(cfg["vdim"])
    q = (h @ w[prefix + "q"].T).reshape(T, H, D)
    k = (h @ w[prefix + "k"].T).reshape(T, G, D)
    v = (h @ w[prefix + "v"].T).reshape(T, G, Dv)
    pos = np.arange(T)
    if cfg.get("rot"):
        freq, mag = rotation_table(cfg["rot"])
        q, k = rotate_interleaved(q, pos, freq, mag), rotate_interleaved(k, pos, freq, mag)
    size = int(cfg["mask"]["size"]) if cfg.get("mask") else None
    scale = float(cfg["scale"])
    out = np.zeros((T, H, Dv), dtype=dtype)
    for hh in range(H):
        g = hh // (H // G)
        for i in range(T):
            lo = 0 if size is None else max(0, i - size + 1)
            s = (k[lo:i + 1, g] @ q[i, hh]) * scale
            m = max(float(s.max()), 0.0)
            e = np.exp(s - m)
            p = e / (math.exp(-m) + e.sum())                  # one more term in the sum below: exp(0), no value
            out[i, hh] = p @ v[lo:i + 1, g]
    return out.reshape(T, H * Dv) @ w[prefix + "o"].T


def decayed_linear_attention(h, w, prefix, cfg, eps, dtype, state=None):
    """The right mixer on one whole sequence, token by token.  Returns ([T, width], final state)."""
    T = h.shape[0]
    H, D, Dv = int(cfg["heads"]), int(cfg["dim"]), int(cfg["vdim"])
    decay = np.asarray(cfg["decay"], dtype=dtype)
    q = silu(h @ w[prefix + "q"].T).reshape(T, H, D)
    k = silu(h @ w[prefix + "k"].T).reshape(T, H, D)
    v = silu(h @ w[prefix + "v"].T).reshape(T, H, Dv)
    S = np.zeros((H, D, Dv), dtype=dtype) if state is None else state.copy()
    o = np.zeros((T, H, Dv), dtype=dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    y = rms_norm(o.reshape(T, H * Dv), w[prefix + "norm"], eps) * sigmoid(h @ w[prefix + "g"].T)
    return y @ w[prefix + "o"].T, S


def side_by_side(h, w, prefix, cfg, eps, dtype):
    left = window_attention(h, w, prefix + "left.", cfg["left"], dtype)
    right, _ = decayed_linear_attention(h, w, prefix + "right.", cfg["right"], eps, dtype)
    return 0.5 * (rms_norm(left, w[prefix + "left.out"], eps) + rms_norm(right, w[prefix + "right.out"], eps))


def feed_forward(h, w, prefix, cfg):
    if cfg is None:
        return 0.0
    if cfg["kind"] != "dense":
        raise ValueError(f"feed-forward kind {cfg['kind']}")
    return relu_squared(h @ w[prefix + "up"].T) @ w[prefix + "down"].T


# ----------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------

def layer_runs(config):
    """[(layer index, pass number or None, first of its pass)] in running order."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None, False) for i in range(start)]
    for t in range(times):
        runs += [(i, t, i == start) for i in range(start, stop)]
    return runs + [(i, None, False) for i in range(stop, n)]


def forward(config, weights, tokens, dtype=np.float64, per_layer=False):
    """tokens: one sequence.  -> logits [T, vocab] (and the stream after every layer run)."""
    w = {k: (v.astype(dtype) if v.dtype.kind == "f" else v) for k, v in weights.items()}
    eps, m = float(config["norm"]["eps"]), float(config["residual_mult"])
    x = w["embed"][np.asarray(tokens)]
    e0 = x.copy()
    streams = []
    for i, t, first in layer_runs(config):
        if first:
            if t > 0:
                x = x + e0
            x = x + w["loop.step"][t]
        L = config["layers"][i]
        if L["type"] != "parallel":
            raise ValueError(f"layer type {L['type']}")
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        x = x + m * (side_by_side(h, w, p + "mix.", L["mixer"], eps, dtype) + feed_forward(h, w, p + "mlp.", L.get("mlp")))
        streams.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = soft_cap(logits, float(cap))
    return (logits, np.stack(streams)) if per_layer else logits
