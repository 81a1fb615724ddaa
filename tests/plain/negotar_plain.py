"""Plain Negotar forward: whole sequences, no cache, one function per mechanism.

Written from the design's equations alone; it shares no code with the engine (own config
reading, plain numpy arithmetic, a loop per token where the engine has kernels).  All
arithmetic runs in the numpy dtype given (float64 by default: a ground truth for judging
rounding).

The design in this file's notation (x: the residual stream [T, width], one sequence):

  x = embed[tokens]
  layer:  x += rms(mixer(x)) * (1 + norm1);  x += rms(ff(x)) * (1 + norm2)      (ff absent: skipped)
          the sublayers read x itself; only their outputs are normed
  mixer "attention": grouped-query attention; q, k, v with biases; half-split rotation of the first
          rot.dims dimensions with frequencies rescaled by wavelength; then q and k divided by their own
          root mean square per head; score = cap * tanh(scale * q.k / cap); causal softmax; values of layers
          with v_mix (all but the first such) become (1 - lam) v + lam v_first
  mixer "mamba2": in -> [z | x | B | C | dt]; causal conv + silu over [x | B | C]; dt = softplus(dt + dt_bias);
          per head S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T,  y_t = S_t^T C_t + D x_t;
          y * silu(z), rms in norm_groups parts, * norm, W_o
  ff "moe": s = sigmoid(W_router x); the `top` largest; out = sum_e expert_e(s_e * x),
          expert(u) = W_down (silu(W_gate u) * (W_up u))
  out:    logits = embed (rms(x) * (1 + final.norm)) * logit_scale
"""
from __future__ import annotations

import math

import numpy as np


# ----------------------------------------------------------------------------
# small pieces
# ----------------------------------------------------------------------------

def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.where(z > 30.0, z, np.log1p(np.exp(np.minimum(z, 30.0))))


# ----------------------------------------------------------------------------
# rotation
# ----------------------------------------------------------------------------

def rotation_frequencies(rot):
    """Frequency per pair [dims/2] from the config's 'rot' entry; with 'scaling', long wavelengths are slowed
    by `factor`, short ones kept, and those in between blended."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            out[i] = fi
        elif wavelength > original / low:
            out[i] = fi / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_half_split(x, positions, freqs, dims):
    """x: [T, heads, dim]; dimension i pairs with i + dims/2 for i < dims/2; dimensions from `dims` on pass."""
    out = x.copy()
    half = dims // 2
    for t, p in enumerate(positions):
        a = p * freqs
        c, s = np.cos(a), np.sin(a)
        u, v = x[t, :, :half], x[t, :, half:dims]
        out[t, :, :half] = u * c - v * s
        out[t, :, half:dims] = v * c + u * s
    return out


# ----------------------------------------------------------------------------
# mixers
# ----------------------------------------------------------------------------

def attention_values(h, W, prefix, m):
    """The layer's own values [T, kv_heads, vdim] (before any mixing)."""
    v = h @ W[prefix + "v"].T + W[prefix + "v.b"]
    return v.reshape(h.shape[0], int(m["kv_heads"]), int(m["vdim"]))


def attention_mixer(h, W, prefix, m, eps, v_first=None, positions=None):
    """h: [T, width] -> ([T, width], this layer's values after mixing)."""
    T = h.shape[0]
    H, G, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    positions = np.arange(T) if positions is None else positions
    q = (h @ W[prefix + "q"].T + W[prefix + "q.b"]).reshape(T, H, dim)
    k = (h @ W[prefix + "k"].T + W[prefix + "k.b"]).reshape(T, G, dim)
    v = attention_values(h, W, prefix, m)
    rot = m.get("rot")
    if rot and int(rot["dims"]) > 0:
        f = rotation_frequencies(rot).astype(h.dtype)
        q = rotate_half_split(q, positions, f, int(rot["dims"]))
        k = rotate_half_split(k, positions, f, int(rot["dims"]))
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    if v_first is not None:
        lam = float(W[prefix + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    scale, cap = float(m["scale"]), m.get("softcap")
    out = np.zeros((T, H, vdim), dtype=h.dtype)
    per = H // G
    for hd in range(H):
        g = hd // per
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, hd]) * scale
            if cap:
                s = float(cap) * np.tanh(s / float(cap))
            p = np.exp(s - s.max())
            out[t, hd] = (p / p.sum()) @ v[:t + 1, g]
    return out.reshape(T, H * vdim) @ W[prefix + "o"].T, v


def causal_conv_silu(u, taps, bias):
    """u: [T, channels]; taps [channels, n]; the last column weighs the current token, zeros before the start."""
    T, n = u.shape[0], taps.shape[1]
    out = np.zeros_like(u)
    for t in range(T):
        acc = bias.copy()
        for j in range(n):
            src = t - (n - 1 - j)
            if src >= 0:
                acc = acc + taps[:, j] * u[src]
        out[t] = silu(acc)
    return out


def selective_scan(x, B, C, dt, A_log, D, groups):
    """x [T, heads, vdim], B and C [T, groups, N], dt [T, heads] (already positive) -> y [T, heads, vdim]."""
    T, heads, vdim = x.shape
    N = B.shape[2]
    per = heads // groups
    y = np.zeros_like(x)
    for hd in range(heads):
        g = hd // per
        S = np.zeros((N, vdim), dtype=x.dtype)
        a = -math.exp(float(A_log[hd]))
        for t in range(T):
            S = np.exp(a * dt[t, hd]) * S + dt[t, hd] * np.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + D[hd] * x[t, hd]
    return y


def grouped_unit_rms(y, parts, eps):
    """y: [T, n] normed in `parts` equal stretches, each by its own root mean square."""
    T, n = y.shape
    return unit_rms(y.reshape(T, parts, n // parts), eps).reshape(T, n)


def mamba2_mixer(h, W, prefix, m, eps):
    T = h.shape[0]
    heads, vdim, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = heads * vdim
    proj = h @ W[prefix + "in"].T
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * G * N]
    dt = proj[:, 2 * inner + 2 * G * N:]
    xbc = causal_conv_silu(xbc, W[prefix + "conv"], W[prefix + "conv.b"])
    x = xbc[:, :inner].reshape(T, heads, vdim)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W[prefix + "dt_bias"])
    y = selective_scan(x, B, C, dt, W[prefix + "A_log"], W[prefix + "D"], G).reshape(T, inner)
    y = grouped_unit_rms(y * silu(z), int(m["norm_groups"]), eps) * W[prefix + "norm"]
    return y @ W[prefix + "o"].T


# ----------------------------------------------------------------------------
# feed-forward
# ----------------------------------------------------------------------------

def routed_experts(h, W, prefix, mlp, gaps=None):
    """Sigmoid router, the `top` best experts, the score multiplies the expert's INPUT; no renormalisation.
    gaps: a list that receives, per row, how far the last chosen expert's router logit lies above the first one left
    out, as a fraction of the logits' root mean square (inf when every expert is used): small means a close call."""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ W[prefix + "router"].T
    s = sigmoid(z)
    if gaps is not None:
        zs = -np.sort(-z, axis=1)
        spread = np.maximum(np.sqrt(np.mean(z * z, axis=1)), 1e-3)
        gaps.append((zs[:, top - 1] - zs[:, top]) / spread if top < E else np.full(len(z), np.inf))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = sorted(range(E), key=lambda e: (-s[t, e], e))[:top]
        for e in chosen:
            u = s[t, e] * h[t]
            p = prefix + f"e{e}."
            out[t] += W[p + "down"] @ (silu(W[p + "gate"] @ u) * (W[p + "up"] @ u))
    return out


# ----------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------

def forward(cfg, W, tokens, dtype=np.float64, streams=None, gaps=None):
    """Logits [T, vocab] of one sequence.  W: tensor name -> numpy array.  streams: a list that receives the
    residual stream after every layer; gaps: a list that receives every routed layer's per-row gaps (routed_experts)."""
    W = {k: np.asarray(v).astype(dtype) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][np.asarray(tokens)]
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        if L["type"] == "attention":
            if m.get("v_mix"):
                y, v = attention_mixer(x, W, p + "mix.", m, eps, v_first=v_first)
                if v_first is None:
                    v_first = v
            else:
                y, _ = attention_mixer(x, W, p + "mix.", m, eps)
        elif L["type"] == "mamba2":
            y = mamba2_mixer(x, W, p + "mix.", m, eps)
        else:
            raise ValueError(f"unknown layer type {L['type']}")
        x = x + offset_norm(y, W[p + "norm1"], eps)
        if L.get("mlp") is not None:
            x = x + offset_norm(routed_experts(x, W, p + "mlp.", L["mlp"], gaps), W[p + "norm2"], eps)
        if streams is not None:
            streams.append(x.copy())
    h = offset_norm(x, W["final.norm"], eps)
    return (h @ W["embed"].T) * float(cfg.get("logit_scale", 1.0))
