"""The selective state-space mixer in its Mamba-2 form, as a part (mixer "mamba2").

With inner = heads * vdim, N = state and G = groups, one projection of the input gives a row
[z: inner | x: inner | B: G*N | C: G*N | dt: heads].  x, B and C pass a causal convolution per channel (taps from the
config, a bias, zeros before the start) and silu.  dt = softplus(dt + dt_bias).  Head h (group h // (heads / G)) keeps a
state S [N, vdim] per request:  S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T;  y_t = S_t^T C_t + D_h x_t.
The heads' outputs, side by side, are multiplied by silu(z), RMS-normed in norm_groups equal stretches (each by its own
root mean square) times a weight, and projected by W_o.  The state and the convolution's last taps-1 inputs live in the
request's slot; the state starts at zero; step sizes, decays and the recurrence are 32-bit in both precisions.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .spec import SlotState, WeightSpec


class Mamba2Mixer(Part):
    """params: hidden, heads, vdim, state, groups, conv (taps), norm_groups, eps (of the gated norm), names (optional
    dict of tensor names after the prefix).

    forward(..., accumulate=False) overwrites `residual` (then any float32 [tokens, hidden] buffer)."""
    adds_with_linear = True
    CHUNK_FROM = 128          # portions from this many tokens on (rounded up to a power of two) run in chunks
    CHUNK = 64

    NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D",
             "norm": "norm", "o": "o"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.vdim = int(p["vdim"])
        self.n_state = int(p["state"])
        self.groups = int(p["groups"])
        self.taps = int(p["conv"])
        self.norm_groups = int(p.get("norm_groups", 1))
        self.eps = float(p["eps"])
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n_state
        self.d_in = 2 * self.inner + 2 * self.groups * self.n_state + self.heads
        if self.heads % self.groups:
            raise ValueError(f"mamba2: groups {self.groups} must divide heads {self.heads}")
        if self.inner % self.norm_groups:
            raise ValueError(f"mamba2: norm_groups {self.norm_groups} must divide heads * vdim = {self.inner}")
        if not 1 <= self.n_state <= 256:
            raise ValueError(f"mamba2: state size {self.n_state} is not supported by the kernel (1 to 256)")
        if not 1 <= self.taps <= 17:
            raise ValueError(f"mamba2: {self.taps} conv taps are not supported by the kernel (1 to 17)")
        self.names = {k: prefix + v for k, v in {**self.NAMES, **p.get("names", {})}.items()}
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.A_log = self.D = self.w_norm = None

    def weight_specs(self):
        n, H = self.names, self.hidden
        return [WeightSpec(n["in"], ((self.d_in, H),)),
                WeightSpec(n["conv"], ((self.channels, self.taps),), role="vector", init=("conv_taps",)),
                WeightSpec(n["conv_bias"], ((self.channels,),), role="vector", init=("bias",)),
                WeightSpec(n["dt_bias"], ((self.heads,),), role="vector", init=("uniform", -4.0, -1.0)),
                WeightSpec(n["A_log"], ((self.heads,),), role="vector", init=("uniform", -1.0, 1.5)),
                WeightSpec(n["D"], ((self.heads,),), role="vector", init=("uniform", 0.5, 1.5)),
                WeightSpec(n["norm"], ((self.inner,),), role="vector", init=("norm",)),
                WeightSpec(n["o"], ((H, self.inner),))]

    def bind(self, tensors):
        n = self.names
        self.w_in, self.w_o = tensors[n["in"]], tensors[n["o"]]
        self.conv_w, self.conv_b = tensors[n["conv"]], tensors[n["conv_bias"]]
        self.dt_bias, self.A_log, self.D, self.w_norm = tensors[n["dt_bias"]], tensors[n["A_log"]], tensors[n["D"]], tensors[n["norm"]]

    def cache_specs(self):
        return (SlotState((self.heads, self.n_state, self.vdim)), SlotState((max(self.taps - 1, 1), self.channels)))

    def forward(self, x, batch, caches, residual, accumulate=True):
        ssm, conv = caches
        rt, T = self.rt, x.shape[0]
        ws = rt.workspace
        inner = self.inner
        # the projection stays 32-bit: step sizes, B, C and x enter the recurrence unrounded
        proj = ws.get("mamba_in", (T, self.d_in), torch.float32, first="tokens")
        ops.linear(x, self.w_in, proj, status=rt.status)
        xbc = ws.get("mamba_xbc", (T, self.channels), torch.float32, first="tokens")
        dt = ws.get("mamba_dt", (T, self.heads), torch.float32, first="tokens")
        ops.mamba2_conv(proj, inner, inner + self.channels, self.channels, self.heads, self.taps, self.conv_w, self.conv_b,
                        self.dt_bias, conv.state, batch.item_row_start, batch.item_of_token, batch.item_slot, batch.n_items,
                        xbc, dt, rt.status)
        y = ws.get("mamba_y", (T, inner), torch.float32, first="tokens")
        chunk, scratch = 0, None
        if batch.max_tokens_per_item >= self.CHUNK_FROM:
            # long portions: chunks of rows side by side; the chunk length is fixed, so the cut depends on the rows alone
            chunk = self.CHUNK
            most = T // chunk + batch.n_items
            scratch = (ws.get("mamba_chunk_i", (3 * most + batch.n_items + 1,), torch.int32),
                       ws.get("mamba_chunk_state", (most * self.heads * self.n_state * self.vdim,), torch.float32),
                       ws.get("mamba_chunk_decay", (most * self.heads,), torch.float32))
        ops.mamba2_scan(xbc, dt, self.A_log, self.D, ssm.state, batch.item_row_start, batch.item_slot, batch.n_items, y,
                        self.heads, self.vdim, self.n_state, self.groups, rt.status, chunk=chunk, scratch=scratch)
        g = ws.get("mamba_gated", (T, inner), rt.act_dtype, first="tokens")
        ops.gate_group_rmsnorm(y, proj[:, :inner], self.w_norm, self.eps, self.norm_groups, g)
        ops.linear(g, self.w_o, residual, accumulate=accumulate, status=rt.status)
