"""Linear attention with a per-head decay, as a part (mixer "decay_linear_attention").

With q_t, k_t (heads x dim) and v_t (heads x vdim) the activated projections of the input, every head keeps a
state S [dim, vdim] per request:  S_t = decay_h * S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t  (no other scale).  The
heads' outputs, side by side, are RMS-normed together (one weight over heads*vdim), multiplied by
sigmoid(W_g x), and projected by W_o.  The state starts at zero for a new request, is 32-bit, and lives in the
request's state slot; the decays, the recurrence, the norm and the gate are 32-bit in both precisions.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .spec import SlotState, WeightSpec


class DecayLinearAttention(Part):
    """params: hidden, heads, dim, vdim, decay (one number per head), eps (of the output norm), act ("silu" or None,
    on q, k and v), names (optional dict of tensor names after the prefix).

    forward(..., accumulate=False) overwrites `residual` (then any float32 [tokens, hidden] buffer)."""
    adds_with_linear = True
    CHUNK_FROM = 128          # portions from this many tokens on (rounded up to a power of two) run in chunks

    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.eps = float(p["eps"])
        self.act = p.get("act", "silu")
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"linear attention: {len(decay)} decays for {self.heads} heads")
        if not 1 <= self.dim <= 256:
            raise ValueError(f"linear attention: key size {self.dim} is not supported by the kernel (1 to 256)")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(rt.device)
        self.names = {k: prefix + v for k, v in {**self.NAMES, **p.get("names", {})}.items()}
        self.w_in = self.w_o = self.w_norm = None

    def weight_specs(self):
        n, H = self.names, self.hidden
        qk, vv = self.heads * self.dim, self.heads * self.vdim
        return [WeightSpec(n["q"], ((qk, H),)), WeightSpec(n["k"], ((qk, H),)), WeightSpec(n["v"], ((vv, H),)),
                WeightSpec(n["g"], ((vv, H),)), WeightSpec(n["o"], ((H, vv),)),
                WeightSpec(n["norm"], ((vv,),), role="vector", init=("norm",))]

    def bind(self, tensors):
        n = self.names
        # one fused projection [q | k | v | g]: a layout choice, the arithmetic is unchanged
        self.w_in = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]]], dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        self.w_norm = tensors[n["norm"]]

    def cache_specs(self):
        return (SlotState((self.heads, self.dim, self.vdim)),)

    def input_rows(self) -> int:
        return 2 * self.heads * self.dim + 2 * self.heads * self.vdim

    def input_weight(self):
        return self.w_in

    def adopt_input_weight(self, view) -> None:
        self.w_in = view

    def forward(self, x, batch, caches, residual, accumulate=True, projected=None):
        st = caches[0]
        rt, T = self.rt, x.shape[0]
        qk, vv = self.heads * self.dim, self.heads * self.vdim
        if projected is not None:
            proj = projected
        else:
            proj = rt.workspace.get("linattn_in", (T, 2 * qk + 2 * vv), rt.act_dtype, first="tokens")
            ops.linear(x, self.w_in, proj, status=rt.status)
        o = rt.workspace.get("linattn_o", (T, vv), torch.float32, first="tokens")
        # long portions: the recurrence in chunks that run side by side (a row-by-row walk of a 2,048-token prompt is 2,048
        # dependent steps on a handful of warps); the chunk length follows the step's size, which is part of its shape
        chunk, scratch = 0, None
        if batch.max_tokens_per_item >= self.CHUNK_FROM:
            chunk = 64 if T <= 4096 else (128 if T <= 16384 else 256)
            scratch = rt.workspace.get("linattn_chunks", ((T // chunk + batch.n_items) * self.heads * self.dim * self.vdim,),
                                       torch.float32)
        ops.linear_attention(proj, 0, qk, 2 * qk, self.decay, st.state, batch.item_row_start, batch.item_slot, batch.n_items,
                             o, self.heads, self.dim, self.vdim, rt.status, act=self.act, chunk=chunk, chunk_state=scratch)
        y = rt.workspace.get("linattn_y", (T, vv), rt.act_dtype, first="tokens")
        ops.gated_rmsnorm(o, self.w_norm, self.eps, proj[:, 2 * qk + vv:], y)
        ops.linear(y, self.w_o, residual, accumulate=accumulate, status=rt.status)
