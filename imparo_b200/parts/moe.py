"""A routed feed-forward (mixture of experts) as a part (feed_forward "routed_experts").

Router logits z = W_r h in 32-bit; scores sigmoid(z) (or a softmax over the experts); each row uses the `top` experts
with the largest scores, weighted by those scores (optionally renormalised to sum 1).  An expert is a gated
feed-forward without biases, W_down (silu(W_gate u) * (W_up u)); the weight multiplies the expert's input u = w h
(weight_on "input") or its output (weight_on "output").  The row's result is the sum over its experts, in the order of
their scores.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .spec import WeightSpec


class RoutedExperts(Part):
    """params: hidden, ff (per expert), experts, top, score ("sigmoid" | "softmax", default sigmoid), renormalise (bool,
    default False), weight_on ("input" | "output", default "output"), names (optional: router, and gate / up / down as
    patterns with {e} for the expert's number).

    forward(x, batch, residual, accumulate=False) overwrites `residual` (a float32 [rows, hidden] buffer)."""
    GROUP_FROM = 65           # steps with at least this many (row, expert) pairs run sorted by expert, in tiles
    TILES_FROM = 256          # and from this many on (bfloat16, aligned sizes) on the tensor-memory product, tiles of 128 rows

    NAMES = {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden"])
        self.ff = int(p["ff"])
        self.experts = int(p["experts"])
        self.top = int(p["top"])
        self.score = p.get("score", "sigmoid")
        self.renormalise = bool(p.get("renormalise", False))
        self.weight_on = p.get("weight_on", "output")
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"routed experts: unknown score '{self.score}' (sigmoid, softmax)")
        if self.weight_on not in ("input", "output"):
            raise ValueError(f"routed experts: weight_on is 'input' or 'output', found '{self.weight_on}'")
        if not 1 <= self.top <= min(self.experts, 32):
            raise ValueError(f"routed experts: top {self.top} must be between 1 and min(experts, 32) = {min(self.experts, 32)}")
        self.names = {k: prefix + v for k, v in {**self.NAMES, **p.get("names", {})}.items()}
        self.w_router = self.w_gu = self.w_down = None

    def weight_specs(self):
        n, H, F = self.names, self.hidden, self.ff
        specs = [WeightSpec(n["router"], ((self.experts, H),), role="vector", init=("normal", 0.5))]
        for e in range(self.experts):
            specs += [WeightSpec(n["gate"].format(e=e), ((F, H),)), WeightSpec(n["up"].format(e=e), ((F, H),)),
                      WeightSpec(n["down"].format(e=e), ((H, F),))]
        return specs

    def bind(self, tensors):
        n = self.names
        self.w_router = tensors[n["router"]]
        # For bfloat16 rows the router's logits come from the tensor-core product: the 32-bit matrix cut into three
        # bfloat16 pieces that add up to it to its last bit, so every product is exact and the sums are 32-bit.
        self.w_router_pieces = None
        if self.rt.act_dtype == torch.bfloat16:
            rest, pieces = self.w_router.float(), []
            for _ in range(3):
                piece = rest.to(torch.bfloat16)
                pieces.append(piece)
                rest = rest - piece.float()
            self.w_router_pieces = torch.cat(pieces, dim=0).contiguous()
        # experts stacked: [experts, 2 ff, hidden] = [gate; up] and [experts, hidden, ff]
        self.w_gu = torch.stack([torch.cat([tensors[n["gate"].format(e=e)], tensors[n["up"].format(e=e)]], dim=0)
                                 for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[n["down"].format(e=e)] for e in range(self.experts)]).contiguous()

    def forward(self, x, batch, residual, accumulate=False):
        if accumulate:
            raise ValueError("routed experts write their output into a buffer of their own (accumulate=False)")
        rt, T = self.rt, x.shape[0]
        ws = rt.workspace
        ids = ws.get("moe_ids", (T, self.top), torch.int32, first="tokens")
        wts = ws.get("moe_wts", (T, self.top), torch.float32, first="tokens")
        if self.w_router_pieces is not None and x.dtype == torch.bfloat16:
            logits = ws.get("moe_logits", (T, 3 * self.experts), torch.float32, first="tokens")
            ops.linear(x, self.w_router_pieces, logits, status=rt.status)
            ops.moe_pick(logits, self.experts, 3, self.top, ids, wts, softmax=self.score == "softmax", renormalise=self.renormalise)
        else:
            ops.moe_route(x, self.w_router, self.top, ids, wts, softmax=self.score == "softmax", renormalise=self.renormalise,
                          logits=ws.get("moe_logits", (T, self.experts), torch.float32, first="tokens"))
        pairs = T * self.top
        if pairs >= self.TILES_FROM and ops.moe_tiles_usable(x, self.w_gu):
            # many rows in bfloat16: sorted into tiles of 128 rows per expert, both products on the tensor-memory kernel
            rows = (pairs // 128 + self.experts) * 128
            ops.moe_experts_tiles(x, self.w_gu, self.w_down, ids, wts, self.top, self.weight_on == "input",
                                  ws.get("moe_sorted_in", (rows, self.hidden), rt.act_dtype),
                                  ws.get("moe_sorted_mid", (rows, self.ff), rt.act_dtype),
                                  ws.get("moe_sorted_out", (rows, self.hidden), torch.float32),
                                  ws.get("moe_tile_plan", (pairs + rows // 128,), torch.int32), residual, rt.status)
            return
        mid = ws.get("moe_mid", (T * self.top, self.ff), rt.act_dtype, first="tokens")
        scratch = None
        if pairs >= self.GROUP_FROM:
            scratch = (ws.get("moe_pair_out", (pairs, self.hidden), torch.float32, first="tokens"),
                       ws.get("moe_plan", (pairs + self.experts + 2 + 3 * (pairs // 32 + self.experts),), torch.int32))
        ops.moe_experts(x, self.w_gu, self.w_down, ids, wts, self.top, self.weight_on == "input", mid, residual, scratch=scratch)
