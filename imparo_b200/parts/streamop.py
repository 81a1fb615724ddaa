"""Parts that work on the residual stream between layers (kind "stream_op"): a schedule entry may name
one that runs right before it (ScheduleEntry.before).

StretchEntry: what a repeated stretch of layers gets at the start of each of its passes: a learned vector
of that pass, row `index` of a [passes, width] tensor, and — from the second pass on — the tokens' embedding
rows once more (the embedding's output is the plain table row, so it is gathered again, not kept)."""
from __future__ import annotations

from ..kernels import ops
from .base import Part
from .spec import WeightSpec


class StretchEntry(Part):
    """params: width, passes, index (which pass), vector (tensor name [passes, width], or None),
    embedding (tensor name of the token table to add again, or None), vocab."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.width = int(params["width"])
        self.passes = int(params["passes"])
        self.index = int(params["index"])
        self.vector_name = params.get("vector")
        self.embedding_name = params.get("embedding")
        self.vocab = int(params.get("vocab", 0))
        if not 0 <= self.index < self.passes:
            raise ValueError(f"stretch entry: pass {self.index} of {self.passes}")
        self.vec = self.table = None

    def weight_specs(self):
        specs = []
        if self.vector_name:
            specs.append(WeightSpec(self.vector_name, ((self.passes, self.width),), role="vector", init=("normal", 0.02)))
        if self.embedding_name:
            specs.append(WeightSpec(self.embedding_name, ((self.vocab, self.width),)))
        return specs

    def bind(self, tensors):
        if self.vector_name:
            self.vec = tensors[self.vector_name][self.index].contiguous()
        if self.embedding_name:
            self.table = tensors[self.embedding_name]

    def forward(self, x, batch):
        ops.stream_inject(x, self.table, batch.token_ids if self.table is not None else None, self.vec, self.rt.status)
