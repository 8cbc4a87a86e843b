"""Parts that rewrite the residual stream between runs of layers."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import DeltaPair, StreamEntry, as_delta, matrix, register_stream_entry, vector_f32


@register_stream_entry("mix_with_embedding")
class MixWithEmbedding(StreamEntry):
    """x <- W [x; x0] + s: the stream and the embedding's output side by side go through one matrix [hidden, 2 hidden]
    (x's columns first), and a vector is added: row `row` of a table [rows, hidden] (one row per pass of a loop over
    layers).  The pending deltas are added to x first, in float32; the product writes the float32 stream.

    params: matrix (tensor name), vectors (tensor name), rows, row, hidden_size.
    """

    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.matrix_name, self.vectors_name = spec["matrix"], spec["vectors"]
        self.rows, self.row, self.hidden = int(spec["rows"]), int(spec["row"]), int(spec["hidden_size"])
        if not 0 <= self.row < self.rows:
            raise ValueError(f"mix_with_embedding: row {self.row} of {self.rows}")

    def tensors(self):
        return [TensorDecl(self.matrix_name, (self.hidden, 2 * self.hidden)), TensorDecl(self.vectors_name, (self.rows, self.hidden), init="bias")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        shared = rt.__dict__.setdefault("shared_weights", {})  # the passes of a loop read one matrix: one copy on the device
        key = ("matrix", self.matrix_name, rt.dtype)
        if key not in shared or shared[key][0] is not tensors[self.matrix_name]:
            shared[key] = (tensors[self.matrix_name], matrix(tensors[self.matrix_name], rt))
        self.weight = shared[key][1]
        self.vector = vector_f32(tensors[self.vectors_name][self.row])

    def forward(self, ctx, residual, pending, first):
        rt, (t, d) = self.rt, residual.shape
        a, b = (pending.a, pending.b) if isinstance(pending, DeltaPair) else (as_delta(pending), None)
        both = rt.workspace.get("entry.both", (t, 2 * d), rt.dtype)
        ops.concat_streams(residual, a, b, first, both)
        ops.linear(both, self.weight, self.vector, residual)
        return None


@register_stream_entry("add_embedding")
class AddEmbedding(StreamEntry):
    """x <- x + x0 + s: the embedding's output is added to the stream (only with `add_first`), then a vector: row `row`
    of a table [rows, hidden] (one row per pass of a loop over layers).  The pending deltas are added to x first; all
    in float32, by one kernel.

    params: vectors (tensor name), rows, row, hidden_size, add_first.
    """

    graph_safe = True
    kernel_files = ('stream',)

    def __init__(self, spec):
        super().__init__(spec)
        self.vectors_name = spec["vectors"]
        self.rows, self.row, self.hidden = int(spec["rows"]), int(spec["row"]), int(spec["hidden_size"])
        self.add_first = bool(spec["add_first"])
        if not 0 <= self.row < self.rows:
            raise ValueError(f"add_embedding: row {self.row} of {self.rows}")

    def tensors(self):
        return [TensorDecl(self.vectors_name, (self.rows, self.hidden), init="bias")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.vector = vector_f32(tensors[self.vectors_name][self.row])

    def forward(self, ctx, residual, pending, first):
        a, b = (pending.a, pending.b) if isinstance(pending, DeltaPair) else (as_delta(pending), None)
        ops.add_streams_rmsnorm(residual, a, b, first if self.add_first else None, self.vector, None, None)
        return None
