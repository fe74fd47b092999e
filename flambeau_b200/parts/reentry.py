"""Re-entry of the embedding output into the stream."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, TensorSpec
from .linear import Linear
from .spec import register_part


class ConcatLinearReentry(Part):
    """x <- W [x ; x0]: the stream and the embedding output x0 side by side through one linear map
    W [width, 2 * width] (the stream's columns first), whose result replaces the stream.  What a part left pending
    is added to the stream first (through the norm it is pending with).  The operands are rounded to the engine's
    dtype for the product; the result is the float32 stream."""
    graph_safe = True
    category = "reentry"

    def __init__(self, runtime=None, prefix="", *, width: int, weight_name: str = "weight", init_std: float = 0.02):
        super().__init__(runtime, prefix)
        self.width, self.weight_name, self.init_std = int(width), weight_name, init_std
        self.map = None

    def own_tensor_specs(self):
        return {self.prefix + self.weight_name: TensorSpec((self.width, 2 * self.width), init=("normal", self.init_std))}

    def own_bind(self, tensors):
        self.map = Linear(tensors[self.prefix + self.weight_name])

    def own_weights(self):
        return [self.map.weight]

    def forward(self, ctx, stream, x0) -> None:
        n = ctx.n_tokens
        stream.settle(ctx)
        with ctx.ws.scope():
            both = ctx.ws.alloc((n, 2 * self.width), self.runtime.dtype)
            ops.concat_cast(stream.x[:n], x0[:n], both)
            self.map(ctx, both, stream.x[:n])
        stream.pending, stream.pending_slabs, stream.pending_norm = None, 0, None


register_part("reentry", "concat_linear", ConcatLinearReentry)
