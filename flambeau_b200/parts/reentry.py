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
    is added to the stream first (through the norm it is pending with, or plainly where it has none).  The operands
    are rounded to the engine's dtype for the product; the result is the float32 stream.  With `step_name`, a tensor
    [passes, width] of that name holds one learned vector per pass, which is added to every token's stream after the
    map (float32)."""
    graph_safe = True
    category = "reentry"

    def __init__(self, runtime=None, prefix="", *, width: int, weight_name: str = "weight", init_std: float = 0.02,
                 step_name: str | None = None, passes: int = 0):
        super().__init__(runtime, prefix)
        self.width, self.weight_name, self.init_std = int(width), weight_name, init_std
        self.step_name, self.passes = step_name, int(passes)
        if step_name is not None and self.passes < 1:
            raise ValueError("a vector per pass needs the number of passes")
        self.map = None
        self.steps = None

    def own_tensor_specs(self):
        specs = {self.prefix + self.weight_name: TensorSpec((self.width, 2 * self.width), init=("normal", self.init_std))}
        if self.step_name is not None:
            specs[self.prefix + self.step_name] = TensorSpec((self.passes, self.width), init=("normal", 0.1))
        return specs

    def own_bind(self, tensors):
        self.map = Linear(tensors[self.prefix + self.weight_name])
        if self.step_name is not None:
            self.steps = tensors[self.prefix + self.step_name].contiguous()

    def own_weights(self):
        return [self.map.weight]

    def forward(self, ctx, stream, x0, pass_index: int = 0) -> None:
        n = ctx.n_tokens
        stream.settle(ctx)
        with ctx.ws.scope():
            both = ctx.ws.alloc((n, 2 * self.width), self.runtime.dtype)
            ops.concat_cast(stream.x[:n], x0[:n], both)
            self.map(ctx, both, stream.x[:n])
        if self.steps is not None:
            if not 0 <= pass_index < self.passes:
                raise ValueError(f"pass {pass_index} of a stretch that has vectors for {self.passes} passes")
            ops.add_row(stream.x[:n], self.steps[pass_index])
        stream.pending, stream.pending_slabs, stream.pending_norm = None, 0, None


register_part("reentry", "concat_linear", ConcatLinearReentry)
