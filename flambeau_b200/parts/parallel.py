"""Mixers that run side by side on one input."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, TensorSpec
from .spec import PartSpec, build_part, register_part


class ParallelMixers(Mixer):
    """out = sum_b coef_b * rmsnorm(mixer_b(h)) * w_b: every branch reads the same input, its output passes an RMS
    norm over the model width with a plain weight of its own (`<prefix><out_names[b]>`), and the results are mixed
    with fixed factors (default: their mean).  At most one branch may keep keys and values and at most one a
    fixed-size state, since a layer call owns one cache and one state slot.

    The branches leave their outputs as float32 (split-K shares of their last products where those leave shares);
    one kernel adds the shares, normalises and mixes."""
    graph_safe = True
    MAX_BRANCHES = 4

    def __init__(self, runtime=None, prefix="", *, width: int, branches, out_names, eps: float, coefs=None,
                 out_init=("one_plus_normal", 0.1)):
        super().__init__(runtime, prefix)
        self.width, self.eps = int(width), float(eps)
        self.branches = [build_part(b, runtime) for b in branches]
        if not 1 <= len(self.branches) <= self.MAX_BRANCHES:
            raise ValueError(f"{len(self.branches)} branches; 1 to {self.MAX_BRANCHES} can run side by side")
        self.out_names = list(out_names)
        if len(self.out_names) != len(self.branches):
            raise ValueError("one output norm per branch wanted")
        self.coefs = [float(c) for c in coefs] if coefs is not None else [1.0 / len(self.branches)] * len(self.branches)
        if len(self.coefs) != len(self.branches):
            raise ValueError("one factor per branch wanted")
        if sum(b.cache_requirement() is not None for b in self.branches) > 1 or \
                sum(b.state_requirement() is not None for b in self.branches) > 1:
            raise ValueError("side by side, at most one mixer may keep keys and values and at most one a state")
        self.out_init = tuple(out_init)
        self.out_weights = None

    def children(self):
        return list(self.branches)

    def cache_requirement(self):
        return next((r for r in (b.cache_requirement() for b in self.branches) if r is not None), None)

    def state_requirement(self):
        return next((r for r in (b.state_requirement() for b in self.branches) if r is not None), None)

    def own_tensor_specs(self):
        return {self.prefix + name: TensorSpec((self.width,), init=self.out_init) for name in self.out_names}

    def own_bind(self, tensors):
        self.out_weights = [tensors[self.prefix + name] for name in self.out_names]

    def own_weights(self):
        return list(self.out_weights)

    def forward(self, ctx, h, out, call):
        n = ctx.n_tokens
        # a branch's output has to pass its norm before it may join the stream: no product adds to the stream here
        kept = (ctx.stream_x, ctx.delta_slabs, ctx.delta)
        ctx.stream_x = None
        try:
            with ctx.ws.scope():
                mix = []
                for branch, weight, coef in zip(self.branches, self.out_weights, self.coefs):
                    y = ctx.ws.alloc((ctx.max_slabs, n, self.width), torch.float32)
                    ctx.delta_slabs, ctx.delta = y, y[0]
                    ctx.pending_slabs = 1
                    branch.forward(ctx, h, y[0], call)
                    mix.append((y[0], max(1, ctx.pending_slabs), y.stride(0), weight, coef))
                ops.branch_norm_mix(mix, self.eps, out, n)
        finally:
            ctx.stream_x, ctx.delta_slabs, ctx.delta = kept
        ctx.pending_slabs = 1


register_part("mixer", "parallel", ParallelMixers)
