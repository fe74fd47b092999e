"""Differential attention over the paged cache."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import KVRequirement, Mixer, TensorSpec
from .linear import Linear, concat_rows
from .spec import register_part


class DifferentialAttention(Mixer):
    """Every head has two softmax maps over the same values, and the head's output is their difference:

        q = Wq h + bq   [H][2][kd]      k = Wk h + bk   [G][2][kd]      v = Wv h + bv   [G][vd]
        a_m = softmax_j(scale * q_m . k_m[j]) v[j]     over the keys j with 0 <= p - j < window   (m = 1, 2)
        lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff                  (one number for the layer)
        o = a_1 - lambda * a_2;   o <- o / sqrt(mean(o^2) + eps) * (1 - diff)       (per head, no weight)
        o <- o * sigmoid(Wg h)_head                                      (with `head_gate`)
        out = Wo [o_0 ; ... ; o_{H-1}]

    Query head h reads key/value head h // (H / G).  No position enters the scores.  kd (`key_dim`, per map) and vd
    (`value_dim`) are independent; the cache keeps both maps of a key side by side (rows of 2 * kd) and values in
    rows of vd.  Scores, softmax weights, weighted sums, lambda, the difference and the head norm are float32 in
    both engine modes; q, k, v and the head outputs are rounded to the engine's dtype once each.

    The four input maps are stacked into one product; the kernel behind it adds the biases, fills the cache and
    forms the gate.  Tensors behind the prefix: q, q.b, k, k.b, v, v.b (biases with `bias`), lq1, lk1, lq2, lk2,
    g (with `head_gate`), o."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, num_heads: int, num_kv_heads: int, key_dim: int,
                 value_dim: int, window: int = 0, scale: float | None = None, diff: float = 0.0, eps: float = 1e-6,
                 bias: bool = True, head_gate: bool = True, init_std: float = 0.02):
        super().__init__(runtime, prefix)
        self.width, self.nh, self.nkv = int(width), int(num_heads), int(num_kv_heads)
        self.kd, self.vd = int(key_dim), int(value_dim)
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} query heads are not a multiple of {self.nkv} key/value heads")
        self.window = int(window or 0)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.kd)
        self.diff, self.eps = float(diff), float(eps)
        self.bias, self.head_gate, self.init_std = bool(bias), bool(head_gate), init_std
        self.qw, self.kw, self.vw = self.nh * 2 * self.kd, self.nkv * 2 * self.kd, self.nkv * self.vd
        self.n_gate = self.nh if self.head_gate else 0
        self.proj = self.o = self.proj_bias = None
        self.lam = None

    def cache_requirement(self):
        return KVRequirement(self.nkv, 2 * self.kd, self.window, v_head_dim=self.vd)

    def own_tensor_specs(self):
        p, init = self.prefix, ("normal", self.init_std)
        specs = {
            p + "q": TensorSpec((self.qw, self.width), init=init),
            p + "k": TensorSpec((self.kw, self.width), init=init),
            p + "v": TensorSpec((self.vw, self.width), init=init),
            p + "o": TensorSpec((self.width, self.nh * self.vd), init=init),
        }
        for name in ("lq1", "lk1", "lq2", "lk2"):
            specs[p + name] = TensorSpec((self.kd,), init=("normal", 0.1))
        if self.bias:
            specs[p + "q.b"] = TensorSpec((self.qw,), init=init)
            specs[p + "k.b"] = TensorSpec((self.kw,), init=init)
            specs[p + "v.b"] = TensorSpec((self.vw,), init=init)
        if self.head_gate:
            specs[p + "g"] = TensorSpec((self.nh, self.width), init=init)
        return specs

    def own_bind(self, tensors):
        p = self.prefix
        stack = [tensors[p + "q"], tensors[p + "k"], tensors[p + "v"]]
        if self.head_gate:
            stack.append(tensors[p + "g"])
        rows = sum(t.shape[0] for t in stack)
        if rows % 8:          # rows of zeros up to a multiple of 8, so that the product's float32 rows stay 16-byte aligned
            stack.append(torch.zeros((8 - rows % 8, self.width), dtype=stack[0].dtype, device=stack[0].device))
        self.proj = Linear(concat_rows(stack))
        self.o = Linear(tensors[p + "o"])
        self.proj_bias = torch.cat([tensors[p + "q.b"], tensors[p + "k.b"], tensors[p + "v.b"]]).contiguous() \
            if self.bias else None

        def dot(a, b):
            return float((tensors[p + a].double() * tensors[p + b].double()).sum())
        self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + self.diff

    def own_weights(self):
        return [self.proj.weight, self.o.weight] + ([self.proj_bias] if self.bias else [])

    def forward(self, ctx, h, out, call):
        n = ctx.n_tokens
        rt, b = self.runtime, ctx.batch
        cache = ctx.cache(call)
        cols = self.proj.out_features                 # q, k, v and gate columns, and the padding behind them
        with ctx.ws.scope():
            slabs = ctx.ws.alloc((ctx.max_slabs, n, cols), torch.float32)
            parts = self.proj.slabs(ctx, h, slabs)
            q = ctx.ws.alloc((n, self.qw), rt.dtype)
            gate = ctx.ws.alloc((n, self.nh), torch.float32) if self.head_gate else None
            ops.qkv_bias_cache_write(slabs[0], self.proj_bias, q, gate, cache, b.positions, b.row_seq, self.nh,
                                     self.nkv, 2 * self.kd, self.vd, self.n_gate, rt.status, n_partials=parts,
                                     partial_stride=slabs.stride(0))
            a = ctx.ws.alloc((n, self.nh * self.vd), rt.dtype)
            ops.diff_attention(ctx, q, a, gate, cache, self.nh, self.nkv, self.kd, self.vd, self.window, self.scale,
                               self.lam, self.eps, 1.0 - self.diff)
            ctx.to_stream(self.o, a)


register_part("mixer", "diff_attention", DifferentialAttention)
