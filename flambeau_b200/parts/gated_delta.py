"""The gated delta rule: a recurrent mixer with a matrix of state per head."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, StateRequirement, TensorSpec
from .linear import Linear, concat_rows
from .spec import register_part


class GatedDeltaRule(Mixer):
    """A linear recurrence over a request's tokens.  With H value heads on G query/key heads (head h reads q/k head
    h // (H / G)), key size dk and value size dv:

        q = Wq x, k = Wk x  [G][dk];   v = Wv x  [H][dv]                          (no biases)
        each channel of q, k and v passes a causal convolution over the last `conv` tokens (its own taps, the last
        tap is the current token's, zeros before the request's start) and then SiLU
        q <- q / sqrt(sum q^2 + unit_eps) * dk^-1/2,  k <- k / sqrt(sum k^2 + unit_eps)        (per head)
        beta = sigmoid(Wb x)  [H];     g = exp(-exp(A_log) * softplus(Wa x + dt_bias))  [H]
        per head, token by token:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
        o <- o / sqrt(mean(o^2) + eps) * norm * silu(Wg x)_head                    (norm [dv] shared by the heads)
        out = Wo [o_0 ; ... ; o_{H-1}]

    S [dk, dv] starts at zero and is carried from step to step in float32, as are the last conv - 1 inputs of the
    convolution: both live in the request's state slot (one float32 array: S for every head, then the tail).  Decays,
    beta, the unit norms, the recurrence and the head norm are float32 in both engine modes.

    The six input maps are one stacked product.  Tensors behind the prefix: q, q.conv, k, k.conv, v, v.conv
    ([channels, conv]), b, a ([H, width]), A_log, dt_bias ([H]), g, norm ([dv]), o."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, num_heads: int, num_qk_heads: int, key_dim: int,
                 value_dim: int, conv: int = 4, eps: float = 1e-6, unit_eps: float = 1e-6, init_std: float = 0.02):
        super().__init__(runtime, prefix)
        self.width, self.H, self.G = int(width), int(num_heads), int(num_qk_heads)
        self.dk, self.dv, self.taps = int(key_dim), int(value_dim), int(conv)
        if self.H % self.G:
            raise ValueError(f"{self.H} value heads are not a multiple of {self.G} query/key heads")
        if self.taps < 1:
            raise ValueError("the short convolution needs at least one tap")
        self.eps, self.unit_eps, self.init_std = float(eps), float(unit_eps), init_std
        self.qk, self.vw = self.G * self.dk, self.H * self.dv
        self.channels = 2 * self.qk + self.vw                    # what passes the convolution
        self.state_floats = self.H * self.dk * self.dv
        self.tail_floats = (self.taps - 1) * self.channels
        self.proj = self.o = self.conv_w = self.a_log = self.dt_bias = self.norm = None

    def state_requirement(self):
        return StateRequirement((self.state_floats + self.tail_floats,), "float32")

    def own_tensor_specs(self):
        p, init = self.prefix, ("normal", self.init_std)
        conv_init = ("normal", 0.5 / max(1, self.taps) ** 0.5)
        return {
            p + "q": TensorSpec((self.qk, self.width), init=init),
            p + "q.conv": TensorSpec((self.qk, self.taps), init=conv_init),
            p + "k": TensorSpec((self.qk, self.width), init=init),
            p + "k.conv": TensorSpec((self.qk, self.taps), init=conv_init),
            p + "v": TensorSpec((self.vw, self.width), init=init),
            p + "v.conv": TensorSpec((self.vw, self.taps), init=conv_init),
            p + "b": TensorSpec((self.H, self.width), init=init),
            p + "a": TensorSpec((self.H, self.width), init=init),
            p + "A_log": TensorSpec((self.H,), init=("normal", 0.5)),
            p + "dt_bias": TensorSpec((self.H,), init=("normal", 0.5)),
            p + "g": TensorSpec((self.vw, self.width), init=init),
            p + "norm": TensorSpec((self.dv,), init=("one_plus_normal", 0.1)),
            p + "o": TensorSpec((self.width, self.vw), init=init),
        }

    def own_bind(self, tensors):
        p = self.prefix
        stack = [tensors[p + n] for n in ("q", "k", "v", "b", "a", "g")]
        rows = sum(t.shape[0] for t in stack)
        if rows % 8:          # rows of zeros up to a multiple of 8, so that the product's float32 rows stay 16-byte aligned
            stack.append(torch.zeros((8 - rows % 8, self.width), dtype=stack[0].dtype, device=stack[0].device))
        self.proj = Linear(concat_rows(stack))
        self.o = Linear(tensors[p + "o"])
        self.conv_w = torch.cat([tensors[p + "q.conv"], tensors[p + "k.conv"], tensors[p + "v.conv"]]).contiguous()
        dt = self.conv_w.dtype
        self.a_log, self.dt_bias = tensors[p + "A_log"].to(dt).contiguous(), tensors[p + "dt_bias"].to(dt).contiguous()
        self.norm = tensors[p + "norm"]

    def own_weights(self):
        return [self.proj.weight, self.o.weight, self.conv_w]

    def forward(self, ctx, h, out, call):
        n = ctx.n_tokens
        rt, b = self.runtime, ctx.batch
        state = ctx.cache(call).state
        if state is None:
            raise ValueError("the gated delta rule needs a state slot per request")
        state = state.view(state.shape[0], -1)
        with ctx.ws.scope():
            slabs = ctx.ws.alloc((ctx.max_slabs, n, self.proj.out_features), torch.float32)
            parts = self.proj.slabs(ctx, h, slabs)
            stride = slabs.stride(0)
            qkv = ctx.ws.alloc((n, self.channels), torch.float32)
            beta = ctx.ws.alloc((n, self.H), torch.float32)
            decay = ctx.ws.alloc((n, self.H), torch.float32)
            ops.gdr_prepare(slabs[0], self.conv_w, self.taps, self.a_log, self.dt_bias, state, self.state_floats, b,
                            qkv, beta, decay, self.G, self.H, self.dk, self.dv, self.dk ** -0.5, self.unit_eps,
                            n_partials=parts, partial_stride=stride)
            o = ctx.ws.alloc((n, self.vw), torch.float32)
            ops.gdr_recurrent(qkv, beta, decay, state, b, o, self.G, self.H, self.dk, self.dv)
            a = ctx.ws.alloc((n, self.vw), rt.dtype)
            ops.gdr_out_norm(o, slabs[0], self.channels + 2 * self.H, self.norm, self.eps, a, self.H, self.dv,
                             n_partials=parts, partial_stride=stride)
            ctx.to_stream(self.o, a)


register_part("mixer", "gated_delta", GatedDeltaRule)
