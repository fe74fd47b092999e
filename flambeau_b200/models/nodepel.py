"""Nodepel: configuration -> ModelSpec.

A decoder of pre-norm blocks ("1 + w" RMS norms) whose mixer is two mixers side by side on the same input: softmax
attention under a sliding window (grouped heads, an RMS norm over the whole q and the whole k projection, rotary
positions on part of a head, a learned sink in every head's softmax) and a gated delta rule (short convolutions, a
float32 matrix of state per head); each side's output passes an RMS norm of its own and the two are averaged.  The
feed-forward, where a layer has one, is a mixture of experts (squared-ReLU experts, softmax over the chosen logits)
plus a shared expert behind a sigmoid gate per token.  The embedding is scaled.  A stretch of layers
[loop.start, loop.stop) runs loop.times times in a row on the same weights, every pass with a cache and state of its
own; at the start of every pass the stream is replaced by a linear map of [stream ; embedding output] (`loop.in`)
plus the pass's learned vector (`loop.step`).  Tensor names are the checkpoint's: embed, loop.in, loop.step,
l<i>.norm1 / norm2, l<i>.mix.left.*, l<i>.mix.right.*, l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

from ..config.nodepel import ARCHITECTURE, NodepelConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, ModelSpec, PartSpec

NORM_INIT = ("normal", 0.1)          # the stored weight is the deviation from one
LEFT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}


def build_spec(cfg: NodepelConfig) -> ModelSpec:
    D = cfg.width

    def norm(prefix, name):
        return PartSpec("norm", "rmsnorm", dict(width=D, eps=cfg.norm_eps, init=NORM_INIT, weight_offset=1.0,
                                                weight_name=name), prefix)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        a, r = layer.mixer.left, layer.mixer.right
        left = PartSpec("mixer", "attention", dict(
            width=D, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, value_dim=a.vdim, window=a.window,
            scale=a.scale, sink=True, names=LEFT_NAMES, qk_norm_reach="projection", weights_float32=True,
            qk_norm=PartSpec("norm", "rmsnorm", dict(width=a.dim, eps=cfg.norm_eps, init=("one_plus_normal", 0.1))),
            position=PartSpec("position", "rotary_half", dict(head_dim=a.dim, theta=a.rot_base, rotary_dim=a.rot_dims))
            if a.rot_dims else None), p + "mix.left.")
        right = PartSpec("mixer", "gated_delta", dict(
            width=D, num_heads=r.heads, num_qk_heads=r.kv_heads, key_dim=r.dim, value_dim=r.vdim, conv=r.conv,
            eps=cfg.norm_eps, unit_eps=1e-6), p + "mix.right.")
        mixer = PartSpec("mixer", "parallel", dict(width=D, branches=[left, right], out_names=["left.out", "right.out"],
                                                   eps=cfg.norm_eps, coefs=[0.5, 0.5]), p + "mix.")
        params = dict(mixer=mixer, mixer_norm=norm(p, "norm1"))
        if layer.mlp is not None:
            m = layer.mlp
            params.update(
                feed_forward=PartSpec("feed_forward", "routed_experts", dict(
                    width=D, inner=m.ff, experts=m.experts, top=m.top, activation="relu_squared",
                    shared_inner=m.shared_ff), p + "mlp."),
                feed_forward_norm=norm(p, "norm2"))
        layers.append(PartSpec("block", "pre_norm", params, p))

    n = len(cfg.layers)
    reentry = None
    if cfg.loop is None:
        order = [LayerCall(i) for i in range(n)]
    else:
        lp = cfg.loop
        order = [LayerCall(i) for i in range(lp.start)]
        for t in range(lp.times):
            order += [LayerCall(i, reenter=(i == lp.start), pass_index=t) for i in range(lp.start, lp.stop)]
        order += [LayerCall(i) for i in range(lp.stop, n)]
        reentry = PartSpec("reentry", "concat_linear", dict(width=D, weight_name="in", step_name="step",
                                                            passes=lp.times), "loop.")
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab=cfg.vocab, width=D, scale=cfg.embedding_scale,
                                                                weight_name="embed"), ""),
        layers=layers, order=order, final_norm=norm("final.", "norm"),
        head=PartSpec("head", "lm_head", dict(vocab=cfg.vocab, width=D, weight_name="head"), ""),
        reentry=reentry)


register_architecture(ARCHITECTURE, NodepelConfig, build_spec, replace=True)
