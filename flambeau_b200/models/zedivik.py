"""Zedivik: configuration -> ModelSpec.

A decoder of blocks with a norm before and behind each sublayer ("1 + w" RMS norms), whose mixer is differential
attention under a sliding window (no position encoding) and whose feed-forward, where a layer has one, is
SiLU-gated.  The embedding is scaled.  A stretch of layers [loop.start, loop.stop) runs loop.times times in a row
on the same weights, every pass with a cache of its own, and at the start of every pass the stream is replaced by
a linear map of [stream ; embedding output] (`loop.in`).  Every layer carries its own sizes and constants, so the
layers of one model may differ in all of them.  Tensor names are the checkpoint's: embed, loop.in,
l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.mix.*, l<i>.mlp.gate / up / down, final.norm, head.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zedivik import ARCHITECTURE, ZedivikConfig
from ..parts.spec import LayerCall, ModelSpec, PartSpec

NORM_INIT = ("normal", 0.1)          # the stored weight is the deviation from one


def build_spec(cfg: ZedivikConfig) -> ModelSpec:
    D = cfg.width

    def norm(prefix, name):
        return PartSpec("norm", "rmsnorm", dict(width=D, eps=cfg.norm_eps, init=NORM_INIT, weight_offset=1.0,
                                                weight_name=name), prefix)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        mixer = PartSpec("mixer", "diff_attention", dict(
            width=D, num_heads=m.heads, num_kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim, window=m.window,
            scale=m.scale, diff=m.diff, eps=cfg.norm_eps, bias=True, head_gate=True), p + "mix.")
        params = dict(mixer=mixer, mixer_norm=norm(p, "norm1"), mixer_post_norm=norm(p, "norm1b"))
        if layer.mlp is not None:
            params.update(
                feed_forward=PartSpec("feed_forward", "gated_mlp", dict(
                    width=D, inner=layer.mlp.ff, activation="silu", names=("gate", "up", "down")), p + "mlp."),
                feed_forward_norm=norm(p, "norm2"), feed_forward_post_norm=norm(p, "norm2b"))
        layers.append(PartSpec("block", "sandwich_norm", params, p))

    n = len(cfg.layers)
    reentry = None
    if cfg.loop is None:
        order = [LayerCall(i) for i in range(n)]
    else:
        lp = cfg.loop
        order = [LayerCall(i) for i in range(lp.start)]
        for _ in range(lp.times):
            order += [LayerCall(i, reenter=(i == lp.start)) for i in range(lp.start, lp.stop)]
        order += [LayerCall(i) for i in range(lp.stop, n)]
        reentry = PartSpec("reentry", "concat_linear", dict(width=D, weight_name="in"), "loop.")
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab=cfg.vocab, width=D, scale=cfg.embedding_scale,
                                                                weight_name="embed"), ""),
        layers=layers, order=order, final_norm=norm("final.", "norm"),
        head=PartSpec("head", "lm_head", dict(vocab=cfg.vocab, width=D, weight_name="head"), ""),
        reentry=reentry)


register_architecture(ARCHITECTURE, ZedivikConfig, build_spec, replace=True)
