"""A plain, slow implementation of the Zedivik design in float64 torch on the CPU: the oracle of the tests.

One function per mechanism; whole sequences only (no cache, no batches, no portions), so that whatever the engine
does with pages, slots and schedules is compared with something that has none of them.  It shares no code with
the product path.  `cfg` is the parsed config.json (a dict); `w` maps tensor names to float64 tensors.

Notation: n tokens, D = width, H query heads, G key/value heads, d = per-map query/key size, e = value size.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


# ---- small mechanisms -------------------------------------------------------------------------------------------
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """RMS norm whose stored weight is the deviation from one: unit_rms(x) * (1 + weight)."""
    return unit_rms(x, eps) * (1.0 + weight)


def embed(tokens, table, scale):
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


def silu(z):
    return z * torch.sigmoid(z)


def dense_ff(h, w, p):
    """down(silu(gate h) * (up h))."""
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def window_mask(positions, n_keys, size):
    """[queries, n_keys] bool: the query at position p sees key j when 0 <= p - j < size (size 0: every j <= p)."""
    i = torch.as_tensor(positions, dtype=torch.long)[:, None]
    j = torch.arange(n_keys)[None, :]
    seen = i - j >= 0
    return seen & (i - j < size) if size else seen


def softmax_map(q, k, v, scale, mask):
    """One attention map: q [n, d], k [n, d], v [n, e]."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~mask, -math.inf)
    return torch.softmax(s, dim=-1) @ v


def lambda_of(w, p, diff):
    return math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) + diff


def diff_heads(q, k, v, gate, positions, *, scale, window, lam, diff, eps):
    """The heads' outputs, concatenated: q [n, H, 2, d] for queries at `positions`, k [T, G, 2, d] and v [T, G, e]
    for the keys at 0 .. T-1, gate [n, H] or None.  Returns [n, H * e]."""
    H, G = q.shape[1], k.shape[1]
    mask = window_mask(positions, k.shape[0], window)
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        a1 = softmax_map(q[:, hh, 0], k[:, g, 0], v[:, g], scale, mask)
        a2 = softmax_map(q[:, hh, 1], k[:, g, 1], v[:, g], scale, mask)
        o = unit_rms(a1 - lam * a2, eps) * (1.0 - diff)
        heads.append(o if gate is None else o * gate[:, hh:hh + 1])
    return torch.cat(heads, dim=-1)


def differential_attention(h, w, p, m, eps):
    """The attention mixer: two softmax maps per head over shared values, their difference normalised per head,
    gated per head, projected.  h [n, D]; m = the layer's 'mixer' object of the configuration."""
    n = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(n, H, 2, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(n, G, 2, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(n, G, e)
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [n, H]
    o = diff_heads(q, k, v, gate, range(n), scale=m["scale"], window=m["mask"]["size"],
                   lam=lambda_of(w, p, m["diff"]), diff=m["diff"], eps=eps)
    return o @ w[p + "o"].T


# ---- the model ----------------------------------------------------------------------------------------------------
def layer(x, w, i, spec, eps):
    """x + norm1b(mixer(norm1 x)), then x + norm2b(ff(norm2 x)) where the layer has a feed-forward."""
    p = f"l{i}."
    if spec["type"] != "attention":
        raise ValueError(f"layer type {spec['type']!r}")
    a = differential_attention(offset_norm(x, w[p + "norm1"], eps), w, p + "mix.", spec["mixer"], eps)
    x = x + offset_norm(a, w[p + "norm1b"], eps)
    if spec.get("mlp") is not None:
        if spec["mlp"]["kind"] != "dense":
            raise ValueError(f"feed-forward kind {spec['mlp']['kind']!r}")
        f = dense_ff(offset_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        x = x + offset_norm(f, w[p + "norm2b"], eps)
    return x


def layer_runs(cfg):
    """[(layer index, first of a pass)] in run order: layers before the loop, the looped layers `times` times, the rest."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        runs += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, return_layers=False):
    """Logits [n, vocab] for one whole sequence (and the stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x0 = embed(tokens, w["embed"], cfg["embedding"]["scale"])
    x = x0
    streams = []
    for i, first in layer_runs(cfg):
        if first:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        x = layer(x, w, i, cfg["layers"][i], eps)
        streams.append(x)
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits


# ---- reading a model folder (a parser of its own: 8-byte length, JSON header, data) ----------------------------
def read_folder(folder):
    """(config dict, {name: float64 tensor})."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = np.frombuffer(raw, dtype=np.uint8, count=b - a, offset=8 + n + a)
        if info["dtype"] == "BF16":
            t = torch.from_numpy((buf.view(np.uint16).astype(np.uint32) << 16).view(np.float32).copy())
        elif info["dtype"] == "F32":
            t = torch.from_numpy(buf.view(np.float32).copy())
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        out[name] = t.to(F64).view(info["shape"])
    return cfg, out


def argmax_lowest(row):
    """The lowest index among the largest entries."""
    return int((row == row.max()).nonzero()[0])
