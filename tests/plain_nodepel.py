"""A plain, slow implementation of the Nodepel design in float64 torch on the CPU: the oracle of the tests.

One function per mechanism; whole sequences only (no cache, no state slots, no batches, no portions), so that
whatever the engine does with pages, slots and schedules is compared with something that has none of them.  It shares
no code with the product path.  `cfg` is the parsed config.json (a dict); `w` maps tensor names to float64 tensors.

Notation: n tokens, D = width.  Softmax side of a mixer: H query heads on G key/value heads, d = query/key size,
e = value size, R = rotated dimensions, W = window.  Recurrent side: Hr value heads on Gr query/key heads, dr = key
size, er = value size, T = taps of the short convolution.  Feed-forward: E experts of which each token uses K.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64

# How much of a difference is rounding?  With `rounding_to(torch.bfloat16)` active, the values that a bfloat16 engine
# may keep in 16 bits (normalised rows, q, k, v, the heads' outputs, activations) are rounded to that type on their
# way; the distance between such a run and the exact one is the noise that rounding alone causes, from which the
# tests take their bfloat16 tolerance.  Without it nothing is rounded.
_ROUND = [None]


class rounding_to:
    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        _ROUND[0] = self.dtype

    def __exit__(self, *exc):
        _ROUND[0] = None


def kept(x):
    return x if _ROUND[0] is None else x.to(_ROUND[0]).to(F64)


# ---- small mechanisms -------------------------------------------------------------------------------------------
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return unit_rms(x, eps) * (1.0 + weight)


def plain_norm(x, weight, eps):
    """RMS norm with the weight as it is stored."""
    return unit_rms(x, eps) * weight


def embed(tokens, table, scale):
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


# ---- the softmax side ----------------------------------------------------------------------------------------------
def rotate_half(x, positions, base, dims):
    """x [n, heads, d]: dimension i < dims/2 of every head is paired with dimension i + dims/2 and the pair turned by
    the angle position * base^(-2i/dims); dimensions from `dims` on pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    ang = torch.as_tensor(positions, dtype=F64)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def window_mask(n, size):
    """[n, n] bool: query i sees key j when 0 <= i - j < size."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (i - j >= 0) & (i - j < size)


def sink_softmax(scores, mask, sink):
    """Softmax over the seen keys whose denominator also holds exp(sink): a slot without key and value."""
    s = scores.masked_fill(~mask, -math.inf)
    m = torch.maximum(s.max(dim=-1, keepdim=True).values, torch.as_tensor(sink, dtype=F64))
    p = torch.exp(s - m)
    return p / (p.sum(dim=-1, keepdim=True) + torch.exp(sink - m))


def windowed_attention(h, w, p, m, eps):
    """The left mixer.  h [n, D] at positions 0 .. n-1."""
    n = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = plain_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).view(n, H, d)          # the norm spans the whole projection
    k = plain_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).view(n, G, d)
    v = (h @ w[p + "v"].T).view(n, G, e)
    pos = list(range(n))
    q = kept(rotate_half(q, pos, m["rot"]["base"], m["rot"]["dims"]))
    k = kept(rotate_half(k, pos, m["rot"]["base"], m["rot"]["dims"]))
    v = kept(v)
    mask = window_mask(n, m["mask"]["size"])
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        a = sink_softmax((q[:, hh] @ k[:, g].T) * m["scale"], mask, w[p + "sink"][hh])
        heads.append(a @ v[:, g])
    return kept(torch.cat(heads, dim=-1)) @ w[p + "o"].T


# ---- the recurrent side ----------------------------------------------------------------------------------------------
def short_convolution(x, taps):
    """x [n, C], taps [C, T]: y[t, c] = sum_j taps[c, j] * x[t - (T-1) + j, c], zeros before the start."""
    n, C = x.shape
    T = taps.shape[1]
    padded = torch.cat([torch.zeros(T - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(T):
        y = y + padded[j:j + n] * taps[:, j][None, :]
    return y


def unit_vector(x):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, decay):
    """One head: q, k [n, dr], v [n, er], beta and decay [n].  The state S [dr, er] starts at zero; for each token
    S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    n, dr = q.shape
    S = torch.zeros(dr, v.shape[1], dtype=F64)
    out = []
    for t in range(n):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out)


def gated_delta(h, w, p, m, eps):
    """The right mixer."""
    n = h.shape[0]
    Hr, Gr, dr, er = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).view(n, Gr, dr)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).view(n, Gr, dr)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).view(n, Hr, er)
    q = unit_vector(q) * dr ** -0.5
    k = unit_vector(k)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                          # [n, Hr]
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :] * softplus(h @ w[p + "a"].T + w[p + "dt_bias"][None, :]))
    gate = silu(h @ w[p + "g"].T).view(n, Hr, er)
    heads = []
    for hh in range(Hr):
        g = hh // (Hr // Gr)
        o = delta_rule(q[:, g], k[:, g], v[:, hh], beta[:, hh], decay[:, hh])
        heads.append(plain_norm(o, w[p + "norm"], eps) * gate[:, hh])
    return kept(torch.cat(heads, dim=-1)) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    """Both sides read h; each output passes an RMS norm over the width with a plain weight; half their sum."""
    left = plain_norm(windowed_attention(h, w, p + "left.", m["left"], eps), w[p + "left.out"], eps)
    right = plain_norm(gated_delta(h, w, p + "right.", m["right"], eps), w[p + "right.out"], eps)
    return 0.5 * (left + right)


# ---- the feed-forward ------------------------------------------------------------------------------------------------
def expert(h, w, p):
    return kept(relu_squared(h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_experts(h, w, p, mlp):
    n = h.shape[0]
    E, K = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"][None, :]
    out = torch.zeros(n, w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(n):
        chosen = torch.argsort(z[t], descending=True, stable=True)[:K]
        share = torch.softmax(z[t][chosen], dim=0)
        for c, s in zip(chosen.tolist(), share):
            out[t] += s * expert(h[t:t + 1], w, f"{p}e{c}.")[0]
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * expert(h, w, p + "shared.")
    return out


# ---- the model ---------------------------------------------------------------------------------------------------
def run_order(cfg):
    """(layer, pass number or None) in the order they run; the pass number is given at the first layer of a pass."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, layer_outputs=None):
    """Logits [n, vocab] of one whole sequence; `layer_outputs` (a list) receives the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x0 = embed(tokens, w["embed"], cfg["embedding"]["scale"])
    x = x0
    for i, start_of_pass in run_order(cfg):
        if start_of_pass is not None:
            x = kept(torch.cat([x, x0], dim=-1)) @ w["loop.in"].T + w["loop.step"][start_of_pass][None, :]
        L, p = cfg["layers"][i], f"l{i}."
        x = x + parallel_mixer(kept(offset_norm(x, w[p + "norm1"], eps)), w, p + "mix.", L["mixer"], eps)
        if L.get("mlp") is not None:
            x = x + routed_experts(kept(offset_norm(x, w[p + "norm2"], eps)), w, p + "mlp.", L["mlp"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return kept(offset_norm(x, w["final.norm"], eps)) @ w["head"].T


def rounding_noise(cfg, w, tokens, dtype=torch.bfloat16):
    """Per position, the largest difference between the logits with the 16-bit values rounded and the exact ones, as a
    fraction of the largest exact logit: (the largest over the positions, their median)."""
    exact = forward(cfg, w, tokens)
    with rounding_to(dtype):
        rounded = forward(cfg, w, tokens)
    per_row = (rounded - exact).abs().max(dim=1).values / exact.abs().max()
    return float(per_row.max()), float(per_row.median())


# ---- a safetensors reader of its own -----------------------------------------------------------------------------------
def read_safetensors(path) -> dict:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = raw[8 + n + lo:8 + n + hi]
        if meta["dtype"] == "BF16":
            a = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif meta["dtype"] == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif meta["dtype"] == "I32":
            a = np.frombuffer(buf, dtype="<i4").astype(np.float64)
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = torch.from_numpy(a.reshape(meta["shape"]).copy())
    return out


def load_folder(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")
