"""Tiny Nodepel configurations and model folders shared by the tests.

Three configurations that differ from each other in every size and option:
  NA: width 64, vocab 200, embedding scale 2, eps 1e-5; three layers whose softmax sides have 4/2, 2/2 and 6/1 heads,
      key sizes 16, 32, 16, value sizes 32, 16, 16, windows 20, 7, 33, 8, 32 and 16 rotated dimensions, and whose
      recurrent sides have 4/2, 2/1 and 3/3 heads, key sizes 8, 16, 24, value sizes 16, 24, 8 and 4, 3 and 2 taps; the
      second layer has no feed-forward, the third routes every token to one of four experts and has no shared
      expert; layers 0-1 run twice
  NB: width 96, vocab 320, embedding scale 1, eps 1e-6; four layers, among them a window of one key, a key size that
      is no multiple of 8 (20) with 4 rotated dimensions, a window longer than any request, 20 query heads on one
      key/value head, a convolution of one tap (no tail), 40 experts of which a token uses 5; layer 2 alone runs
      three times
  NC: two layers, no loop at all
"""
from __future__ import annotations

from pathlib import Path

import torch


def layer(left, right, mlp):
    h, g, d, e, w, base, dims, scale = left
    H, G, dk, dv, conv = right
    m = None
    if mlp is not None:
        experts, top, ff, shared = mlp
        m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
        if shared:
            m["shared"] = {"ff": shared}
    return {"type": "parallel",
            "mixer": {"left": {"heads": h, "kv_heads": g, "dim": d, "vdim": e, "mask": {"size": w},
                               "rot": {"base": base, "dims": dims}, "scale": scale},
                      "right": {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "conv": conv}},
            "mlp": m}


CONFIG_NA = {"architecture": "Nodepel", "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5}, "vocab": 200, "width": 64,
             "layers": [layer((4, 2, 16, 32, 20, 10000.0, 8, 0.3), (4, 2, 8, 16, 4), (6, 2, 24, 40)),
                        layer((2, 2, 32, 16, 7, 500.0, 32, 0.2), (2, 1, 16, 24, 3), None),
                        layer((6, 1, 16, 16, 33, 1e6, 16, 0.25), (3, 3, 24, 8, 2), (4, 1, 32, None))],
             "loop": {"start": 0, "stop": 2, "times": 2}}
CONFIG_NB = {"architecture": "Nodepel", "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "vocab": 320, "width": 96,
             "layers": [layer((3, 3, 20, 40, 1, 100.0, 4, 0.35), (2, 2, 40, 12, 1), (40, 5, 16, 24)),
                        layer((8, 2, 48, 64, 500, 1e4, 24, 0.15), (6, 2, 32, 32, 5), (3, 3, 48, 16)),
                        layer((2, 1, 64, 128, 40, 1e5, 64, 0.12), (1, 1, 136, 72, 4), None),
                        layer((20, 1, 16, 8, 12, 50.0, 16, 0.25), (4, 1, 12, 20, 2), (8, 2, 20, 96))],
             "loop": {"start": 2, "stop": 3, "times": 3}}
CONFIG_NC = {"architecture": "Nodepel", "embedding": {"scale": 0.7}, "norm": {"eps": 1e-5}, "vocab": 96, "width": 32,
             "layers": [layer((2, 1, 16, 16, 9, 1e4, 16, 0.25), (2, 2, 16, 16, 4), (5, 2, 16, 16)),
                        layer((1, 1, 32, 48, 4, 1e3, 2, 0.2), (2, 1, 8, 32, 3), (2, 1, 24, None))]}
CONFIGS = {"NA": CONFIG_NA, "NB": CONFIG_NB, "NC": CONFIG_NC}


def layer_runs(cfg: dict) -> int:
    loop = cfg.get("loop")
    return len(cfg["layers"]) + ((loop["stop"] - loop["start"]) * (loop["times"] - 1) if loop else 0)


def make_folder(folder, cfg: dict, seed: int, dtype: str, sharp: float = 0.2, steady_router: bool = False) -> Path:
    """A model folder with seeded random weights.  The query and key maps of the softmax side are redrawn with
    standard deviation `sharp` and its norm weights spread, so that scores spread over several units and a wrong,
    missing or extra key shows in the logits; sinks of about the size of the scores; decays that neither vanish nor
    stay at one, so that a lost or doubled state shows; router logits wide enough that choices are rarely close.
    `steady_router`: the router's biases lie several units apart and its map is small, so that no choice is ever close
    (for runs in bfloat16, where the rounding of a close call would send a token to another expert than the oracle's;
    the float32 runs route by the token); the recurrent side's maps and the experts are drawn smaller as well, since
    decays, gates and squared activations that swing widely turn the 8-bit rounding of their input into several
    per cent of the logits, which would hide a fault as well as excuse one."""
    from flambeau_b200.config.nodepel import NodepelConfig
    from flambeau_b200.weights.random_init import write_random_model
    from flambeau_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    folder = Path(folder)
    write_random_model(folder, NodepelConfig.from_dict(cfg), seed=seed, dtype=dtype)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    g = torch.Generator().manual_seed(seed * 7919 + 13)

    def redraw(n, std, mean=0.0):
        t = tensors[n]
        tensors[n] = (torch.randn(t.shape, generator=g) * std + mean).to(t.dtype)
    for n in sorted(tensors):
        if n.endswith(".left.q") or n.endswith(".left.k"):
            redraw(n, sharp)
        elif n.endswith(".q.norm") or n.endswith(".k.norm"):
            # (q and k are normalised, so these weights, not the maps, set how far the scores spread)
            redraw(n, *((0.3, 1.2) if steady_router else (0.5, 3.0)))
        elif n.endswith(".sink"):
            redraw(n, 1.5)
        elif n.endswith(".right.a") or n.endswith(".right.b"):
            redraw(n, 0.04 if steady_router else 0.3)
        elif n.endswith(".A_log"):
            redraw(n, 0.5, -1.0)
        elif n.endswith(".right.q") or n.endswith(".right.k") or n.endswith(".right.v") or n.endswith(".right.g"):
            redraw(n, 0.08 if steady_router else 0.3)
        elif n.endswith(".router"):
            redraw(n, 0.03 if steady_router else 0.6)
        elif n.endswith(".router.b") and steady_router:
            t = tensors[n]
            tensors[n] = (torch.randperm(t.numel(), generator=g).float() * 4.0).to(t.dtype)
        elif n.endswith(".up") or n.endswith(".down"):
            redraw(n, 0.06 if steady_router else 0.15)
        elif n == "loop.step":
            redraw(n, 0.5)
    write_safetensors(folder / "model.safetensors", tensors)
    return folder
