"""Tiny Zedivik configurations, model folders and hand-made paged caches shared by the tests.

Three configurations that differ from each other in every size and option:
  ZA: width 64, vocab 200, embedding scale 3.5, eps 1e-5; three layers with 4/2, 2/2 and 6/1 heads, key sizes 16, 32,
      16, value sizes 48, 16, 32, windows 20, 7, 33; the second layer has no feed-forward; layers 0-1 run twice
  ZB: width 96, vocab 320, embedding scale 1, eps 1e-6; four layers, among them a window of one key, a key size the
      tensor cores do not take (8), a value size that is no multiple of 16 (20), a window longer than any request,
      20 query heads on one key/value head, diff = 0; layer 2 alone runs three times
  ZC: two layers, no loop at all
"""
from __future__ import annotations

from pathlib import Path

import torch


def attn(heads, kv_heads, dim, vdim, window, scale, diff, ff):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
                      "scale": scale, "diff": diff},
            "mlp": {"ff": ff, "kind": "dense"} if ff else None}


CONFIG_ZA = {"architecture": "Zedivik", "embedding": {"scale": 3.5}, "norm": {"eps": 1e-5}, "vocab": 200, "width": 64,
             "layers": [attn(4, 2, 16, 48, 20, 0.3, 0.3, 96), attn(2, 2, 32, 16, 7, 0.2, 0.6, None),
                        attn(6, 1, 16, 32, 33, 0.25, 0.45, 160)],
             "loop": {"start": 0, "stop": 2, "times": 2}}
CONFIG_ZB = {"architecture": "Zedivik", "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "vocab": 320, "width": 96,
             "layers": [attn(3, 3, 8, 20, 1, 0.35, 0.2, 128), attn(8, 2, 48, 64, 500, 0.15, 0.0, 64),
                        attn(2, 1, 64, 128, 40, 0.12, 0.7, None), attn(20, 1, 16, 16, 12, 0.25, 0.5, 96)],
             "loop": {"start": 2, "stop": 3, "times": 3}}
CONFIG_ZC = {"architecture": "Zedivik", "embedding": {"scale": 0.5}, "norm": {"eps": 1e-5}, "vocab": 96, "width": 32,
             "layers": [attn(2, 1, 16, 16, 9, 0.25, 0.4, 48), attn(1, 1, 32, 48, 4, 0.2, 0.1, 40)]}
CONFIGS = {"ZA": CONFIG_ZA, "ZB": CONFIG_ZB, "ZC": CONFIG_ZC}


def layer_runs(cfg: dict) -> int:
    loop = cfg.get("loop")
    return len(cfg["layers"]) + ((loop["stop"] - loop["start"]) * (loop["times"] - 1) if loop else 0)


def make_folder(folder, cfg: dict, seed: int, dtype: str, sharp: float = 0.2) -> Path:
    """A model folder with seeded random weights.  The query and key maps are redrawn with standard deviation
    `sharp`, so that scores spread over several units and a wrong, missing or extra key shows in the logits; the
    vectors behind lambda are redrawn larger, so that lambda is not just the configuration's constant."""
    from flambeau_b200.config.zedivik import ZedivikConfig
    from flambeau_b200.weights.random_init import write_random_model
    from flambeau_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    folder = Path(folder)
    write_random_model(folder, ZedivikConfig.from_dict(cfg), seed=seed, dtype=dtype)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    g = torch.Generator().manual_seed(seed * 7919 + 13)
    for n in sorted(tensors):
        t = tensors[n]
        if n.endswith(".mix.q") or n.endswith(".mix.k"):
            tensors[n] = (torch.randn(t.shape, generator=g) * sharp).to(t.dtype)
        elif n.split(".")[-1] in ("lq1", "lk1", "lq2", "lk2"):
            tensors[n] = (torch.randn(t.shape, generator=g) * 0.25).to(t.dtype)
        elif n.endswith(".b"):
            tensors[n] = (torch.randn(t.shape, generator=g) * 0.3).to(t.dtype)
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


# ---- a hand-made paged cache for kernel tests ---------------------------------------------------------------------
class PagedCase:
    """Sequences given as (tokens already in the cache, new tokens of this step); keys and values of all of them
    scattered into pools whose pages are handed out in random order, unwritten slots poisoned with NaN, block-table
    rows that start at the first page a window still needs."""

    def __init__(self, seqs, *, nh, nkv, kd, vd, window, page_size, dtype, device, seed=0, plant=True):
        from flambeau_b200.cache.manager import LayerCacheView
        g = torch.Generator().manual_seed(seed)
        self.seqs, self.nh, self.nkv, self.kd, self.vd, self.window = seqs, nh, nkv, kd, vd, window
        self.dtype = dtype

        def rnd(*shape, s=1.0):
            return (torch.randn(*shape, generator=g) * s).to(dtype).double()     # values the dtype holds exactly
        self.q, self.k, self.v, self.positions = [], [], [], []
        for ctx, n in seqs:
            T = ctx + n
            q, k, v = rnd(n, nh, 2, kd), rnd(T, nkv, 2, kd), rnd(T, nkv, vd, s=2.0)
            if plant:
                # a key just inside and one just outside the window of the last query (and of the first), both with a
                # score that would dominate its map: the one outside must not be seen
                for row in {0, n - 1}:
                    p = ctx + row
                    for mp in (0, 1):
                        for hh in range(0, nh, max(1, nh // 2)):
                            qv = q[row, hh, mp]
                            gk = hh // (nh // nkv)
                            unit = qv / (qv * qv).sum()
                            edge = p - window + 1 if window else 0
                            if edge >= 0:
                                k[edge, gk, mp] = (unit * 40.0).to(dtype).double()
                            if window and edge - 1 >= 0:
                                k[edge - 1, gk, mp] = (unit * 90.0).to(dtype).double()
            self.q.append(q); self.k.append(k); self.v.append(v)
            self.positions.append(list(range(ctx, T)))
        # ---- pools ----
        first_page = [max(0, (ctx - window + 1)) // page_size if window else 0 for ctx, _ in seqs]
        n_pages_of = [-(-(ctx + n) // page_size) - fp for (ctx, n), fp in zip(seqs, first_page)]
        total = sum(n_pages_of) + 3
        order = torch.randperm(total, generator=g).tolist()
        width = max(n_pages_of) + 1
        table = torch.full((len(seqs), width), -1, dtype=torch.int32)
        k_pool = torch.full((total, nkv, page_size, 2 * kd), float("nan"), dtype=dtype)
        v_pool = torch.full((total, nkv, page_size, vd), float("nan"), dtype=dtype)
        for s, ((ctx, n), fp) in enumerate(zip(seqs, first_page)):
            for j in range(n_pages_of[s]):
                page = order.pop()
                table[s, j] = page
                lo = (fp + j) * page_size
                hi = min(lo + page_size, ctx + n)
                k_pool[page, :, :hi - lo] = self.k[s][lo:hi].reshape(hi - lo, nkv, 2 * kd).transpose(0, 1).to(dtype)
                v_pool[page, :, :hi - lo] = self.v[s][lo:hi].transpose(0, 1).to(dtype)
        dev = device
        i32 = dict(dtype=torch.int32, device=dev)
        self.cache = LayerCacheView(k_pool.to(dev), v_pool.to(dev), table.to(dev), torch.tensor(first_page, **i32),
                                    page_size, False, 0, None)
        lens = [n for _, n in seqs]
        starts = [sum(lens[:i]) for i in range(len(lens))]
        self.n = sum(lens)
        self.seq_q_start = torch.tensor(starts, **i32)
        self.seq_q_len = torch.tensor(lens, **i32)
        self.seq_pos_start = torch.tensor([ctx for ctx, _ in seqs], **i32)
        self.pos_d = torch.tensor([p for ps in self.positions for p in ps], **i32)
        self.row_seq = torch.tensor([s for s, n in enumerate(lens) for _ in range(n)], **i32)
        self.q_d = torch.cat([q.reshape(q.shape[0], -1) for q in self.q]).to(dtype).to(dev).contiguous()
        self.gate = torch.rand(self.n, nh, generator=g).float()
        self.gate_d = self.gate.to(dev)
        self.max_q_len, self.max_kv_len = max(lens), max(ctx + n for ctx, n in seqs)
        G = nh // nkv
        self.any_short = any(n * G <= 16 for n in lens)
        self.any_long = any(n * G > 16 for n in lens)

    def expected(self, *, scale, lam, diff, eps):
        import plain_zedivik as pz
        outs, at = [], 0
        for s, (ctx, n) in enumerate(self.seqs):
            outs.append(pz.diff_heads(self.q[s], self.k[s], self.v[s], self.gate[at:at + n].double(), self.positions[s],
                                      scale=scale, window=self.window, lam=lam, diff=diff, eps=eps))
            at += n
        return torch.cat(outs)
