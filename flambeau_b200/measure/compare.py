"""Zedivik beside Mistral dense at equal size: prefill and decode throughput and the kernels that differ.

`bench.py --only zedivik` runs, for each size of SIZES, a Zedivik model (differential attention under a sliding
window, norms before and behind each sublayer, no loop) and a Mistral model with the same width, head counts, row
sizes of queries, keys and values, feed-forward size, window, vocabulary and number of layers, both with random
weights in bfloat16, through the same engine calls: one decode step of `batch` sequences that each hold `context`
tokens, and one step of `prefill` prompt tokens.  Per design it reports tokens a second and, per launcher (CUDA
events around every launcher call of an eager step, so serialised kernels), microseconds per layer; for the kernels
that the designs do not share (attention, the row-wise kernel between projection and attention, the norms) also the
work and the fraction of the measured peak that bounds it.

Work of the attention of one layer over `seen` (query, visible key) pairs:
  Mistral   4 * seen * heads * head size flops (Q K^T and P V);            cache bytes: keys * kv heads * 2 * head size
  Zedivik   4 * seen * heads * (key size + value size) flops (two maps of Q K^T over key size, two of P V over value
            size; what the kernel issues beside that for the float32 weights, a second P V product, is not counted);
            cache bytes: keys * kv heads * (2 * key size + value size)
"""
from __future__ import annotations

import gc
import statistics

import torch

from ..config.mistral import MistralConfig
from ..config.zedivik import ZedivikConfig
from ..engine.batch import Entry
from ..engine.step import Engine, EngineOptions
from ..kernels import ops
from . import work, workloads
from .timers import SectionTimer

PAGE = 16

# width, query heads, key/value heads, row size of a head's queries and keys (Mistral: head size; Zedivik: both maps,
# 2 * key size) and of its values, feed-forward size, window, vocabulary
SIZES = {
    "1b": dict(width=2048, heads=16, kv_heads=4, qk_row=128, v_row=128, ff=8192, window=1024, vocab=32000),
    "7b": dict(width=4096, heads=32, kv_heads=8, qk_row=128, v_row=128, ff=14336, window=4096, vocab=32000),
    "12b": dict(width=5120, heads=32, kv_heads=8, qk_row=128, v_row=128, ff=14336, window=2048, vocab=131072),
}


def configs(size: dict, layers: int):
    z = ZedivikConfig.from_dict({
        "architecture": "Zedivik", "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "vocab": size["vocab"],
        "width": size["width"],
        "layers": [{"type": "attention",
                    "mixer": {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["qk_row"] // 2,
                              "vdim": size["v_row"], "mask": {"size": size["window"]},
                              "scale": (size["qk_row"] // 2) ** -0.5, "diff": 0.5},
                    "mlp": {"ff": size["ff"], "kind": "dense"}}] * layers})
    m = MistralConfig.from_dict(dict(
        architectures=["MistralForCausalLM"], rms_norm_eps=1e-6, hidden_size=size["width"], num_hidden_layers=layers,
        num_attention_heads=size["heads"], num_key_value_heads=size["kv_heads"], head_dim=size["qk_row"],
        intermediate_size=size["ff"], vocab_size=size["vocab"], sliding_window=size["window"],
        max_position_embeddings=1 << 20))
    return {"zedivik": z, "mistral": m}


ATTENTION = ("paged_attention_mma", "diff_attention_mma", "paged_attention_simt", "diff_attention_simt")
CLASS_OF = {"paged_attention_mma": "attention", "diff_attention_mma": "attention", "rope_kv_write": "cache_write",
            "qkv_bias_cache_write": "cache_write", "add_rms_norm": "norm", "norm_add_rms_norm": "norm",
            "gate_mul": "gate_mul", "embedding": "embedding", "rope_table": "rope_table", "sample": "sample",
            "concat_cast": "concat_cast"}


def sections_by_class(engine, entries, end=(), reps: int = 3) -> dict:
    """class -> (launches, milliseconds) per step of one eager step; products are keyed by their matrix."""
    was = engine.use_graphs
    engine.use_graphs = False
    try:
        engine.step(entries, end=end)
        totals: dict = {}
        for _ in range(reps):
            torch.cuda._sleep(int(40.0 * 2.0e6))
            with SectionTimer() as t:
                logits = engine.step(entries, end=end)
                if logits is not None:
                    ops.sample(logits, torch.zeros(logits.shape[0], dtype=torch.int32, device=logits.device))
            for what, note, ms in t.sections():
                key = CLASS_OF.get(what) or (f"product {note[1]}x{note[2]}" if what.startswith("gemm") and note else what)
                n, total = totals.get(key, (0, 0.0))
                totals[key] = (n + 1, total + ms)
        return {k: (n / reps, total / reps) for k, (n, total) in totals.items()}
    finally:
        engine.use_graphs = was


def attention_work(design: str, size: dict, rows: int, contexts) -> dict:
    """flops and bytes of one layer's attention for a step of `rows` rows (decoded tokens: one per context; a
    portion: one context that the rows end at)."""
    W, H, G = size["window"], size["heads"], size["kv_heads"]
    if len(contexts) == rows:
        seen = sum(work.live_keys(c, W) for c in contexts)
        keys = seen
    else:
        ctx = contexts[0]
        seen = work.keys_seen(range(ctx - rows, ctx), W)
        keys = ctx - (max(0, ctx - rows - W + 1) if W else 0)
    if design == "mistral":
        flops = 4.0 * seen * H * size["qk_row"]
        q_out = rows * H * 2 * size["qk_row"] * 2
    else:
        flops = 4.0 * seen * H * (size["qk_row"] // 2 + size["v_row"])
        q_out = rows * H * (size["qk_row"] + size["v_row"]) * 2
    return dict(flops=flops, bytes=keys * G * (size["qk_row"] + size["v_row"]) * 2 + q_out)


def rowwise_work(design: str, size: dict, rows: int) -> dict:
    """Bytes one launch of the norm kernel and of the kernel between projection and attention must move."""
    D, H, G = size["width"], size["heads"], size["kv_heads"]
    cols = H * size["qk_row"] + G * (size["qk_row"] + size["v_row"])
    # Norm.  Zedivik: the stream in and out, the part's output in, normalised rows out (the part's output has to pass
    # its own norm before it may join the stream, so no product can add it there).  Mistral: the same for few rows;
    # over a portion its projections add to the stream themselves and the norm reads the stream and writes the rows.
    norm = rows * D * ((4 + 2) if design == "mistral" and rows > 128 else (4 + 4 + 4 + 2))
    # projection rows in (float32), q and cache rows out
    return {"norm": norm, "cache_write": rows * cols * (4 + 2)}


def measure(name: str, size: dict, layers: int, batch: int, context: int, prefill: int, steps: int, warmup: int,
            peaks: dict, gen, say) -> dict:
    out = {"size": dict(size), "layers": layers, "batch": batch, "context": context, "prefill_tokens": prefill}
    for design, cfg in configs(size, layers).items():
        say(f"{name}: building {design}, {layers} layers")
        live = min(context, size["window"] + PAGE)
        per_seq = -(-(live + 2 * PAGE + steps + warmup + 64) // PAGE) * PAGE
        engine = Engine.from_config(cfg, seed=0, options=EngineOptions(
            dtype="bfloat16", page_size=PAGE, cache_tokens=max(batch * per_seq + 512, prefill + PAGE),
            max_requests=batch, max_step_tokens=max(prefill, batch), max_seq_len=context + 4096))
        workloads.randomise_cache(engine)
        ms, launches = workloads.decode_device(engine, batch, context, steps, warmup, gen)
        pre_ms = workloads.prefill_step(engine, prefill, gen)
        rec = {"decode_ms": round(ms, 4), "decode_tok_s": round(batch / (ms / 1e3), 1), "launches_per_step": launches,
               "prefill_ms": round(pre_ms, 3), "prefill_tok_s": round(prefill / (pre_ms / 1e3), 1),
               "weight_bytes": engine.model.step_weight_bytes(), "kv_bytes_per_token": engine.cache.kv_bytes_per_token()}
        nbytes = work.decode_step_bytes(rec["weight_bytes"], rec["kv_bytes_per_token"], [context] * batch, size["window"])
        rec["decode_hbm_frac"] = round(nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        vocab = engine.model.vocab_size
        ids = workloads.seat(engine, [context] * batch)
        entries = [Entry(r, [int(torch.randint(0, vocab, (1,), generator=gen))], [0]) for r in ids]
        toks = torch.randint(0, vocab, (prefill,), generator=gen).tolist()
        for label, ent, end, rows, ctxs in (
                (f"decode_b{batch}", entries, (), batch, [context] * batch),
                (f"prefill_{prefill}", [Entry("prompt", toks, [prefill - 1])], ("prompt",), prefill, [prefill])):
            if label.startswith("prefill"):
                engine.cache.release_all()
            secs = sections_by_class(engine, ent, end=end)
            table = {}
            for key, (n, total) in sorted(secs.items()):
                per = layers if n >= layers else 1
                row = {"launches": round(n / per, 2), "us": round(total * 1e3 / per, 2)}
                w = None
                if key == "attention":
                    w = attention_work(design, size, rows, ctxs)
                elif key in ("norm", "cache_write"):
                    w = {"bytes": rowwise_work(design, size, rows)[key] * (n / per), "flops": 0.0}
                if w and row["us"] > 0:
                    by_mem = w["bytes"] / (row["us"] * 1e-6) / 1e9 / peaks["hbm_gbs"]
                    by_math = w.get("flops", 0.0) / (row["us"] * 1e-6) / 1e12 / peaks["bf16_tflops"]
                    row.update(bound="tensor" if by_math > by_mem else "hbm", frac=round(max(by_mem, by_math), 4))
                table[key] = row
            rec[label] = table
        engine.cache.release_all()
        out[design] = rec
        engine = None
        gc.collect()
        torch.cuda.empty_cache()
    z, m = out["zedivik"], out["mistral"]
    out["zedivik_over_mistral"] = {"decode_tok_s": round(z["decode_tok_s"] / m["decode_tok_s"], 3),
                                   "prefill_tok_s": round(z["prefill_tok_s"] / m["prefill_tok_s"], 3)}
    return out


def run(sizes, layers: int, batch: int, prefill: int, steps: int, warmup: int, peaks: dict, gen, say) -> dict:
    result = {}
    for name in sizes:
        size = SIZES[name]
        result[name] = measure(name, size, layers, batch, 2 * size["window"], prefill, steps, warmup, peaks, gen, say)
    return result
