"""Nodepel beside Mistral dense at equal size: prefill and decode throughput and the kernels that differ.

`bench.py --only nodepel` runs, for each size of SIZES, a Nodepel model (sliding-window attention with a sink beside a
gated delta rule, routed experts with a shared expert, no loop) and a Mistral model with the same width, attention
geometry, window, vocabulary and number of layers, whose feed-forward is as wide as what a Nodepel token passes
through (its chosen experts plus the shared one), both with random weights in bfloat16, through the same engine
calls: one decode step of `batch` sequences that each hold `context` tokens, and one step of `prefill` prompt tokens.
Per design it reports tokens a second and, per launcher (CUDA events around every launcher call of an eager step, so
serialised kernels), microseconds per layer; for the kernels of the new mechanisms also their work and the fraction
of the measured peak that bounds them, beside the like kernel of Mistral.

Work, per layer:
  attention          4 * seen * heads * head size flops; cache bytes keys * kv heads * (key + value size) * 2
  recurrence         per token and head 8 * dk * dv flops (decay, S^T k, the rank-one update, S^T q), float32 on the CUDA
                     cores (bounded by the float32 FMA rate, 2 * 128 lanes * SMs * clock); per request and step the
                     state is read and written once: 2 * heads * dk * dv * 4 bytes
  routed products    4 * pairs * width * expert inner size flops for both products; bytes: the weights of the experts
                     that were chosen, once
"""
from __future__ import annotations

import gc

import torch

from ..config.mistral import MistralConfig
from ..config.nodepel import NodepelConfig
from ..engine.batch import Entry
from ..engine.step import Engine, EngineOptions
from . import work, workloads
from .compare import PAGE, attention_work, sections_by_class

# width, heads, key/value heads, head size, window, vocabulary; recurrent side: value heads, query/key heads, key and
# value size, taps; experts, how many a token uses, their inner size, the shared expert's inner size
SIZES = {
    "1b": dict(width=2048, heads=16, kv_heads=4, qk_row=128, v_row=128, window=1024, vocab=32000,
               r_heads=16, r_qk_heads=4, r_dk=128, r_dv=128, conv=4, experts=32, top=4, expert_ff=1024, shared_ff=4096),
    "7b": dict(width=4096, heads=32, kv_heads=8, qk_row=128, v_row=128, window=4096, vocab=32000,
               r_heads=32, r_qk_heads=8, r_dk=128, r_dv=128, conv=4, experts=64, top=6, expert_ff=1792, shared_ff=3584),
}

CLASS_OF = {"paged_attention_mma": "attention", "paged_attention_simt": "attention", "rope_kv_write": "cache_write",
            "qk_norm_rope_kv_write": "cache_write", "add_rms_norm": "norm", "gate_mul": "gate_mul",
            "gdr_prepare": "recurrence_prepare", "gdr_recurrent": "recurrence", "gdr_out_norm": "recurrence_out",
            "branch_norm_mix": "branch_mix", "moe_choose": "router", "moe_sort": "expert_order",
            "moe_gather_rows": "expert_gather", "moe_combine": "expert_combine", "activation": "activation",
            "gemm_tc_grouped": "routed_product", "gemm_simt_grouped": "routed_product"}


def configs(size: dict, layers: int):
    n = NodepelConfig.from_dict({
        "architecture": "Nodepel", "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "vocab": size["vocab"],
        "width": size["width"],
        "layers": [{"type": "parallel",
                    "mixer": {"left": {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["qk_row"],
                                       "vdim": size["v_row"], "mask": {"size": size["window"]},
                                       "rot": {"base": 1e6, "dims": size["qk_row"]}, "scale": size["qk_row"] ** -0.5},
                              "right": {"heads": size["r_heads"], "kv_heads": size["r_qk_heads"], "dim": size["r_dk"],
                                        "vdim": size["r_dv"], "conv": size["conv"]}},
                    "mlp": {"kind": "moe", "router": {"experts": size["experts"], "top": size["top"]},
                            "expert": {"ff": size["expert_ff"]}, "shared": {"ff": size["shared_ff"]}}}] * layers})
    m = MistralConfig.from_dict(dict(
        architectures=["MistralForCausalLM"], rms_norm_eps=1e-6, hidden_size=size["width"], num_hidden_layers=layers,
        num_attention_heads=size["heads"], num_key_value_heads=size["kv_heads"], head_dim=size["qk_row"],
        intermediate_size=size["top"] * size["expert_ff"] + size["shared_ff"], vocab_size=size["vocab"],
        sliding_window=size["window"], max_position_embeddings=1 << 20))
    return {"nodepel": n, "mistral": m}


def fp32_fma_tflops(device) -> float:
    p = torch.cuda.get_device_properties(device)
    return 2.0 * 128 * p.multi_processor_count * (p.clock_rate if hasattr(p, "clock_rate") else 1.9e6) * 1e3 / 1e12


def new_kernel_work(size: dict, rows: int, n_seqs: int) -> dict:
    H, dk, dv, D = size["r_heads"], size["r_dk"], size["r_dv"], size["width"]
    pairs = rows * size["top"]
    experts_read = min(size["experts"], pairs)
    return {
        "recurrence": dict(fma_flops=8.0 * rows * H * dk * dv, bytes=n_seqs * 2 * H * dk * dv * 4 + rows * H * dv * 4),
        "routed_product": dict(flops=4.0 * pairs * D * size["expert_ff"],
                               bytes=experts_read * 2 * D * size["expert_ff"] * 2),
    }


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
               "weight_bytes": engine.model.step_weight_bytes(), "kv_bytes_per_token": engine.cache.kv_bytes_per_token(),
               "state_bytes_per_request": engine.cache.state_bytes_per_request()}
        # what a decode step must read: every weight that takes part (of the routed experts those that the batch's
        # tokens are expected to choose between them, each once), the live keys and values, and the state twice
        nbytes = work.decode_step_bytes(rec["weight_bytes"], rec["kv_bytes_per_token"], [context] * batch, size["window"])
        if design == "nodepel":
            E, K = size["experts"], size["top"]
            distinct = E * (1.0 - (1.0 - K / E) ** batch)
            per_expert = 2 * size["width"] * size["expert_ff"] * 2
            nbytes += layers * (distinct - K) * per_expert + 2 * batch * rec["state_bytes_per_request"]
        rec["decode_bytes"] = int(nbytes)
        rec["decode_hbm_frac"] = round(nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        vocab = engine.model.vocab_size
        ids = workloads.seat(engine, [context] * batch)
        entries = [Entry(r, [int(torch.randint(0, vocab, (1,), generator=gen))], [0]) for r in ids]
        toks = torch.randint(0, vocab, (prefill,), generator=gen).tolist()
        fma_peak = fp32_fma_tflops(engine.runtime.device)
        for label, ent, end, rows, ctxs in (
                (f"decode_b{batch}", entries, (), batch, [context] * batch),
                (f"prefill_{prefill}", [Entry("prompt", toks, [prefill - 1])], ("prompt",), prefill, [prefill])):
            if label.startswith("prefill"):
                engine.cache.release_all()
            secs = sections_by_class(engine, ent, end=end)
            merged: dict = {}
            for key, (n, total) in secs.items():
                key = CLASS_OF.get(key, key)
                a, b = merged.get(key, (0, 0.0))
                merged[key] = (a + n, b + total)
            extra = new_kernel_work(size, rows, len(ctxs) if len(ctxs) == rows else 1)
            table = {}
            for key, (n, total) in sorted(merged.items()):
                per = layers if n >= layers else 1
                row = {"launches": round(n / per, 2), "us": round(total * 1e3 / per, 2)}
                w = attention_work("mistral", size, rows, ctxs) if key == "attention" else extra.get(key)
                if w and row["us"] > 0:
                    sec = row["us"] * 1e-6
                    by_mem = w["bytes"] / sec / 1e9 / peaks["hbm_gbs"]
                    by_math = w.get("flops", 0.0) / sec / 1e12 / peaks["bf16_tflops"]
                    by_fma = w.get("fma_flops", 0.0) / sec / 1e12 / fma_peak
                    best = max(by_mem, by_math, by_fma)
                    row.update(bound="hbm" if best == by_mem else "tensor" if best == by_math else "fp32 fma",
                               frac=round(best, 4))
                table[key] = row
            rec[label] = table
        engine.cache.release_all()
        out[design] = rec
        engine = None
        gc.collect()
        torch.cuda.empty_cache()
    z, m = out["nodepel"], out["mistral"]
    out["nodepel_over_mistral"] = {"decode_tok_s": round(z["decode_tok_s"] / m["decode_tok_s"], 3),
                                   "prefill_tok_s": round(z["prefill_tok_s"] / m["prefill_tok_s"], 3)}
    return out


def run(sizes, layers: int, batch: int, prefill: int, steps: int, warmup: int, peaks: dict, gen, say) -> dict:
    result = {}
    for name in sizes:
        size = SIZES[name]
        result[name] = measure(name, size, layers, batch, 2 * size["window"], prefill, steps, warmup, peaks, gen, say)
    return result
