"""Zedivik on the GPU against the plain implementation (tests/plain_zedivik.py): each mechanism alone through its
kernels, then whole models under schedules (whole, token by token, portions down to two tokens, mixed batches on a
pool so small that pages and slots are used again), long decoding, and greedy generation through generate()."""
import math

import pytest
import torch

import plain_zedivik as pz
import tiny
import zedivik_tiny as zt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rel_err(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max())


# ---------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------
def test_scaled_embedding():
    from flambeau_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    table = torch.randn(50, 24, generator=g).bfloat16()
    ids = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32)
    x = torch.empty(5, 24, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embedding(table.to(DEV), ids.to(DEV), x, status, scale=2.75)
    want = pz.embed(ids.tolist(), table.double(), 2.75)
    assert rel_err(x, want) < 1e-6 and int(status.item()) == 0


@pytest.mark.parametrize("width,slabs", [(24, 1), (64, 3), (1000, 2), (4100, 1)])
@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
def test_normed_delta_joins_the_stream_and_is_normed_again(width, slabs, out_dtype):
    """x += norm_b(sum of the slabs); out = norm(x): both norms with weights stored around zero."""
    from flambeau_b200.kernels import ops
    g = torch.Generator().manual_seed(width + slabs)
    n, eps_b, eps = 7, 1e-5, 1e-6
    x = torch.randn(n, width, generator=g) * 3
    delta = torch.randn(slabs, n, width, generator=g) * 0.01          # small: eps inside the root matters
    wb, w = torch.randn(width, generator=g) * 0.3, torch.randn(width, generator=g) * 0.3
    xs = x.to(DEV).clone()
    d = delta.to(DEV).contiguous()
    out = torch.empty(n, width, dtype=DT[out_dtype], device=DEV)
    ops.norm_add_rms_norm(xs, d[0], wb.to(DEV), eps_b, 1.0, w.to(DEV), eps, out, n_partials=slabs,
                          partial_stride=d.stride(0), weight_offset=1.0)
    x_want = x.double() + pz.offset_norm(delta.double().sum(0), wb.double(), eps_b)
    assert rel_err(xs, x_want) < 1e-6
    assert rel_err(out, pz.offset_norm(x_want, w.double(), eps)) < (1e-5 if out_dtype == "float32" else 6e-3)
    # chosen rows: normalised, and the stream untouched; then the stream alone, without an output
    xs2 = x.to(DEV).clone()
    rows = torch.tensor([5, 0, 2], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, width, dtype=torch.float32, device=DEV)
    ops.norm_add_rms_norm(xs2, d[0], wb.to(DEV), eps_b, 1.0, w.to(DEV), eps, out2, rows=rows, n_partials=slabs,
                          partial_stride=d.stride(0), weight_offset=1.0)
    assert torch.equal(xs2.cpu(), x) and rel_err(out2, pz.offset_norm(x_want[[5, 0, 2]], w.double(), eps)) < 1e-5
    ops.norm_add_rms_norm(xs2, d[0], wb.to(DEV), eps_b, 1.0, None, eps, None, n_partials=slabs,
                          partial_stride=d.stride(0))
    assert rel_err(xs2, x_want) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_reentry_of_the_embedding(dtype):
    """x <- W [x ; x0]."""
    from flambeau_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    n, D = 9, 40
    x, x0 = torch.randn(n, D, generator=g), torch.randn(n, D, generator=g)
    W = (torch.randn(D, 2 * D, generator=g) * 0.2).to(DT[dtype])
    both = torch.empty(n, 2 * D, dtype=DT[dtype], device=DEV)
    ops.concat_cast(x.to(DEV), x0.to(DEV), both)
    out = torch.empty(n, D, dtype=torch.float32, device=DEV)
    ops.linear(both, W.to(DEV), out)
    want = torch.cat([x, x0], dim=-1).double() @ W.double().T
    assert rel_err(out, want) < (1e-5 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_projection_rows_reach_q_cache_and_gate(dtype):
    from flambeau_b200.kernels import ops
    nh, nkv, kd, vd, page = 3, 1, 8, 20, 4
    case = zt.PagedCase([(5, 3), (0, 2)], nh=nh, nkv=nkv, kd=kd, vd=vd, window=0, page_size=page, dtype=DT[dtype],
                        device=DEV, seed=3, plant=False)
    g = torch.Generator().manual_seed(9)
    cols = nh * 2 * kd + nkv * 2 * kd + nkv * vd + nh
    proj = torch.randn(2, case.n, cols + 5, generator=g)               # two shares, rows wider than the columns
    bias = torch.randn(cols - nh, generator=g).to(DT[dtype])
    q = torch.empty(case.n, nh * 2 * kd, dtype=DT[dtype], device=DEV)
    gate = torch.empty(case.n, nh, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    case.cache.writable = True
    pd = proj.to(DEV)
    ops.qkv_bias_cache_write(pd[0], bias.to(DEV), q, gate, case.cache, case.pos_d, case.row_seq, nh, nkv, 2 * kd, vd,
                             nh, status, n_partials=2, partial_stride=pd.stride(0))
    s = proj.double().sum(0)
    s[:, :cols - nh] += bias.double()
    tol = 1e-6 if dtype == "float32" else 5e-3
    assert rel_err(q, s[:, :nh * 2 * kd]) < tol
    assert rel_err(gate, torch.sigmoid(s[:, cols - nh:cols])) < 1e-6
    kp, vp, table = case.cache.k_pool.cpu(), case.cache.v_pool.cpu(), case.cache.block_table.cpu()
    for r in range(case.n):
        sq, pos = int(case.row_seq[r]), int(case.pos_d[r])
        pg = int(table[sq, pos // page])
        kw = s[r, nh * 2 * kd:nh * 2 * kd + nkv * 2 * kd].view(nkv, 2 * kd)
        vw = s[r, nh * 2 * kd + nkv * 2 * kd:cols - nh].view(nkv, vd)
        assert rel_err(kp[pg, :, pos % page], kw) < tol and rel_err(vp[pg, :, pos % page], vw) < tol
    assert int(status.item()) == 0


# (heads, kv heads, key size per map, value size, window, page size)
GEOMETRIES = [(4, 2, 16, 48, 20, 16), (6, 1, 16, 32, 33, 16), (8, 2, 48, 64, 100, 16), (2, 1, 64, 128, 40, 8),
              (20, 1, 16, 16, 12, 16), (4, 1, 32, 80, 0, 16), (2, 2, 128, 256, 64, 32), (3, 3, 8, 20, 5, 16),
              (1, 1, 16, 16, 1, 16),
              # the head sizes that the tensor-core kernel is also built for with its sizes known to the compiler
              (6, 3, 48, 96, 50, 16), (4, 4, 32, 64, 70, 16), (2, 1, 64, 64, 0, 64), (4, 2, 128, 128, 31, 16)]
# (tokens in the cache, new tokens): first tokens, decoded tokens far into a request and at page borders, portions
# that start in mid-page beyond the window, portions of two tokens
SEQS = [(0, 1), (0, 37), (150, 1), (63, 2), (130, 70), (17, 3), (95, 1), (64, 1), (15, 1), (16, 1), (31, 130)]


@pytest.mark.parametrize("geometry", GEOMETRIES, ids=lambda g: "h%d.%d-k%d-v%d-w%d-p%d" % g)
@pytest.mark.parametrize("kernel", ["simt-float32", "simt-bfloat16", "mma-bfloat16"])
def test_differential_attention_kernels(geometry, kernel):
    """Planted keys just inside and just outside every window, at page borders, far back; unwritten slots hold NaN."""
    from flambeau_b200.kernels import ops
    nh, nkv, kd, vd, window, page = geometry
    which, dtype = kernel.split("-")
    case = zt.PagedCase(SEQS, nh=nh, nkv=nkv, kd=kd, vd=vd, window=window, page_size=page, dtype=DT[dtype], device=DEV,
                        seed=nh * 100 + kd)
    scale, lam, diff, eps = 0.3, 0.62, 0.35, 1e-5
    out = torch.full((case.n, nh * vd), float("nan"), dtype=DT[dtype], device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    if which == "mma":
        if not ops.diff_attention_mma_supported(case.q_d, nh, nkv, kd, vd):
            pytest.skip("sizes the tensor-core arrangements do not take run on the float32-math kernel")
        ops.diff_attention_mma(case.q_d, out, case.gate_d, case.cache, case.seq_q_start, case.seq_q_len,
                               case.seq_pos_start, len(SEQS), case.max_q_len, case.max_kv_len, case.any_short,
                               case.any_long, nh, nkv, kd, vd, window, scale, lam, eps, 1.0 - diff, status)
    else:
        ops.diff_attention_simt(case.q_d, out, case.gate_d, case.cache, case.pos_d, case.row_seq, nh, nkv, kd, vd,
                                window, scale, lam, eps, 1.0 - diff, status)
    want = case.expected(scale=scale, lam=lam, diff=diff, eps=eps)
    assert int(status.item()) == 0
    assert torch.isfinite(out.float()).all()
    err = rel_err(out, want)
    assert err < (2e-5 if dtype == "float32" else 8e-3), f"{kernel}: error {err:.2e} of the largest output"


# ---------------------------------------------------------------------------------------------------------------
# whole models under schedules
# ---------------------------------------------------------------------------------------------------------------
SHARP = {"float32": 0.2, "bfloat16": 0.1}
LENGTHS = {"ZA": [1, 9, 40, 75, 33, 21, 64, 110], "ZB": [2, 70, 17, 48, 130, 5], "ZC": [30, 3]}


@pytest.fixture(scope="module", params=[(c, d) for c in ("ZA", "ZB") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    name, dtype = request.param
    cfg = zt.CONFIGS[name]
    folder = zt.make_folder(tmp_path_factory.mktemp(f"z{name}{dtype}"), cfg, seed=17 if name == "ZA" else 29,
                            dtype=dtype, sharp=SHARP[dtype])
    requests = tiny.random_requests({"vocab_size": cfg["vocab"]}, LENGTHS[name], seed=4)
    pcfg, W = pz.read_folder(folder)
    want = {rid: pz.forward(pcfg, W, toks) for rid, toks in requests.items()}
    return dict(name=name, dtype=dtype, cfg=cfg, folder=folder, requests=requests, want=want,
                tol=tiny.tol_at_depth(dtype, zt.layer_runs(cfg)))


def run(case, schedule, tmp_path, cuda_graphs=True):
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    tokens = schedule.max_live_tokens(case["requests"])
    engine = Engine.from_folder(case["folder"], EngineOptions(
        dtype=case["dtype"], cache_tokens=tokens, max_requests=4, max_step_tokens=max(tokens, 128),
        max_seq_len=max(tokens, 192), cuda_graphs=cuda_graphs))
    replay(engine, schedule.lines(), tmp_path)
    run.last_engine = engine
    engine.cache.check_invariants()
    assert not engine.cache.requests, "requests left live after the trace"
    assert all(g.pool.n_free == g.pool.n_pages for g in engine.cache.groups), "pages lost"
    got = tiny.read_rows(tmp_path, schedule, case["cfg"]["vocab"])
    return tiny.compare_rows(got, case["want"], case["tol"], f"{case['name']} {case['dtype']}")


def test_whole(case, tmp_path):
    run(case, tiny.schedule_whole(case["requests"]), tmp_path)


def test_last_tokens_one_by_one_past_every_window(case, tmp_path):
    """The tail is longer than every window of ZA and than three of ZB's, so windows pass over decoded tokens."""
    run(case, tiny.schedule_tail(case["requests"], 45), tmp_path)


def test_portions_down_to_two_tokens(case, tmp_path):
    run(case, tiny.schedule_portions(case["requests"]), tmp_path)
    run(case, tiny.schedule_portions(case["requests"], sizes=(2, 31, 2, 2, 17, 64, 3)), tmp_path / "b")


@pytest.mark.parametrize("seed", [1, 2])
def test_mixed_batches_with_pages_and_slots_used_again(case, tmp_path, seed):
    sched = tiny.schedule_mixed(case["requests"], seed=seed)
    total_pages = sum(-(-len(t) // 16) for t in case["requests"].values())
    assert sched.max_live_tokens(case["requests"]) // 16 < total_pages, "the pool must be smaller than all requests"
    assert len(case["requests"]) > 4, "more requests than slots, so that slots are used again"
    run(case, sched, tmp_path)


def test_every_token_decoded_from_the_first(case, tmp_path):
    """One token a step from position 0 (replayed from CUDA graphs where the engine captures them)."""
    rid = max(case["requests"], key=lambda r: len(case["requests"][r]))
    toks = case["requests"][rid]
    s = tiny.Schedule()
    for p, t in enumerate(toks):
        s.add([(rid, [t], [0], p)], end=[rid] if p == len(toks) - 1 else [])
    one = dict(case, requests={rid: toks}, want={rid: case["want"][rid]})
    run(one, s, tmp_path)
    assert run.last_engine.graph_replays > len(toks) // 2, "single-token steps are replayed from a captured graph"


def test_no_loop_at_all(tmp_path):
    cfg = zt.CONFIGS["ZC"]
    folder = zt.make_folder(tmp_path / "m", cfg, seed=3, dtype="float32")
    requests = tiny.random_requests({"vocab_size": cfg["vocab"]}, LENGTHS["ZC"], seed=2)
    pcfg, W = pz.read_folder(folder)
    c = dict(name="ZC", dtype="float32", cfg=cfg, folder=folder, requests=requests, tol=1e-4,
             want={rid: pz.forward(pcfg, W, toks) for rid, toks in requests.items()})
    run(c, tiny.schedule_portions(requests, sizes=(5, 2, 9)), tmp_path / "o")


def test_a_token_beyond_the_window_does_not_matter_and_one_inside_does(tmp_path):
    """One layer, float32: changing the token just outside the last query's window leaves its logits as they were
    (to rounding); changing the one just inside moves them."""
    from flambeau_b200.engine.step import Engine, EngineOptions
    W_ = 11
    cfg = dict(zt.CONFIG_ZC, layers=[zt.attn(2, 1, 16, 32, W_, 0.25, 0.4, 48)])
    folder = zt.make_folder(tmp_path / "m", cfg, seed=8, dtype="float32")
    engine = Engine.from_folder(folder, EngineOptions(dtype="float32", cache_tokens=256, max_requests=2,
                                                      max_step_tokens=128))
    base = tiny.random_requests({"vocab_size": cfg["vocab"]}, [40], seed=1)["r0"]

    def last_logits(tokens, cut):
        engine.step([("a", tokens[:cut], [])])
        lg = engine.step([("a", tokens[cut:], [len(tokens) - cut - 1])], end=["a"])
        return lg[0].double().cpu()
    p = len(base) - 1
    ref = last_logits(base, 25)
    outside = list(base); outside[p - W_] = (outside[p - W_] + 1) % cfg["vocab"]
    inside = list(base); inside[p - W_ + 1] = (inside[p - W_ + 1] + 1) % cfg["vocab"]
    scale = float(ref.abs().max())
    assert float((last_logits(outside, 33) - ref).abs().max()) / scale < 1e-5
    assert float((last_logits(inside, 38) - ref).abs().max()) / scale > 1e-3


# ---------------------------------------------------------------------------------------------------------------
# generation through the entry point and the scheduler
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("ZA", "float32"), ("ZB", "bfloat16")])
def test_greedy_generation(tmp_path, name, dtype):
    from flambeau_b200 import generate
    cfg = zt.CONFIGS[name]
    folder = zt.make_folder(tmp_path / "m", cfg, seed=41, dtype=dtype, sharp=SHARP[dtype])
    pcfg, W = pz.read_folder(folder)
    prompts = list(tiny.random_requests({"vocab_size": cfg["vocab"]}, [3, 26, 50, 1, 12], seed=6).values())
    n_new = 10
    outs = generate(folder, prompts, max_tokens=n_new, temperature=0.0, dtype=dtype, prefill_chunk_tokens=16,
                    prefill_ubatch=40, inflight_slots=3)
    tol = tiny.tol_at_depth("bfloat16", zt.layer_runs(cfg))
    for prompt, out in zip(prompts, outs):
        assert len(out) == n_new
        toks = list(prompt)
        for t in out:
            logits = pz.forward(pcfg, W, toks)[-1]
            if dtype == "float32":
                assert t == pz.argmax_lowest(logits), "greedy token differs from the plain implementation"
            else:
                gap = float(logits.max() - logits[t]) / float(logits.abs().max())
                assert gap <= 2 * tol, f"token {t} is {gap:.3f} of the scale below the best logit"
            toks.append(t)
