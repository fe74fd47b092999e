"""Zedivik without a GPU: the configuration reader, the run order that a loop gives, the tensors a model wants,
the random-weights folder, and properties of the plain implementation that the GPU tests lean on."""
import copy
import json

import pytest
import torch

import plain_zedivik as pz
import zedivik_tiny as zt
from flambeau_b200.config.base import BadValue, MissingKey
from flambeau_b200.config.registry import load_config, resolve
from flambeau_b200.config.zedivik import ZedivikConfig


def test_the_registry_finds_it_by_the_single_architecture_key(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(zt.CONFIG_ZA))
    arch, cfg = load_config(tmp_path)
    assert arch.name == "Zedivik" and isinstance(cfg, ZedivikConfig)
    assert cfg.to_dict() == zt.CONFIG_ZA
    assert cfg.layers[1].mlp is None and cfg.layers[0].mixer.window == 20 and cfg.loop.times == 2


@pytest.mark.parametrize("edit,error", [
    (lambda c: c.pop("width"), MissingKey),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), MissingKey),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), BadValue),
    (lambda c: c["layers"][0].update(type="recurrent"), BadValue),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), BadValue),
    (lambda c: c["loop"].update(stop=9), BadValue),
    (lambda c: c["loop"].update(times=0), BadValue),
    (lambda c: c["norm"].update(eps=0.0), BadValue),
])
def test_bad_configurations_are_named(edit, error):
    cfg = copy.deepcopy(zt.CONFIG_ZA)
    edit(cfg)
    with pytest.raises(error):
        ZedivikConfig.from_dict(cfg)


def order_of(cfg):
    spec = resolve("Zedivik").build_spec(ZedivikConfig.from_dict(cfg))
    spec.validate()
    return [(c.layer, c.reenter) for c in spec.order], spec


def test_run_order_of_a_loop():
    order, spec = order_of(zt.CONFIG_ZA)
    assert order == [(0, True), (1, False), (0, True), (1, False), (2, False)] and spec.reentry is not None
    order, _ = order_of(zt.CONFIG_ZB)
    assert order == [(0, False), (1, False), (2, True), (2, True), (2, True), (3, False)]
    order, spec = order_of(zt.CONFIG_ZC)
    assert order == [(0, False), (1, False)] and spec.reentry is None
    assert order == [(i, f) for i, f in pz.layer_runs(zt.CONFIG_ZC)]
    assert [(i, f) for i, f in pz.layer_runs(zt.CONFIG_ZB)] == order_of(zt.CONFIG_ZB)[0]


def test_every_pass_of_a_loop_owns_a_cache_and_values_have_their_own_width():
    from flambeau_b200.models.decoder import DecoderModel
    _, spec = order_of(zt.CONFIG_ZB)
    plans = DecoderModel(spec, runtime=None).cache_plans()
    assert len(plans) == 6 and all(p.cache_from is None for p in plans)
    assert (plans[2].kv.kv_heads, plans[2].kv.head_dim, plans[2].kv.value_dim, plans[2].kv.window) == (1, 128, 128, 40)
    assert (plans[0].kv.head_dim, plans[0].kv.value_dim, plans[0].kv.window) == (16, 20, 1)
    assert plans[2].kv == plans[3].kv == plans[4].kv          # one group, three owners


def test_tensor_names_and_shapes(tmp_path):
    from flambeau_b200.weights.random_init import model_tensor_specs
    specs = model_tensor_specs(ZedivikConfig.from_dict(zt.CONFIG_ZA))
    assert specs["embed"].shape == (200, 64) and specs["head"].shape == (200, 64)
    assert specs["loop.in"].shape == (64, 128) and specs["final.norm"].shape == (64,)
    assert specs["l0.mix.q"].shape == (4 * 2 * 16, 64) and specs["l0.mix.k"].shape == (2 * 2 * 16, 64)
    assert specs["l0.mix.v"].shape == (2 * 48, 64) and specs["l0.mix.o"].shape == (64, 4 * 48)
    assert specs["l0.mix.g"].shape == (4, 64) and specs["l0.mix.q.b"].shape == (128,) and specs["l2.mix.lk2"].shape == (16,)
    assert specs["l0.mlp.gate"].shape == (96, 64) and specs["l0.mlp.down"].shape == (64, 96)
    assert "l1.mlp.gate" not in specs and "l1.norm2" not in specs and "l1.norm1b" in specs
    assert "loop.in" not in model_tensor_specs(ZedivikConfig.from_dict(zt.CONFIG_ZC))
    folder = zt.make_folder(tmp_path, zt.CONFIG_ZA, seed=1, dtype="bfloat16")
    cfg, w = pz.read_folder(folder)
    assert set(w) == set(specs) and all(tuple(w[n].shape) == tuple(specs[n].shape) for n in specs)


def test_plain_implementation_sees_exactly_the_window():
    mask = pz.window_mask([0, 4, 9], 10, 3)
    assert mask[0].tolist() == [True] + [False] * 9
    assert mask[1].nonzero().flatten().tolist() == [2, 3, 4] and mask[2].nonzero().flatten().tolist() == [7, 8, 9]
    assert pz.window_mask([5], 10, 0)[0].nonzero().flatten().tolist() == [0, 1, 2, 3, 4, 5]


def test_plain_implementation_is_causal_and_loops(tmp_path):
    cfg, w = pz.read_folder(zt.make_folder(tmp_path, zt.CONFIG_ZA, seed=2, dtype="float32"))
    toks = [3, 7, 1, 9, 4, 4, 8, 2, 6, 5, 0, 11]
    full, streams = pz.forward(cfg, w, toks, return_layers=True)
    assert streams.shape[0] == zt.layer_runs(cfg) == 5
    assert torch.allclose(pz.forward(cfg, w, toks[:7]), full[:7], atol=1e-12)
    once = dict(cfg, loop=dict(cfg["loop"], times=1))
    assert not torch.allclose(pz.forward(once, w, toks), full, atol=1e-6)


def test_command_line_writes_and_inspects_a_model(tmp_path, capsys):
    from flambeau_b200.cli import main
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(zt.CONFIG_ZC))
    assert main(["random-model", "--config", str(cfg_file), "--out", str(tmp_path / "m"), "--seed", "3"]) == 0
    assert main(["inspect", "--model", str(tmp_path / "m")]) == 0
    out = capsys.readouterr().out
    assert '"architecture": "Zedivik"' in out and "l1.mix.lq2" in out and "final.norm" in out
    cfg, w = pz.read_folder(tmp_path / "m")
    assert pz.forward(cfg, w, [1, 2, 3]).shape == (3, zt.CONFIG_ZC["vocab"])
