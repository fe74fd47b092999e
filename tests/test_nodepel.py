"""Nodepel without a GPU: the configuration reader, the model as data (run order, caches and state slots, tensor names),
the random-weights folder, and properties of the plain implementation that the GPU tests rely on."""
import copy

import pytest
import torch

import nodepel_tiny as nt
import plain_nodepel as pn


def spec_of(cfg):
    from flambeau_b200 import models  # noqa: F401
    from flambeau_b200.config.registry import resolve
    arch = resolve("Nodepel")
    return arch.build_spec(arch.config_class.from_dict(cfg))


def test_config_round_trip_and_errors():
    from flambeau_b200.config.base import BadValue, MissingKey
    from flambeau_b200.config.nodepel import NodepelConfig
    for cfg in nt.CONFIGS.values():
        c = NodepelConfig.from_dict(cfg)
        assert NodepelConfig.from_dict(c.to_dict()) == c
    c = NodepelConfig.from_dict(nt.CONFIG_NA)
    assert c.layers[1].mlp is None and c.layers[2].mlp.shared_ff is None and c.layers[0].mlp.shared_ff == 40
    assert (c.layers[0].mixer.left.rot_dims, c.layers[0].mixer.right.conv) == (8, 4)
    bad = copy.deepcopy(nt.CONFIG_NA)
    bad["layers"][0]["mixer"]["left"]["rot"]["dims"] = 18                 # more than the head has
    with pytest.raises(BadValue):
        NodepelConfig.from_dict(bad)
    bad = copy.deepcopy(nt.CONFIG_NA)
    bad["layers"][0]["mlp"]["router"]["top"] = 7                          # more than there are experts
    with pytest.raises(BadValue):
        NodepelConfig.from_dict(bad)
    bad = copy.deepcopy(nt.CONFIG_NA)
    bad["layers"][2]["type"] = "attention"
    with pytest.raises(BadValue):
        NodepelConfig.from_dict(bad)
    bad = copy.deepcopy(nt.CONFIG_NA)
    del bad["layers"][1]["mixer"]["right"]["conv"]
    with pytest.raises(MissingKey):
        NodepelConfig.from_dict(bad)
    bad = copy.deepcopy(nt.CONFIG_NA)
    bad["loop"]["stop"] = 4
    with pytest.raises(BadValue):
        NodepelConfig.from_dict(bad)


def test_run_order_and_passes():
    order = spec_of(nt.CONFIG_NA).order
    assert [(c.layer, c.reenter, c.pass_index) for c in order] == \
        [(0, True, 0), (1, False, 0), (0, True, 1), (1, False, 1), (2, False, 0)]
    order = spec_of(nt.CONFIG_NB).order
    assert [(c.layer, c.reenter, c.pass_index) for c in order] == \
        [(0, False, 0), (1, False, 0), (2, True, 0), (2, True, 1), (2, True, 2), (3, False, 0)]
    assert [(i, t) for i, t in pn.run_order(nt.CONFIG_NB)] == [(0, None), (1, None), (2, 0), (2, 1), (2, 2), (3, None)]
    spec = spec_of(nt.CONFIG_NC)
    assert spec.reentry is None and [c.layer for c in spec.order] == [0, 1]


def test_every_pass_owns_pages_and_a_state_slot():
    from flambeau_b200.models.decoder import DecoderModel
    plans = DecoderModel(spec_of(nt.CONFIG_NA), runtime=None).cache_plans()
    assert len(plans) == 5 and all(p.cache_from is None for p in plans)
    kv, st = plans[0].kv, plans[0].state
    assert (kv.kv_heads, kv.head_dim, kv.value_dim, kv.window) == (2, 16, 32, 20)
    # the state of a pass: a matrix per head, then the convolution's kept inputs
    assert st.shape == (4 * 8 * 16 + 3 * (2 * 2 * 8 + 4 * 16),) and st.dtype == "float32"
    assert plans[2].kv == plans[0].kv and plans[2].state == plans[0].state
    assert plans[4].kv.value_dim == 16 and plans[4].kv.window == 33
    one_tap = DecoderModel(spec_of(nt.CONFIG_NB), runtime=None).cache_plans()[0].state
    assert one_tap.shape == (2 * 40 * 12,)                       # a convolution of one tap keeps nothing


def test_tensor_names_and_shapes():
    from flambeau_b200.models.decoder import DecoderModel
    specs = DecoderModel(spec_of(nt.CONFIG_NA), runtime=None).tensor_specs()
    want = {"embed": (200, 64), "head": (200, 64), "final.norm": (64,), "loop.in": (64, 128), "loop.step": (2, 64),
            "l0.norm1": (64,), "l0.norm2": (64,), "l0.mix.left.q": (64, 64), "l0.mix.left.k": (32, 64),
            "l0.mix.left.v": (64, 64), "l0.mix.left.q.norm": (64,), "l0.mix.left.k.norm": (32,),
            "l0.mix.left.sink": (4,), "l0.mix.left.o": (64, 128), "l0.mix.left.out": (64,), "l0.mix.right.out": (64,),
            "l0.mix.right.q": (16, 64), "l0.mix.right.q.conv": (16, 4), "l0.mix.right.v": (64, 64),
            "l0.mix.right.v.conv": (64, 4), "l0.mix.right.b": (4, 64), "l0.mix.right.a": (4, 64),
            "l0.mix.right.A_log": (4,), "l0.mix.right.dt_bias": (4,), "l0.mix.right.g": (64, 64),
            "l0.mix.right.norm": (16,), "l0.mix.right.o": (64, 64), "l0.mlp.e5.up": (24, 64),
            "l0.mlp.e5.down": (64, 24), "l0.mlp.router": (6, 64), "l0.mlp.router.b": (6,),
            "l0.mlp.shared.up": (40, 64), "l0.mlp.shared.down": (64, 40), "l0.mlp.shared.sg": (1, 64),
            "l2.mlp.e3.up": (32, 64)}
    for name, shape in want.items():
        assert name in specs and tuple(specs[name].shape) == shape, name
    assert not any(n.startswith("l1.mlp.") or n == "l1.norm2" for n in specs), "a layer without feed-forward has no such tensors"
    assert not any(n.startswith("l2.mlp.shared") for n in specs) and "l0.mlp.e6.up" not in specs
    assert "loop.in" not in DecoderModel(spec_of(nt.CONFIG_NC), runtime=None).tensor_specs()


def test_random_folder_is_read_back_by_the_oracle(tmp_path):
    folder = nt.make_folder(tmp_path / "m", nt.CONFIG_NC, seed=5, dtype="bfloat16")
    cfg, w = pn.load_folder(folder)
    assert cfg["layers"][1]["mixer"]["right"]["conv"] == 3 and w["l1.mix.right.k.conv"].shape == (8, 3)
    logits = pn.forward(cfg, w, [1, 2, 3, 4, 5, 6, 7])
    assert logits.shape == (7, 96) and bool(torch.isfinite(logits).all())


def test_command_line_writes_and_inspects_a_model(tmp_path, capsys):
    import json
    from flambeau_b200.cli import main
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(nt.CONFIG_NC))
    assert main(["random-model", "--config", str(cfg_file), "--out", str(tmp_path / "m"), "--seed", "3"]) == 0
    assert main(["inspect", "--model", str(tmp_path / "m")]) == 0
    out = capsys.readouterr().out
    assert '"architecture": "Nodepel"' in out and "l1.mix.right.A_log" in out and "l0.mlp.e4.down" in out
    cfg, w = pn.load_folder(tmp_path / "m")
    assert pn.forward(cfg, w, [1, 2, 3]).shape == (3, nt.CONFIG_NC["vocab"])


def test_plain_mechanisms():
    g = torch.Generator().manual_seed(0)
    # the window: itself and size - 1 tokens before it
    m = pn.window_mask(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True] and m[1].tolist() == [True, True] + [False] * 4
    # a sink far below the scores changes nothing; a sink far above takes nearly all the weight, and has no value
    s = torch.randn(4, 4, generator=g, dtype=torch.float64)
    full = torch.ones(4, 4, dtype=torch.bool)
    assert torch.allclose(pn.sink_softmax(s, full, torch.tensor(-80.0, dtype=torch.float64)), torch.softmax(s, -1))
    assert float(pn.sink_softmax(s, full, torch.tensor(40.0, dtype=torch.float64)).sum(-1).max()) < 1e-12
    # the rotation keeps lengths, leaves the tail of the head alone and is the identity at position 0
    x = torch.randn(3, 2, 10, generator=g, dtype=torch.float64)
    y = pn.rotate_half(x, [0, 5, 9], 100.0, 6)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.allclose(y[0], x[0])
    assert torch.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))
    # the convolution's last tap is the current token's, and it sees nothing ahead
    taps = torch.tensor([[0.0, 0.0, 1.0]], dtype=torch.float64)
    z = torch.arange(5, dtype=torch.float64)[:, None]
    assert torch.equal(pn.short_convolution(z, taps), z)
    assert torch.equal(pn.short_convolution(z, torch.tensor([[1.0, 0.0, 0.0]], dtype=torch.float64))[:, 0],
                       torch.tensor([0.0, 0.0, 0.0, 1.0, 2.0], dtype=torch.float64))
    # the delta rule with beta = 1 and no decay stores a value under a unit key and reads it back with the same key
    k = torch.zeros(2, 4, dtype=torch.float64); k[0, 1] = 1.0; k[1, 2] = 1.0
    v = torch.randn(2, 3, generator=g, dtype=torch.float64)
    o = pn.delta_rule(k, k, v, torch.ones(2, dtype=torch.float64), torch.ones(2, dtype=torch.float64))
    assert torch.allclose(o, v)
    # one expert of one: its share is 1 whatever the logit
    w = {"m.router": torch.randn(1, 8, generator=g, dtype=torch.float64), "m.router.b": torch.zeros(1, dtype=torch.float64),
         "m.e0.up": torch.randn(5, 8, generator=g, dtype=torch.float64),
         "m.e0.down": torch.randn(8, 5, generator=g, dtype=torch.float64)}
    h = torch.randn(3, 8, generator=g, dtype=torch.float64)
    assert torch.allclose(pn.routed_experts(h, w, "m.", {"router": {"experts": 1, "top": 1}}), pn.expert(h, w, "m.e0."))
