"""Tubepel without a GPU: the configuration reader, the model as data (run order, one cache per pass of the looped
stretch, cache groups, tensor names), the random-weights folder, and properties of the plain implementation that the
GPU tests rely on."""
import copy
import math

import pytest
import torch

import plain_tubepel as pt
import tubepel_tiny as tt

F64 = torch.float64


def spec_of(cfg):
    from flambeau_b200 import models  # noqa: F401
    from flambeau_b200.config.registry import resolve
    arch = resolve("Tubepel")
    return arch.build_spec(arch.config_class.from_dict(cfg))


def test_config_round_trip_and_errors():
    from flambeau_b200.config.base import BadValue, MissingKey
    from flambeau_b200.config.tubepel import TubepelConfig
    for cfg in tt.CONFIGS.values():
        c = TubepelConfig.from_dict(cfg)
        assert TubepelConfig.from_dict(c.to_dict()) == c
    c = TubepelConfig.from_dict(tt.CONFIG_TA)
    assert (c.streams, c.loop.start, c.loop.stop, c.loop.times) == (3, 1, 3, 3)
    a = c.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.keep_first, a.rot_dims) == (4, 2, 16, 24, 9, 2, 8)
    assert c.layers[2].mlp is None and c.layers[3].mlp.shared_ff is None and c.layers[0].mlp.shared_ff == 40
    assert (c.layers[0].mlp.experts, c.layers[0].mlp.top, c.layers[3].mlp.top) == (5, 2, 1)
    b = TubepelConfig.from_dict(tt.CONFIG_TB)
    assert b.loop is None and b.streams == 1
    assert (b.layers[2].mixer.window, b.layers[2].mixer.keep_first, b.layers[2].mixer.rot_dims) == (0, 0, 0)
    assert TubepelConfig.from_dict(tt.CONFIG_TC).streams == 0
    for path, value, err in [(("layers", 1, "mixer", "rot", "dims"), 4, BadValue),     # latents turn their whole rotated part
                             (("layers", 0, "mixer", "rot", "dims"), 18, BadValue),    # more than a head has
                             (("layers", 0, "mixer", "kv_heads"), 3, BadValue),        # does not divide the query heads
                             (("layers", 0, "mlp", "router", "top"), 6, BadValue),     # more than there are experts
                             (("layers", 1, "type"), "gla", BadValue),
                             (("layers", 3, "mlp", "kind"), "sparse", BadValue),
                             (("loop", "stop"), 5, BadValue),                          # behind the last layer
                             (("streams",), -1, BadValue)]:
        bad = copy.deepcopy(tt.CONFIG_TA)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(err):
            TubepelConfig.from_dict(bad)
    bad = copy.deepcopy(tt.CONFIG_TA)
    del bad["layers"][1]["mixer"]["kv_rank"]
    with pytest.raises(MissingKey):
        TubepelConfig.from_dict(bad)
    bad = copy.deepcopy(tt.CONFIG_TA)
    del bad["layers"][0]["mixer"]["scale"]
    with pytest.raises(MissingKey):
        TubepelConfig.from_dict(bad)


def test_run_order_and_caches():
    from flambeau_b200.models.decoder import DecoderModel
    spec = spec_of(tt.CONFIG_TA)
    assert [c.layer for c in spec.order] == [0, 1, 2, 1, 2, 1, 2, 3] == pt.run_order(tt.CONFIG_TA)
    assert all(c.cache_from is None and not c.reenter for c in spec.order), "every pass has a cache of its own"
    plans = DecoderModel(spec, runtime=None).cache_plans()
    assert len(plans) == 8 and all(p.state is None for p in plans)
    kv = plans[0].kv
    assert (kv.kv_heads, kv.head_dim, kv.value_dim, kv.window, kv.keep_first) == (2, 16, 24, 9, 2)
    assert kv.release_window == 9 and kv.kept_pages(16) == 1 and kv.kept_pages(1) == 2, \
        "the window gives pages back; those that hold the kept first keys stay"
    assert plans[7].kv.release_window == 20 and plans[7].kv.keep_first == 0 and plans[7].kv.kept_pages(16) == 0
    lat = plans[1].kv
    assert (lat.kv_heads, lat.head_dim, lat.window, lat.values_in_keys) == (1, 48, 0, True)
    assert plans[1].kv == plans[3].kv == plans[5].kv and plans[2].kv.head_dim == 32
    assert [c.layer for c in spec_of(tt.CONFIG_TC).order] == [0, 1, 0, 1]
    assert [c.layer for c in spec_of(tt.CONFIG_TB).order] == [0, 1, 2, 3]
    # the block arrangement follows `streams`: copies of the stream with their weights, or a plain residual
    assert spec.layers[0].kind == "hyper_connections" and spec_of(tt.CONFIG_TB).layers[0].kind == "hyper_connections"
    assert spec_of(tt.CONFIG_TC).layers[0].kind == "pre_norm"


def test_tensor_names_and_shapes():
    from flambeau_b200.models.decoder import DecoderModel
    specs = DecoderModel(spec_of(tt.CONFIG_TA), runtime=None).tensor_specs()
    want = {"embed": (200, 64), "head": (200, 64), "final.norm": (64,), "l0.norm1": (64,), "l0.norm2": (64,),
            "l0.hc1.in": (3,), "l0.hc1.out": (3,), "l0.hc1.mix": (3, 3), "l0.hc2.mix": (3, 3),
            "l0.mix.q": (64, 64), "l0.mix.k": (32, 64), "l0.mix.v": (48, 64), "l0.mix.g": (96, 64), "l0.mix.o": (64, 96),
            "l0.mix.sink": (4,), "l0.mlp.router": (5, 64), "l0.mlp.e4.gate": (24, 64), "l0.mlp.e4.up": (24, 64),
            "l0.mlp.e4.down": (64, 24), "l0.mlp.shared.gate": (40, 64), "l0.mlp.shared.down": (64, 40),
            "l1.mix.dq": (24, 64), "l1.mix.dq.norm": (24,), "l1.mix.uq": (2 * 24, 24), "l1.mix.dkv": (48, 64),
            "l1.mix.dkv.norm": (40,), "l1.mix.uk": (32, 40), "l1.mix.uv": (48, 40), "l1.mix.o": (64, 48),
            "l1.mlp.up": (48, 64), "l1.mlp.down": (64, 48), "l2.mix.uq": (3 * 16, 16), "l2.hc1.in": (3,),
            "l3.mix.g": (64, 64), "l3.mlp.router": (4, 64)}
    for name, shape in want.items():
        assert name in specs and tuple(specs[name].shape) == shape, name
    assert not any(n.startswith(("l2.mlp.", "l2.hc2.")) or n == "l2.norm2" for n in specs), "a layer without feed-forward"
    assert not any(n.startswith("l3.mlp.shared") or n.endswith((".mix.dq.b", ".router.b", "mlp.gate")) for n in specs)
    assert "l1.mix.g" not in specs and "l1.mix.sink" not in specs, "latent attention has neither gate nor sink"
    plain = DecoderModel(spec_of(tt.CONFIG_TC), runtime=None).tensor_specs()
    assert not any(".hc" in n for n in plain), "without streams there are no stream weights"
    one = DecoderModel(spec_of(tt.CONFIG_TB), runtime=None).tensor_specs()
    assert tuple(one["l0.hc1.mix"].shape) == (1, 1) and tuple(one["l2.mix.v"].shape) == (24, 96)


def test_random_folder_is_read_back_by_the_oracle(tmp_path):
    for name, dtype in (("TC", "bfloat16"), ("TA", "float32")):
        folder = tt.make_folder(tmp_path / name, tt.CONFIGS[name], seed=5, dtype=dtype, steady_router=dtype == "bfloat16")
        cfg, w = pt.read_folder(folder)
        assert cfg["width"] == tt.CONFIGS[name]["width"] and "l1.mix.dkv" in w
        runs = []
        logits = pt.forward(cfg, w, [1, 2, 3, 4, 5, 6, 7], collect=runs)
        assert logits.shape == (7, cfg["vocab"]) and bool(torch.isfinite(logits).all())
        assert len(runs) == len(pt.run_order(cfg))


def test_command_line_makes_and_inspects_a_model(tmp_path):
    import json
    from flambeau_b200.cli import main
    (tmp_path / "c.json").write_text(json.dumps(tt.CONFIG_TC))
    assert main(["random-model", "--config", str(tmp_path / "c.json"), "--out", str(tmp_path / "m"), "--seed", "3"]) == 0
    cfg, w = pt.read_folder(tmp_path / "m")
    assert cfg["architecture"] == "Tubepel" and w["l1.mlp.e1.down"].shape == (32, 16)


# ---- properties of the plain implementation ----------------------------------------------------------------------
def test_what_a_position_sees():
    seen = pt.visible(12, window=3, keep_first=2)
    assert seen[11].nonzero().flatten().tolist() == [0, 1, 9, 10, 11]
    assert seen[3].nonzero().flatten().tolist() == [0, 1, 2, 3] and seen[0].tolist() == [True] + [False] * 11
    assert pt.visible(5, window=2)[4].nonzero().flatten().tolist() == [3, 4]
    assert bool((pt.visible(6) == torch.tril(torch.ones(6, 6, dtype=torch.bool))).all())
    assert bool((pt.visible(6, window=1, keep_first=1)[5] == torch.tensor([1, 0, 0, 0, 0, 1], dtype=torch.bool)).all())


def test_a_sink_takes_weight_and_gives_nothing():
    g = torch.Generator().manual_seed(0)
    s = torch.randn(2, 4, 4, generator=g, dtype=F64)
    seen = pt.visible(4)
    plain, sunk = pt.softmax_with_sink(s, seen), pt.softmax_with_sink(s, seen, torch.tensor([0.0, 50.0], dtype=F64))
    assert torch.allclose(plain.sum(-1), torch.ones(2, 4, dtype=F64))
    assert bool((sunk.sum(-1) < 1.0).all()) and float(sunk[1].sum(-1).max()) < 1e-15
    want = torch.exp(s[0, 3]) / (torch.exp(s[0, 3]).sum() + 1.0)       # exp(0) = 1 once in the denominator, not scaled
    assert torch.allclose(sunk[0, 3], want)


def test_both_pairings_turn_by_the_same_angles():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 2, 10, generator=g, dtype=F64)
    rot = {"base": 100.0, "dims": 6}
    a, b = pt.rotate(x, [0, 1, 2, 7, 300], rot, "neighbours"), pt.rotate(x, [0, 1, 2, 7, 300], rot, "halves")
    assert torch.equal(a[0], x[0]) and torch.equal(b[0], x[0]) and torch.equal(a[..., 6:], x[..., 6:])
    # the halves' layout is the neighbours' layout of the same vector with its dimensions dealt out again
    deal = [0, 3, 1, 4, 2, 5]
    y = x.clone()
    y[..., :6] = x[..., deal]
    assert torch.allclose(pt.rotate(y, [0, 1, 2, 7, 300], rot, "neighbours")[..., :6], b[..., deal])
    assert torch.allclose((a * a).sum(-1), (x * x).sum(-1))              # a turn keeps lengths


def test_streams_that_only_copy_are_a_plain_residual():
    g = torch.Generator().manual_seed(2)
    x, y = torch.randn(4, 6, generator=g, dtype=F64), torch.randn(4, 6, generator=g, dtype=F64)
    xs = torch.stack([x, x])
    w = {"in": torch.tensor([0.5, 0.5], dtype=F64), "out": torch.ones(2, dtype=F64), "mix": torch.eye(2, dtype=F64)}
    assert torch.allclose(pt.streams_read(xs, w, ""), x)
    assert torch.allclose(pt.streams_write(xs, y, w, ""), torch.stack([x + y, x + y]))
    w["mix"] = torch.tensor([[0.0, 1.0], [0.0, 0.0]], dtype=F64)          # [from, to]: stream 0 goes to stream 1 only
    moved = pt.streams_write(torch.stack([x, 2 * x]), 0 * y, w, "")
    assert torch.allclose(moved[1], x) and float(moved[0].abs().max()) == 0.0


def test_a_score_scales_what_the_expert_reads():
    g = torch.Generator().manual_seed(3)
    D, f = 8, 6
    w = {f"e{e}.{n}": torch.randn((f, D) if n != "down" else (D, f), generator=g, dtype=F64) for e in range(3)
         for n in ("gate", "up", "down")}
    w["router"] = torch.randn(3, D, generator=g, dtype=F64)
    h = torch.randn(5, D, generator=g, dtype=F64)
    mlp = {"router": {"experts": 3, "top": 2}}
    chosen, weights = pt.route(h, w, "", mlp["router"])
    s = torch.sigmoid(h @ w["router"].T)
    assert torch.equal(chosen[:, 0], s.argmax(-1)) and torch.allclose(weights, torch.gather(s, 1, chosen))
    assert bool((weights.sum(-1) != 1.0).all()), "the scores are not renormalised"
    out = pt.routed_ff(h, w, "", mlp)
    t = 2
    want = sum(pt.gated_ff(weights[t, k] * h[t:t + 1], w, f"e{int(chosen[t, k])}.")[0] for k in range(2))
    wrong = sum(weights[t, k] * pt.gated_ff(h[t:t + 1], w, f"e{int(chosen[t, k])}.")[0] for k in range(2))
    assert torch.allclose(out[t], want) and not torch.allclose(out[t], wrong)


def test_the_feed_forward_squares_what_is_positive():
    w = {"up": torch.tensor([[1.0], [-1.0]], dtype=F64), "down": torch.tensor([[1.0, 10.0]], dtype=F64)}
    out = pt.dense_ff(torch.tensor([[3.0], [-2.0]], dtype=F64), w, "")
    assert out.flatten().tolist() == [9.0, 40.0]
    assert math.isclose(float(pt.silu(torch.tensor(0.0, dtype=F64))), 0.0)
