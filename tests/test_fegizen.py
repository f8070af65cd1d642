"""Fegizen without a GPU: the configuration reader, the model as data (run order, who owns and who reads which cache,
state slots, tensor names), the random-weights folder, and properties of the plain implementation that the GPU tests
rely on."""
import copy
import math

import pytest
import torch

import fegizen_tiny as ft
import plain_fegizen as pf

F64 = torch.float64


def spec_of(cfg):
    from flambeau_b200 import models  # noqa: F401
    from flambeau_b200.config.registry import resolve
    arch = resolve("Fegizen")
    return arch.build_spec(arch.config_class.from_dict(cfg))


def test_config_round_trip_and_errors():
    from flambeau_b200.config.base import BadValue, MissingKey
    from flambeau_b200.config.fegizen import FegizenConfig
    for cfg in ft.CONFIGS.values():
        c = FegizenConfig.from_dict(cfg)
        assert FegizenConfig.from_dict(c.to_dict()) == c
    c = FegizenConfig.from_dict(ft.CONFIG_FA)
    assert c.layers[1].mlp is None and c.layers[3].mlp.shared_ff is None and c.layers[2].mlp.shared_ff == 40
    assert (c.layers[2].mlp.identity, c.layers[2].mlp.scale, c.layers[3].mlp.identity) == (2, 1.5, 0)
    assert (c.canon_taps, c.logit_scale, c.layers[0].mixer.stretch.factor, c.layers[2].mixer.kv_from) == (3, 0.5, 4.0, 0)
    assert FegizenConfig.from_dict(ft.CONFIG_FB).logit_scale == 1.0 and FegizenConfig.from_dict(ft.CONFIG_FB).layers[1].mixer.stretch is None
    bad = copy.deepcopy(ft.CONFIG_FA)
    bad["layers"][0]["mixer"]["rot"]["dims"] = 10                         # more than the rotated part has
    with pytest.raises(BadValue):
        FegizenConfig.from_dict(bad)
    bad = copy.deepcopy(ft.CONFIG_FA)
    bad["layers"][2]["mlp"]["router"]["top"] = 8                          # more than experts + identity experts
    with pytest.raises(BadValue):
        FegizenConfig.from_dict(bad)
    bad = copy.deepcopy(ft.CONFIG_FA)
    bad["layers"][1]["type"] = "attention"
    with pytest.raises(BadValue):
        FegizenConfig.from_dict(bad)
    bad = copy.deepcopy(ft.CONFIG_FA)
    bad["layers"][2]["mixer"]["kv_from"] = 1                              # that layer has no latents
    with pytest.raises(BadValue):
        FegizenConfig.from_dict(bad)
    bad = copy.deepcopy(ft.CONFIG_FA)
    bad["layers"][2]["mixer"]["kv_rank"] = 48                             # another latent size than the owner's
    with pytest.raises(BadValue):
        FegizenConfig.from_dict(bad)
    bad = copy.deepcopy(ft.CONFIG_FA)
    del bad["layers"][1]["mixer"]["tau"]
    with pytest.raises(MissingKey):
        FegizenConfig.from_dict(bad)
    bad = copy.deepcopy(ft.CONFIG_FA)
    bad["layers"][3]["mlp"]["kind"] = "sparse"
    with pytest.raises(BadValue):
        FegizenConfig.from_dict(bad)


def test_run_order_caches_and_state_slots():
    from flambeau_b200.models.decoder import DecoderModel
    spec = spec_of(ft.CONFIG_FA)
    assert [(c.layer, c.cache_from) for c in spec.order] == [(0, None), (1, None), (2, 0), (3, None)]
    plans = DecoderModel(spec, runtime=None).cache_plans()
    assert len(plans) == 4
    # one cache row per token: latent + the shared rotated key part, one key/value head, kept as far back as the
    # furthest-looking reader wants (layer 2's window, not layer 0's own)
    kv = plans[0].kv
    assert (kv.kv_heads, kv.head_dim, kv.window) == (1, 48, 20)
    assert plans[2].cache_from == 0 and plans[1].kv is None
    D, T = 64, 3
    # what a layer keeps per request: the mixer's matrices of state, then the kept inputs of the convolutions in front
    # of the mixer and in front of the feed-forward
    assert plans[0].state.shape == (2 * (T - 1) * D,) and plans[0].state.dtype == "float32"
    assert plans[1].state.shape == (2 * 24 * 16 + (T - 1) * D,)           # no feed-forward: one convolution
    assert plans[2].state.shape == (2 * (T - 1) * D,)
    assert plans[3].state.shape == (40 * 8 + 2 * (T - 1) * D,)
    plans = DecoderModel(spec_of(ft.CONFIG_FB), runtime=None).cache_plans()
    assert plans[0].state.shape == (3 * 12 * 20,)                          # one tap keeps nothing
    assert plans[1].state is None and plans[1].kv.window == 1 and plans[1].kv.head_dim == 26
    assert plans[4].cache_from == 2 and plans[2].kv.window == 500
    plans = DecoderModel(spec_of(ft.CONFIG_FC), runtime=None).cache_plans()
    assert plans[0].kv.window == 6 and plans[0].state.shape == (2 * 4 * 32,)


def test_tensor_names_and_shapes():
    from flambeau_b200.models.decoder import DecoderModel
    specs = DecoderModel(spec_of(ft.CONFIG_FA), runtime=None).tensor_specs()
    want = {"embed": (200, 64), "head": (200, 64), "final.norm": (64,),
            "l0.norm1": (64,), "l0.norm2": (64,), "l0.canon1": (64, 3), "l0.canon2": (64, 3), "l0.dwa": (2,),
            "l0.mix.dq": (24, 64), "l0.mix.dq.norm": (24,), "l0.mix.uq": (2 * 24, 24), "l0.mix.dkv": (48, 64),
            "l0.mix.dkv.norm": (40,), "l0.mix.uk": (32, 40), "l0.mix.uv": (48, 40), "l0.mix.g": (48, 64),
            "l0.mix.o": (64, 48), "l0.mlp.gate": (48, 64), "l0.mlp.up": (48, 64), "l0.mlp.down": (64, 48),
            "l1.mix.q": (48, 64), "l1.mix.k": (48, 64), "l1.mix.v": (32, 64), "l1.mix.g": (32, 64), "l1.mix.o": (64, 32),
            "l1.mix.norm": (16,), "l1.mix.a2.b": (48,), "l1.dwa": (3,), "l1.canon1": (64, 3),
            "l2.mix.uq": (3 * 16, 16), "l2.mix.uk": (24, 40), "l2.mix.uv": (48, 40), "l2.dwa": (4,),
            "l2.mlp.router": (7, 64), "l2.mlp.correction": (7,), "l2.mlp.e4.gate": (24, 64), "l2.mlp.e4.up": (24, 64),
            "l2.mlp.e4.down": (64, 24), "l2.mlp.shared.gate": (40, 64), "l2.mlp.shared.down": (64, 40),
            "l3.mix.q": (40, 64), "l3.mix.v": (8, 64), "l3.mix.norm": (8,), "l3.dwa": (5,), "l3.mlp.router": (4, 64)}
    for name, shape in want.items():
        assert name in specs and tuple(specs[name].shape) == shape, name
    assert specs["l1.mix.a1"].shape[0] == specs["l1.mix.a2"].shape[1]
    assert not any(n.startswith("l1.mlp.") or n in ("l1.norm2", "l1.canon2") for n in specs)
    assert not any(n.startswith("l2.mix.dkv") for n in specs), "a reader of another layer's latents has no map of its own"
    assert "l2.mlp.e5.up" not in specs, "identity experts have no tensors"
    assert not any(n.startswith("l3.mlp.shared") for n in specs)
    one_tap = DecoderModel(spec_of(ft.CONFIG_FB), runtime=None).tensor_specs()
    assert tuple(one_tap["l0.canon1"].shape) == (96, 1)


def test_random_folder_is_read_back_by_the_oracle(tmp_path):
    folder = ft.make_folder(tmp_path / "m", ft.CONFIG_FC, seed=5, dtype="bfloat16")
    cfg, w = pf.read_folder(folder)
    assert cfg["canon"]["taps"] == 5 and w["l1.canon2"].shape == (32, 5) and "l1.mix.dkv" not in w
    logits = pf.forward(cfg, w, [1, 2, 3, 4, 5, 6, 7])
    assert logits.shape == (7, 96) and bool(torch.isfinite(logits).all())


def test_command_line_writes_and_inspects_a_model(tmp_path, capsys):
    import json
    from flambeau_b200.cli import main
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(ft.CONFIG_FC))
    assert main(["random-model", "--config", str(cfg_file), "--out", str(tmp_path / "m"), "--seed", "3"]) == 0
    assert main(["inspect", "--model", str(tmp_path / "m")]) == 0
    out = capsys.readouterr().out
    assert '"architecture": "Fegizen"' in out and "l1.mix.uk" in out and "l0.mlp.e1.down" in out
    cfg, w = pf.read_folder(tmp_path / "m")
    assert pf.forward(cfg, w, [1, 2, 3]).shape == (3, ft.CONFIG_FC["vocab"])


def test_plain_small_mechanisms():
    g = torch.Generator().manual_seed(0)
    # the norm takes the mean off: a constant added to every channel changes nothing, and the result has mean zero
    x = torch.randn(3, 10, generator=g, dtype=F64)
    w = torch.ones(10, dtype=F64)
    assert torch.allclose(pf.centred_norm(x + 7.0, w, 1e-6), pf.centred_norm(x, w, 1e-6))
    assert float(pf.centred_norm(x, w, 1e-6).mean(-1).abs().max()) < 1e-12
    # eps lies inside the root
    tiny_x = torch.full((1, 4), 1e-3, dtype=F64)
    assert torch.allclose(pf.unit_rms(tiny_x, 1e-2), tiny_x / math.sqrt(1e-6 + 1e-2))
    # the convolution is added to its input, its last tap is the current token's, and it sees nothing ahead
    z = torch.arange(1.0, 6.0, dtype=F64)[:, None]
    assert torch.equal(pf.add_time_conv(z, torch.tensor([[0.0, 0.0, 1.0]], dtype=F64)), 2 * z)
    assert torch.equal(pf.add_time_conv(z, torch.tensor([[1.0, 0.0, 0.0]], dtype=F64))[:, 0],
                       torch.tensor([1.0, 2.0, 3.0 + 1.0, 4.0 + 2.0, 5.0 + 3.0], dtype=F64))
    # the rotation pairs neighbours, keeps lengths without a stretch, and is the identity at position 0
    v = torch.randn(3, 2, 8, generator=g, dtype=F64)
    f, mag = pf.rotary_frequencies({"base": 100.0, "dims": 8})
    assert mag == 1.0 and torch.allclose(f, torch.tensor([100.0 ** (-2 * i / 8) for i in range(4)], dtype=F64))
    y = pf.rotate_neighbours(v, [0, 5, 9], f, mag)
    assert torch.allclose(y[0], v[0]) and torch.allclose((y ** 2).sum(-1), (v ** 2).sum(-1))
    a = 5 * float(f[1])
    assert torch.allclose(y[1, 0, 2], v[1, 0, 2] * math.cos(a) - v[1, 0, 3] * math.sin(a))
    assert torch.allclose(y[1, 0, 3], v[1, 0, 3] * math.cos(a) + v[1, 0, 2] * math.sin(a))
    # the stretch: fast pairs keep their frequency, slow ones are divided by the factor, and both tables grow
    fs, mags = pf.rotary_frequencies({"base": 1e4, "dims": 16, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}})
    plain, _ = pf.rotary_frequencies({"base": 1e4, "dims": 16})
    assert mags == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert float(fs[0]) == float(plain[0]) and float(fs[-1]) == pytest.approx(float(plain[-1]) / 4.0)
    assert all(float(plain[i]) / 4.0 - 1e-15 <= float(fs[i]) <= float(plain[i]) + 1e-15 for i in range(8))


def test_plain_recurrence_and_router():
    g = torch.Generator().manual_seed(1)
    # decays of one: the state is the sum of k v^T, so the output is causal linear attention
    n, H, d, e = 6, 2, 4, 3
    q, k = torch.randn(n, H, d, generator=g, dtype=F64), torch.randn(n, H, d, generator=g, dtype=F64)
    v = torch.randn(n, H, e, generator=g, dtype=F64)
    o, S = pf.linear_attention_recurrence(q, k, v, torch.ones(n, H, d, dtype=F64))
    want = torch.einsum("ihd,jhd->hij", q, k).tril().permute(1, 0, 2)
    assert torch.allclose(o, torch.einsum("ihj,jhe->ihe", want, v))
    # a decay of zero on one key channel forgets what that channel held before the current token
    alpha = torch.ones(n, H, d, dtype=F64)
    alpha[-1, :, 0] = 0.0
    _, S0 = pf.linear_attention_recurrence(q, k, v, alpha)
    assert torch.allclose(S0[:, 0], k[-1, :, 0, None] * v[-1]) and torch.allclose(S0[:, 1:], S[:, 1:])
    # a state handed on continues the sequence
    o1, S1 = pf.linear_attention_recurrence(q[:4], k[:4], v[:4], torch.ones(4, H, d, dtype=F64))
    o2, S2 = pf.linear_attention_recurrence(q[4:], k[4:], v[4:], torch.ones(2, H, d, dtype=F64), state=S1)
    assert torch.allclose(torch.cat([o1, o2]), o) and torch.allclose(S2, S)
    # the decay is sigmoid(z)^(1/tau)
    w = {"m.a1": torch.randn(3, 8, generator=g, dtype=F64), "m.a2": torch.randn(4, 3, generator=g, dtype=F64),
         "m.a2.b": torch.randn(4, generator=g, dtype=F64)}
    h = torch.randn(5, 8, generator=g, dtype=F64)
    z = (h @ w["m.a1"].T) @ w["m.a2"].T + w["m.a2.b"]
    assert torch.allclose(pf.channel_decays(h, w, "m.", {"heads": 2, "dim": 2, "tau": 7.0}).reshape(5, 4),
                          torch.sigmoid(z) ** (1.0 / 7.0))
    # the router: the correction moves the choice and not the weights; the weights sum to the router's scale
    w = {"r.router": torch.randn(5, 8, generator=g, dtype=F64), "r.correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 9.0], dtype=F64)}
    chosen, weights = pf.route(h, w, "r.", {"top": 2, "scale": 1.5})
    s = torch.softmax(h @ w["r.router"].T, -1)
    assert bool((chosen[:, 0] == 4).all()), "a large correction always wins the choice"
    assert torch.allclose(weights.sum(-1), torch.full((5,), 1.5, dtype=F64))
    assert torch.allclose(weights[:, 0] / weights[:, 1], s[:, 4] / torch.gather(s, 1, chosen[:, 1:2])[:, 0])
    # an identity expert hands the input on: with one identity expert of one and no others, out = scale * h
    w = {"i.router": torch.randn(1, 8, generator=g, dtype=F64)}
    out = pf.routed_ff(h, w, "i.", {"router": {"experts": 0, "identity": 1, "top": 1, "scale": 0.25}})
    assert torch.allclose(out, 0.25 * h)


def test_plain_latent_attention_sees_its_window_and_no_more():
    """One layer: a token just outside the last query's window must not matter, the one just inside must."""
    g = torch.Generator().manual_seed(2)
    D, W = 16, 5
    m = ft.latent(2, 4, 4, 6, 8, 6, W, 100.0, 0.5)
    shapes = {"dq": (6, D), "dq.norm": (6,), "uq": (16, 6), "dkv": (12, D), "dkv.norm": (8,), "uk": (8, 8), "uv": (12, 8),
              "g": (12, D), "o": (D, 12)}
    w = {"m." + k: torch.randn(s, generator=g, dtype=F64) for k, s in shapes.items()}
    h = torch.randn(12, D, generator=g, dtype=F64)
    pos = list(range(12))
    ref, (c, kr) = pf.latent_attention(h, w, "m.", m, 1e-6, pos)
    assert c.shape == (12, 8) and kr.shape == (12, 4)
    h2 = h.clone()
    h2[11 - W] += 1.0
    out, _ = pf.latent_attention(h2, w, "m.", m, 1e-6, pos)
    assert torch.allclose(out[11], ref[11])
    h2 = h.clone()
    h2[11 - W + 1] += 1.0
    out, _ = pf.latent_attention(h2, w, "m.", m, 1e-6, pos)
    assert not torch.allclose(out[11], ref[11])
    # a reader of these latents with maps of its own: the same (c, kr), other heads
    out, (c2, kr2) = pf.latent_attention(h, w, "m.", m, 1e-6, pos, latent=(c, kr))
    assert torch.allclose(out, ref) and c2 is c and kr2 is kr


def test_large_head_groups_are_cut_into_equal_stretches_for_decoded_tokens():
    """More than 16 query heads on one key/value head: the split-key attention arrangement takes equal stretches of at
    most 16 heads, and a single token is short for it whatever the group's size."""
    from flambeau_b200.kernels import ops
    for heads in range(1, 65):
        share = ops.attention_kv_share(heads, 1)
        assert heads % share == 0 and heads // share <= 16
        assert share == 1 or all(heads % s or heads // s > 16 for s in range(1, share)), "the fewest stretches"
        assert ops.attention_is_short(1, heads, 1)
    assert ops.attention_kv_share(32, 1) == 2 and ops.attention_kv_share(64, 2) == 2 and ops.attention_kv_share(17, 1) == 17
    assert ops.attention_is_short(2, 8, 1) and not ops.attention_is_short(3, 8, 1)
    assert not ops.attention_is_short(2, 32, 1) and ops.attention_is_short(2, 16, 2)
