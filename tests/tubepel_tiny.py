"""Tiny Tubepel configurations and model folders shared by the tests.

Three configurations that differ from each other in every size and option:
  TA: width 64, vocab 200, three residual streams, layers 1 and 2 looped three times; windowed attention with grouped
      heads (4 on 2), values wider than keys, a window of 9 that keeps the first 2 keys, half of a head rotated, 5
      experts of which 2 and a shared expert; latent attention pairing neighbours with a dense feed-forward; latent
      attention pairing halves without feed-forward; windowed attention without grouping, the whole head rotated, a
      window that keeps nothing, one of 4 experts and no shared expert
  TB: width 96, vocab 320, ONE stream with its own weights, no loop; 5 heads over latents whose cache row is no
      multiple of 8 wide (20 + 6), 40 experts of which 5; 6 heads on one key/value head of 64 under a window of 70
      that keeps the first 66 keys (more than a tile of keys); attention without a mask, without rotation, values
      narrower than keys; one head over latents with cache rows of 64
  TC: width 32, vocab 96, no streams (a plain residual), both layers looped twice; a window of ONE key that keeps the
      first key; both of 2 experts chosen
"""
from __future__ import annotations

import math
from pathlib import Path

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=1e4, scale=0.2):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "rot": {"base": base, "dims": rot_dim}, "scale": scale}


def attention(heads, kv_heads, dim, vdim, window, keep_first, rot_dims, base=1e4, scale=0.2):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


CONFIG_TA = {"architecture": "Tubepel", "norm": {"eps": 1e-5}, "streams": 3, "vocab": 200, "width": 64,
             "loop": {"start": 1, "stop": 3, "times": 3},
             "layers": [layer("attention", attention(4, 2, 16, 24, 9, 2, 8, 1e4, 0.3), moe(5, 2, 24, 40)),
                        layer("latent_attention", latent(2, 16, 8, 24, 40, 24, 1e4, 0.2), dense(48)),
                        layer("latent_attention_2", latent(3, 8, 8, 16, 24, 16, 1e3, 0.3), None),
                        layer("attention", attention(2, 2, 32, 32, 20, 0, 32, 5e5, 0.2), moe(4, 1, 32))]}
CONFIG_TB = {"architecture": "Tubepel", "norm": {"eps": 1e-6}, "streams": 1, "vocab": 320, "width": 96,
             "layers": [layer("latent_attention_2", latent(5, 4, 6, 8, 20, 40, 100.0, 0.35), moe(40, 5, 16, 16)),
                        layer("attention", attention(6, 1, 64, 64, 70, 66, 16, 1e6, 0.15), dense(80)),
                        layer("attention", attention(3, 3, 24, 8, 0, 0, 0, 1e4, 0.25), dense(24)),
                        layer("latent_attention", latent(1, 32, 16, 32, 48, 56, 1e6, 0.15), None)]}
CONFIG_TC = {"architecture": "Tubepel", "norm": {"eps": 1e-5}, "vocab": 96, "width": 32,
             "loop": {"start": 0, "stop": 2, "times": 2},
             "layers": [layer("attention", attention(2, 1, 8, 8, 1, 1, 4, 1e3, 0.3), dense(40)),
                        layer("latent_attention", latent(2, 8, 4, 8, 16, 12, 1e3, 0.25), moe(2, 2, 16, 8))]}
CONFIGS = {"TA": CONFIG_TA, "TB": CONFIG_TB, "TC": CONFIG_TC}


def read_tensors(folder) -> dict:
    from flambeau_b200.weights.safetensors_io import SafetensorsFile
    f = SafetensorsFile(Path(folder) / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    return tensors


def write_tensors(folder, tensors: dict) -> None:
    from flambeau_b200.weights.safetensors_io import write_safetensors
    write_safetensors(Path(folder) / "model.safetensors", tensors)


def make_folder(folder, cfg: dict, seed: int, dtype: str, sharp: float = 0.25, steady_router: bool = False) -> Path:
    """A model folder with seeded random weights.  The maps that form queries and keys are redrawn with standard
    deviation `sharp`, so that scores spread over several units and a wrong, missing or extra key shows in the logits;
    sinks of a unit's spread, so that leaving one out shows; router logits wide enough that choices are rarely close.
    `steady_router` (for runs in bfloat16, where the rounding of a close call would send a token to another expert
    than the oracle's; the float32 runs route by the token): channel 0 of the stream is made a positive constant that
    no sublayer writes to (the embedding's column 0 is 0.2, the rows for channel 0 of every output map are zero, the
    streams' read and mix weights are positive), and every router reads that channel alone with a different factor
    per expert: the order of the experts is then the same for every token, while their scores still differ from token
    to token."""
    from flambeau_b200.config.tubepel import TubepelConfig
    from flambeau_b200.weights.random_init import write_random_model
    folder = Path(folder)
    write_random_model(folder, TubepelConfig.from_dict(cfg), seed=seed, dtype=dtype)
    tensors = read_tensors(folder)
    g = torch.Generator().manual_seed(seed * 7919 + 13)

    def redraw(n, std, mean=0.0):
        t = tensors[n]
        tensors[n] = (torch.randn(t.shape, generator=g) * std + mean).to(t.dtype)
    for n in sorted(tensors):
        if n.endswith((".mix.uq", ".mix.uk", ".mix.dkv", ".mix.q", ".mix.k")):
            redraw(n, sharp)
        elif n.endswith((".mix.v", ".mix.uv", ".mix.g")):
            redraw(n, 0.1)
        elif n.endswith(".router"):
            redraw(n, 0.5)
        if not steady_router:
            continue
        t = tensors[n]
        if n == "embed":
            t[:, 0] = 0.2
        elif n.endswith((".o", ".down")):
            t[0] = 0.0
        elif n.endswith((".in", ".mix")) and ".hc" in n:
            tensors[n] = t.abs()
        elif n.endswith(".router"):
            # (a power of two as the unit keeps the factors exact in bfloat16; the largest logit, factor x the
            # channel's value of at most sqrt(width), stays where float32 still tells the sigmoids apart)
            unit = 2.0 ** math.floor(math.log2(6.0 / math.sqrt(t.shape[1]) / t.shape[0]))
            factors = (torch.randperm(t.shape[0], generator=g).float() + 1.0) * unit
            tensors[n] = torch.zeros_like(t)
            tensors[n][:, 0] = factors.to(t.dtype)
    write_tensors(folder, tensors)
    return folder
