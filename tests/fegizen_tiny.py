"""Tiny Fegizen configurations and model folders shared by the tests.

Three configurations that differ from each other in every size and option:
  FA: width 64, vocab 200, embedding scale 2, eps 1e-5, logits times 0.5, 3 taps; four layers: latent attention
      (2 heads, 16 + 8 query/key dimensions, values of 24, latents of 40 and 24, a window of 9, stretched rotation)
      with a dense feed-forward; linear attention (2 heads, keys 24, values 16) without feed-forward; latent attention
      that reads layer 0's latents with 3 heads and a longer window (20) than their owner's, experts 5 + 2 without
      weights of which 3, shares times 1.5, a shared expert; linear attention of the second name with one head and
      keys wider than values (40, 8), one of 4 experts, neither identity nor shared expert
  FB: width 96, vocab 320, one tap (nothing kept), no logit scale; five layers, among them a window of one key, 20
      heads, latents whose cache row is no multiple of 8 wide (20 + 6), a window longer than any request, cache rows
      of 64, a reader two layers behind its owner, keys of 136 and values of 72 on the linear side, 40 experts of
      which 5
  FC: two layers, five taps, a reader right behind its owner with the same window
"""
from __future__ import annotations

from pathlib import Path

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base=1e4, scale=0.2, scaling=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim}, "scale": scale}
    if scaling is not None:
        factor, original, fast, slow = scaling
        m["rot"]["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def linear(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff, scale=1.0, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top, "scale": scale},
         "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


CONFIG_FA = {"architecture": "Fegizen", "canon": {"taps": 3}, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
             "logit_scale": 0.5, "vocab": 200, "width": 64,
             "layers": [layer("latent_attention", latent(2, 16, 8, 24, 40, 24, 9, 1e4, 0.2, (4.0, 16, 8.0, 1.0)), dense(48)),
                        layer("gla", linear(2, 24, 16, 8.0), None),
                        layer("latent_attention", latent(3, 8, 8, 16, 40, 16, 20, 1e4, 0.3, (4.0, 16, 8.0, 1.0), kv_from=0),
                              moe(5, 2, 3, 24, 1.5, 40)),
                        layer("gla_2", linear(1, 40, 8, 2.0), moe(4, 0, 1, 32))]}
CONFIG_FB = {"architecture": "Fegizen", "canon": {"taps": 1}, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
             "vocab": 320, "width": 96,
             "layers": [layer("gla", linear(3, 12, 20, 1.0), dense(80)),
                        layer("latent_attention", latent(20, 4, 6, 8, 20, 40, 1, 100.0, 0.35), moe(40, 1, 5, 16)),
                        layer("latent_attention", latent(1, 32, 16, 32, 48, 56, 500, 1e6, 0.15, (8.0, 64, 4.0, 0.5)), None),
                        layer("gla_2", linear(2, 136, 72, 30.0), dense(24)),
                        layer("latent_attention", latent(2, 16, 16, 40, 48, 8, 40, 1e6, 0.2, (8.0, 64, 4.0, 0.5), kv_from=2),
                              moe(3, 3, 2, 48, 0.5, 16))]}
CONFIG_FC = {"architecture": "Fegizen", "canon": {"taps": 5}, "embedding": {"scale": 0.7}, "norm": {"eps": 1e-5},
             "logit_scale": 2.0, "vocab": 96, "width": 32,
             "layers": [layer("latent_attention", latent(2, 8, 4, 8, 16, 12, 6, 1e3, 0.3), moe(2, 1, 2, 16, 1.0, 8)),
                        layer("latent_attention", latent(1, 16, 4, 24, 16, 20, 6, 1e3, 0.25, kv_from=0), dense(40))]}
CONFIGS = {"FA": CONFIG_FA, "FB": CONFIG_FB, "FC": CONFIG_FC}


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
    """A model folder with seeded random weights.  The maps that form queries and the latents' keys are redrawn with
    standard deviation `sharp`, so that scores spread over several units and a wrong, missing or extra key shows in the
    logits; decays that neither vanish nor stay at one, so that a lost or doubled state shows; taps and depth weights
    large enough that a lost tail or a wrong mix shows; router logits wide enough that choices are rarely close.
    `steady_router`: the corrections lie far apart and the router's map is small, so that no choice is ever close (for
    runs in bfloat16, where the rounding of a close call would send a token to another expert than the oracle's; the
    float32 runs route by the token)."""
    from flambeau_b200.config.fegizen import FegizenConfig
    from flambeau_b200.weights.random_init import write_random_model
    folder = Path(folder)
    write_random_model(folder, FegizenConfig.from_dict(cfg), seed=seed, dtype=dtype)
    tensors = read_tensors(folder)
    g = torch.Generator().manual_seed(seed * 7919 + 13)

    def redraw(n, std, mean=0.0):
        t = tensors[n]
        tensors[n] = (torch.randn(t.shape, generator=g) * std + mean).to(t.dtype)
    for n in sorted(tensors):
        if n.endswith(".mix.uq") or n.endswith(".mix.uk") or n.endswith(".mix.dkv"):
            redraw(n, sharp)
        elif n.endswith(".mix.a2.b"):
            redraw(n, 1.5, 2.0)
        elif n.endswith(".mix.a2"):
            redraw(n, 0.5)
        elif n.endswith(".mix.q") or n.endswith(".mix.k") or n.endswith(".mix.v"):
            redraw(n, 0.08 if steady_router else 0.2)
        elif n.endswith(".router"):
            redraw(n, 0.02 if steady_router else 0.5)
        elif n.endswith(".correction"):
            t = tensors[n]
            if steady_router:       # scores lie in (0, 1): corrections a whole unit apart decide every choice
                tensors[n] = torch.randperm(t.numel(), generator=g).float().to(t.dtype)
            else:
                redraw(n, 0.05)
        elif n.endswith(".canon1") or n.endswith(".canon2"):
            redraw(n, 0.3)
    write_tensors(folder, tensors)
    return folder
