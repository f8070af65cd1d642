"""A plain, slow implementation of the Tubepel design in float64 torch on the CPU: the oracle of the tests.

One function per mechanism; whole sequences only (no cache, no pages, no batches, no portions), so that whatever the
engine does with pages and schedules is compared with something that has none of them.  It shares no code with the
product path.  `cfg` is the parsed config.json (a dict); `w` maps tensor names to float64 tensors.

Notation: n tokens, D = width, S = residual streams.  Latent attention: H heads, d = unrotated and r = rotated
query/key size of a head, e = value size, Rq and Rc the sizes of the query's and the key/value's latent.  Windowed
attention: H query heads on G key/value heads, d = key size, e = value size, R = rotated dimensions of a head,
W = window, F = first tokens that stay visible.  Feed-forward: E experts of which each token uses K.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64

# With `rounding_to(torch.bfloat16)` active, the values that a bfloat16 engine may keep in 16 bits (the inputs of
# products, cached rows, activations) are rounded to that type on their way; the distance between such a run and the
# exact one is the noise that rounding alone causes, from which the tests take their bfloat16 tolerance.
_ROUND = [None]


class rounding_to:
    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        _ROUND[0] = self.dtype

    def __exit__(self, *exc):
        _ROUND[0] = None


def kept(x):
    return x if _ROUND[0] is None else x.to(_ROUND[0]).to(F64)


# ---- small mechanisms -------------------------------------------------------------------------------------------
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


# ---- rotation -----------------------------------------------------------------------------------------------------
def rotation_angles(positions, rot):
    """[n, dims/2]: position * base^(-2i/dims)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    return torch.as_tensor(positions, dtype=F64)[:, None] * f[None, :]


def rotate(x, positions, rot, layout):
    """x [n, heads, m]: the first rot.dims dimensions of every head are turned pair by pair, the rest pass.  `layout`
    'neighbours' pairs dimension 2i with 2i + 1, 'halves' pairs dimension i with i + dims/2."""
    dims = int(rot["dims"])
    ang = rotation_angles(positions, rot)[:, None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)
    out = x.clone()
    if layout == "neighbours":
        a, b = slice(0, dims, 2), slice(1, dims, 2)
    elif layout == "halves":
        a, b = slice(0, dims // 2), slice(dims // 2, dims)
    else:
        raise ValueError(layout)
    u, v = x[..., a], x[..., b]
    out[..., a] = u * cos - v * sin
    out[..., b] = v * cos + u * sin
    return out


# ---- what a position sees ---------------------------------------------------------------------------------------
def visible(n, window=None, keep_first=0):
    """[n, n] bool: query i sees key j when j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & ((i - j < window) | (j < keep_first))
    return seen


def softmax_with_sink(scores, seen, sink=None):
    """scores [H, n, n] -> weights over the visible keys; with `sink` [H] the denominator holds exp(sink_h) as well."""
    scores = scores.masked_fill(~seen[None], -math.inf)
    if sink is None:
        return torch.softmax(scores, dim=-1)
    both = torch.cat([scores, sink[:, None, None].expand(-1, scores.shape[1], 1)], dim=-1)
    return torch.softmax(both, dim=-1)[..., :-1]


# ---- latent attention -------------------------------------------------------------------------------------------
def latent_attention(h, w, p, m, eps, positions, layout):
    n = h.shape[0]
    H, d, r, e, Rc = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    hk = kept(h)
    cq = kept(rms_norm(hk @ w[p + "dq"].T, w[p + "dq.norm"], eps))
    q = (cq @ w[p + "uq"].T).reshape(n, H, d + r)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], positions, m["rot"], layout)
    z = hk @ w[p + "dkv"].T
    c = kept(rms_norm(z[:, :Rc], w[p + "dkv.norm"], eps))
    kr = kept(rotate(z[:, None, Rc:Rc + r], positions, m["rot"], layout)[:, 0])
    k_plain = (c @ w[p + "uk"].T).reshape(n, H, d)
    v = (c @ w[p + "uv"].T).reshape(n, H, e)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, kr)) * m["scale"]
    a = softmax_with_sink(scores, visible(n))
    o = torch.einsum("hij,jhe->ihe", a, v).reshape(n, H * e)
    return kept(o) @ w[p + "o"].T


# ---- grouped attention under a window that keeps the first tokens, with a sink and an output gate ------------------
def windowed_attention(h, w, p, m, positions):
    n = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    hk = kept(h)
    q = (hk @ w[p + "q"].T).reshape(n, H, d)
    k = (hk @ w[p + "k"].T).reshape(n, G, d)
    v = kept((hk @ w[p + "v"].T).reshape(n, G, e))
    if m.get("rot") and m["rot"].get("dims"):
        q, k = rotate(q, positions, m["rot"], "halves"), rotate(k, positions, m["rot"], "halves")
    q, k = kept(q), kept(k)
    group = torch.arange(H) // (H // G)
    scores = torch.einsum("ihd,jhd->hij", q, k[:, group]) * m["scale"]
    mask = m.get("mask")
    seen = visible(n, mask["size"], mask.get("keep_first", 0)) if mask else visible(n)
    a = softmax_with_sink(scores, seen, w.get(p + "sink"))
    o = torch.einsum("hij,jhe->ihe", a, v[:, group]).reshape(n, H * e)
    if p + "g" in w:
        o = kept(o) * torch.sigmoid(hk @ w[p + "g"].T)
    return kept(o) @ w[p + "o"].T


# ---- feed-forwards ----------------------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return kept(relu_squared(kept(h) @ w[p + "up"].T)) @ w[p + "down"].T


def gated_ff(h, w, p):
    hk = kept(h)
    return kept(silu(hk @ w[p + "gate"].T) * (hk @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, router):
    """(chosen [n, K], weights [n, K]): the scores are the sigmoids of the router's logits; the K largest are chosen
    (the lower index on a tie) and weigh as they are."""
    s = torch.sigmoid(kept(h) @ w[p + "router"].T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :router["top"]]
    return order, torch.gather(s, 1, order)


def routed_ff(h, w, p, mlp):
    """sum over the chosen experts of expert(weight * h): the weight scales what the expert reads."""
    chosen, weights = route(h, w, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for kk in range(chosen.shape[1]):
            out[t] += gated_ff(weights[t, kk] * kept(h[t:t + 1]), w, f"{p}e{int(chosen[t, kk])}.")[0]
    if mlp.get("shared"):
        out = out + gated_ff(h, w, p + "shared.")
    return out


def feed_forward(h, w, p, mlp):
    return dense_ff(h, w, p) if mlp["kind"] == "dense" else routed_ff(h, w, p, mlp)


# ---- several residual streams -----------------------------------------------------------------------------------
def streams_read(xs, w, p):
    """u = sum_s in[s] x_s.  xs [S, n, D]."""
    return torch.einsum("s,snd->nd", w[p + "in"], xs)


def streams_write(xs, y, w, p):
    """x_t <- sum_s mix[s, t] x_s + out[t] y, every new stream from the old ones."""
    return torch.einsum("st,snd->tnd", w[p + "mix"], xs) + w[p + "out"][:, None, None] * y[None]


# ---- the model --------------------------------------------------------------------------------------------------
def run_order(cfg):
    """Layer indices in the order they run: the stretch [start, stop) `times` times in a row, then the rest."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b = loop["start"], loop["stop"]
    return list(range(a)) + list(range(a, b)) * loop["times"] + list(range(b, n))


def mixer(kind, h, w, p, m, eps, positions):
    if kind == "latent_attention":
        return latent_attention(h, w, p, m, eps, positions, "neighbours")
    if kind == "latent_attention_2":
        return latent_attention(h, w, p, m, eps, positions, "halves")
    if kind == "attention":
        return windowed_attention(h, w, p, m, positions)
    raise ValueError(f"unknown mixer {kind!r}")


def forward(cfg: dict, w: dict, tokens, collect=None):
    """Logits [n, vocab] of one whole sequence.  `collect` (a list) receives the stream (the sum of the streams where
    there are several) after every layer run."""
    eps = cfg["norm"]["eps"]
    positions = list(range(len(tokens)))
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    S = cfg.get("streams")
    xs = torch.stack([x] * S) if S else None
    for i in run_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        subs = [("norm1", "hc1.", lambda hh: mixer(layer["type"], hh, w, p + "mix.", layer["mixer"], eps, positions))]
        if layer.get("mlp") is not None:
            subs.append(("norm2", "hc2.", lambda hh: feed_forward(hh, w, p + "mlp.", layer["mlp"])))
        for norm, hc, fn in subs:
            if S:
                y = fn(rms_norm(streams_read(xs, w, p + hc), w[p + norm], eps))
                xs = streams_write(xs, y, w, p + hc)
            else:
                x = x + fn(rms_norm(x, w[p + norm], eps))
        if collect is not None:
            collect.append((xs.sum(dim=0) if S else x).clone())
    if S:
        x = xs.sum(dim=0)
    return kept(rms_norm(x, w["final.norm"], eps)) @ w["head"].T


def rounding_noise(cfg, w, tokens, dtype=torch.bfloat16):
    """Per position, the largest difference between the logits with the 16-bit values rounded and the exact ones, as a
    fraction of the largest exact logit: (the largest over the positions, their median)."""
    exact = forward(cfg, w, tokens)
    with rounding_to(dtype):
        rounded = forward(cfg, w, tokens)
    per_row = (rounded - exact).abs().max(dim=1).values / exact.abs().max()
    return float(per_row.max()), float(per_row.median())


# ---- reading a model folder -------------------------------------------------------------------------------------
def read_folder(folder):
    """(cfg, w): config.json as a dict and every tensor of model.safetensors as float64 (own parser)."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    w = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = raw[8 + hlen + lo:8 + hlen + hi]
        if info["dtype"] == "BF16":
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).astype(np.float64))
        elif info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f4").astype(np.float64))
        elif info["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<i4").astype(np.int64))
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        w[name] = t.reshape(info["shape"])
    return cfg, w
