"""A plain, slow implementation of the Fegizen design in float64 torch on the CPU: the oracle of the tests.

One function per mechanism; whole sequences only (no cache, no state slots, no batches, no portions), so that
whatever the engine does with pages, slots and schedules is compared with something that has none of them.  It shares
no code with the product path.  `cfg` is the parsed config.json (a dict); `w` maps tensor names to float64 tensors.

Notation: n tokens, D = width, T = taps of the convolution in front of every sublayer.  Latent attention: H heads,
d = unrotated and r = rotated query/key size of a head, e = value size, Rq and Rc the sizes of the query's and the
key/value's latent, W = window.  Linear attention: H heads, d = key size, e = value size.  Feed-forward: E experts
and I identity experts of which each token uses K.
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


def centred_norm(x, weight, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * weight over the last axis; no bias."""
    dev = x - x.mean(dim=-1, keepdim=True)
    return dev / torch.sqrt((dev * dev).mean(dim=-1, keepdim=True) + eps) * weight


def embed(tokens, table, scale):
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def add_time_conv(h, taps_w):
    """h [n, D] -> h + c with c_t = sum_j taps_w[:, j] * h_(t - T + 1 + j): every channel's own taps over the last T
    inputs (the last tap is the current token's), zeros before the sequence starts."""
    n, _ = h.shape
    T = taps_w.shape[1]
    out = h.clone()
    for t in range(n):
        for j in range(T):
            s = t - T + 1 + j
            if s >= 0:
                out[t] += taps_w[:, j] * h[s]
    return out


# ---- rotation -----------------------------------------------------------------------------------------------------
def rotary_frequencies(rot: dict):
    """(frequencies [dims/2], magnitude) of a rotation described by base, dims and an optional stretch `scaling`
    (factor, original, fast, slow): frequencies whose wavelength is long against `original` are divided by the factor,
    short ones stay, those between are blended linearly by their index; cos and sin are then both multiplied by
    0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def index_of(turns):                       # the (fractional) pair index whose wave makes `turns` turns over `original`
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(index_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x, positions, freqs, magnitude):
    """x [n, ..., m]: dimensions (2i, 2i + 1), i < len(freqs), are a pair that is turned by position * freqs[i] (and
    stretched by `magnitude`); dimensions from 2 len(freqs) on pass unchanged."""
    dims = 2 * freqs.numel()
    pos = torch.as_tensor(positions, dtype=F64)
    ang = pos[:, None] * freqs[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = (torch.cos(ang) * magnitude).reshape(shape), (torch.sin(ang) * magnitude).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ---- latent attention -------------------------------------------------------------------------------------------
def latent_keys(h, w, p, m, eps, positions):
    """(c [n, Rc], kr [n, r]): the normalised latent of keys and values and the one rotated key part all heads share."""
    Rc, r = m["kv_rank"], m["rot_dim"]
    z = kept(h) @ w[p + "dkv"].T
    c = unit_rms(z[:, :Rc], eps) * w[p + "dkv.norm"]
    freqs, mag = rotary_frequencies(m["rot"])
    kr = rotate_neighbours(z[:, Rc:Rc + r], positions, freqs, mag)
    return kept(c), kept(kr)


def latent_attention(h, w, p, m, eps, positions, latent=None):
    """Returns (output [n, D], (c, kr)).  `latent`: another layer's (c, kr) to read instead of forming one's own."""
    n = h.shape[0]
    H, d, r, e = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    Rc, W = m["kv_rank"], (m["mask"]["size"] if m.get("mask") else n)
    hk = kept(h)
    cq = kept(unit_rms(hk @ w[p + "dq"].T, eps) * w[p + "dq.norm"])
    q = (cq @ w[p + "uq"].T).reshape(n, H, d + r)
    freqs, mag = rotary_frequencies(m["rot"])
    q_plain, q_rot = q[..., :d], rotate_neighbours(q[..., d:], positions, freqs, mag)
    c, kr = latent if latent is not None else latent_keys(h, w, p, m, eps, positions)
    k_plain = (c @ w[p + "uk"].T).reshape(n, H, d)
    v = (c @ w[p + "uv"].T).reshape(n, H, e)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, kr)) * m["scale"]
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = (j <= i) & (i - j < W)
    scores = scores.masked_fill(~seen[None], -math.inf)
    a = torch.softmax(scores, dim=-1)
    o = torch.einsum("hij,jhe->ihe", a, v).reshape(n, H * e)
    o = kept(kept(o) * torch.sigmoid(hk @ w[p + "g"].T))
    return o @ w[p + "o"].T, (c, kr)


# ---- gated linear attention ---------------------------------------------------------------------------------------
def channel_decays(h, w, p, m):
    """alpha [n, H, d] = sigmoid(z)^(1/tau), z = W_a2 (W_a1 h) + b."""
    z = (kept(h) @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    return torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).reshape(h.shape[0], m["heads"], m["dim"])


def linear_attention_recurrence(q, k, v, alpha, state=None):
    """Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k, alpha [n, H, d], v [n, H, e]; the
    state [H, d, e] starts at zero.  Returns (o [n, H, e], the last state)."""
    n, H, d = q.shape
    e = v.shape[-1]
    S = torch.zeros(H, d, e, dtype=F64) if state is None else state.clone()
    o = torch.zeros(n, H, e, dtype=F64)
    for t in range(n):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    return o, S


def gated_linear_attention(h, w, p, m, eps):
    n = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    hk = kept(h)
    q = (hk @ w[p + "q"].T).reshape(n, H, d) * d ** -0.5
    k = (hk @ w[p + "k"].T).reshape(n, H, d)
    v = (hk @ w[p + "v"].T).reshape(n, H, e)
    o, _ = linear_attention_recurrence(q, k, v, channel_decays(h, w, p, m))
    o = unit_rms(o, eps) * w[p + "norm"]
    o = kept(o.reshape(n, H * e) * silu(hk @ w[p + "g"].T))
    return o @ w[p + "o"].T


# ---- feed-forwards ----------------------------------------------------------------------------------------------
def gated_ff(h, w, p, act):
    hk = kept(h)
    return kept(act(hk @ w[p + "gate"].T) * (hk @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, router):
    """(chosen [n, K], weights [n, K]): scores are the softmax of the router's logits over all experts, identity
    experts included; the K largest of scores + correction are chosen (the lower index on a tie); the weights are the
    chosen scores themselves, divided by their sum and multiplied by the router's scale."""
    K = router["top"]
    s = torch.softmax(kept(h) @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"] if p + "correction" in w else s
    order = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :K]
    picked = torch.gather(s, 1, order)
    return order, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * router.get("scale", 1.0)


def routed_ff(h, w, p, mlp):
    router = mlp["router"]
    E = router["experts"]
    chosen, weights = route(h, w, p, router)
    hk = kept(h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for kk in range(chosen.shape[1]):
            ex = int(chosen[t, kk])
            y = gated_ff(h[t:t + 1], w, f"{p}e{ex}.", silu)[0] if ex < E else hk[t]      # identity experts hand h on
            out[t] += weights[t, kk] * y
    if mlp.get("shared"):
        out = out + gated_ff(h, w, p + "shared.", silu)
    return out


# ---- the model --------------------------------------------------------------------------------------------------
def forward(cfg: dict, w: dict, tokens, collect=None, skip_mixers=()):
    """Logits [n, vocab] of one whole sequence.  `collect` (a list) receives what goes on to the next layer after
    every layer.  `skip_mixers`: layer indices whose mixer is left out (for tests that switch one side off)."""
    eps = cfg["norm"]["eps"]
    positions = list(range(len(tokens)))
    x = embed(tokens, w["embed"], cfg["embedding"]["scale"])
    history = [x]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = centred_norm(x, w[p + "norm1"], eps)
        if p + "canon1" in w:
            h = add_time_conv(h, w[p + "canon1"])
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            y, latents[i] = latent_attention(h, w, p + "mix.", m, eps, positions,
                                             latent=latents[src] if src is not None else None)
        elif layer["type"] in ("gla", "gla_2"):
            y = gated_linear_attention(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(f"layer {i}: unknown mixer {layer['type']!r}")
        if i not in skip_mixers:
            x = x + y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = centred_norm(x, w[p + "norm2"], eps)
            if p + "canon2" in w:
                h = add_time_conv(h, w[p + "canon2"])
            x = x + (gated_ff(h, w, p + "mlp.", gelu_tanh) if mlp["kind"] == "dense" else routed_ff(h, w, p + "mlp.", mlp))
        history.append(x)
        x = sum(w[p + "dwa"][j] * history[j] for j in range(i + 2))
        if collect is not None:
            collect.append(x.clone())
    return kept(centred_norm(x, w["final.norm"], eps)) @ w["head"].T * cfg.get("logit_scale", 1.0)


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
