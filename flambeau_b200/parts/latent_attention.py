"""Attention over a cache of latents: one narrow row per token from which every head's key and value follow."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import KVRequirement, Mixer, TensorSpec
from .linear import Linear, concat_rows
from .spec import PartSpec, build_part, register_part


class LatentAttention(Mixer):
    """With H heads, d unrotated and r rotated query/key dimensions a head, value size e, latent sizes Rq and Rc:

        cq = rmsnorm(Wdq h) * wq;   q_h = Wuq_h cq = [qn_h : d | qr_h : r]
        [z : Rc | zr : r] = Wdkv h;  c = rmsnorm(z) * wc;  kr = rot(zr)        (one rotated key part for all heads)
        k_h = [Wuk_h c | kr];  v_h = Wuv_h c
        s_ij = scale * (qn_h . Wuk_h c_j + rot(qr_h) . kr_j)  over the keys with 0 <= i - j < window (0: all earlier)
        out = Wo ((softmax(s) v)_heads * sigmoid(Wg h))                       (`gate` False: no Wg, the heads as they are)

    Only [c | kr] is cached, once per token and not per head.  Keys and values are never formed: the query is carried
    into the latent (Wuk_h^T qn_h, a map per head) so that the attention runs as one shared key/value head of size
    Rc + r whose cache rows are keys and values at once, and Wuv_h is applied to the head's mix of latents afterwards
    (another map per head), which is the same arithmetic.  `shares_latent`: the mixer has no Wdkv; the layer call
    reads the cache that another call owns (LayerCall.cache_from), with its own Wuk, Wuv, queries and window.
    `keep_window`: how many keys the cache must keep (an owner whose readers look further back than itself).
    The position part turns the rotated part of a head: it hands out its tables (`half`, `prepare`) and says which
    dimensions form a pair (`pairing`: neighbours (2i, 2i + 1) or halves (i, i + half)).
    Rotation angles, both RMS norms, scores and softmax weights are float32 in both engine modes; the weights enter
    the product with the latents as two bfloat16 numbers each when serving.

    Tensors behind the prefix: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g (with `gate`), o."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, num_heads: int, head_dim: int, rot_dim: int,
                 value_dim: int, kv_rank: int, q_rank: int, window: int, scale: float, eps: float,
                 position: PartSpec | None = None, shares_latent: bool = False, keep_window: int | None = None,
                 init_std: float = 0.02, gate: bool = True):
        super().__init__(runtime, prefix)
        self.gate = bool(gate)
        self.width, self.H, self.d, self.r, self.e = int(width), int(num_heads), int(head_dim), int(rot_dim), int(value_dim)
        self.Rc, self.Rq, self.window = int(kv_rank), int(q_rank), int(window or 0)
        self.keep_window = self.window if keep_window is None else int(keep_window)
        self.scale, self.eps, self.init_std = float(scale), float(eps), init_std
        self.shares_latent = bool(shares_latent)
        self.hd = self.Rc + self.r                     # a cache row, and the size of the one key/value head
        self.position = build_part(position, runtime) if position is not None else None
        if self.position is not None and (not hasattr(self.position, "half") or self.position.head_dim != self.r):
            raise ValueError("latent attention: the position encoding turns the rotated part of a head and hands out "
                             "its tables (half, prepare)")
        self.proj = self.uq = self.o = self.uk_t = self.uv = self.q_norm = self.c_norm = None

    def children(self):
        return [self.position] if self.position is not None else []

    def cache_requirement(self):
        return KVRequirement(1, self.hd, self.keep_window, values_in_keys=True)

    def own_tensor_specs(self):
        p, init = self.prefix, ("normal", self.init_std)
        norm = ("one_plus_normal", 0.1)
        specs = {
            p + "dq": TensorSpec((self.Rq, self.width), init=init),
            p + "dq.norm": TensorSpec((self.Rq,), init=norm),
            p + "uq": TensorSpec((self.H * (self.d + self.r), self.Rq), init=init),
            p + "uk": TensorSpec((self.H * self.d, self.Rc), init=init),
            p + "uv": TensorSpec((self.H * self.e, self.Rc), init=init),
            p + "o": TensorSpec((self.width, self.H * self.e), init=init),
        }
        if self.gate:
            specs[p + "g"] = TensorSpec((self.H * self.e, self.width), init=init)
        if not self.shares_latent:
            specs[p + "dkv"] = TensorSpec((self.hd, self.width), init=init)
            specs[p + "dkv.norm"] = TensorSpec((self.Rc,), init=norm)
        return specs

    def own_bind(self, tensors):
        p = self.prefix
        stack = [tensors[p + "dq"]] + ([] if self.shares_latent else [tensors[p + "dkv"]]) + \
            ([tensors[p + "g"]] if self.gate else [])
        rows = sum(t.shape[0] for t in stack)
        self.kv_off = self.Rq
        self.gate_off = self.Rq + (0 if self.shares_latent else self.hd)
        if rows % 8:          # rows of zeros up to a multiple of 8, so that the product's float32 rows stay 16-byte aligned
            stack.append(torch.zeros((8 - rows % 8, self.width), dtype=stack[0].dtype, device=stack[0].device))
        self.proj = Linear(concat_rows(stack))
        self.uq = Linear(tensors[p + "uq"])
        self.o = Linear(tensors[p + "o"])
        # per head: the map that carries a query into the latent is Wuk_h^T, stored with the latent as its outputs
        self.uk_t = tensors[p + "uk"].view(self.H, self.d, self.Rc).transpose(1, 2).contiguous()     # [H, Rc, d]
        self.uv = tensors[p + "uv"].view(self.H, self.e, self.Rc).contiguous()                      # [H, e, Rc]
        self.q_norm = tensors[p + "dq.norm"].contiguous()
        self.c_norm = None if self.shares_latent else tensors[p + "dkv.norm"].to(self.q_norm.dtype).contiguous()

    def own_weights(self):
        return [self.proj.weight, self.uq.weight, self.uk_t, self.uv, self.o.weight]

    def forward(self, ctx, h, out, call):
        n, rt, b = ctx.n_tokens, self.runtime, ctx.batch
        cache = ctx.cache(call)
        if cache.k_pool is None or cache.writable == self.shares_latent:
            raise ValueError("latent attention: a mixer with a down-projection of its own owns its cache rows, one "
                             "without reads another call's")
        H, d, r, e, Rc, hd = self.H, self.d, self.r, self.e, self.Rc, self.hd
        pos = self.position
        half = pos.half if pos is not None else 0
        pairing = getattr(pos, "pairing", "neighbours")
        with ctx.ws.scope():
            slabs = ctx.ws.alloc((ctx.max_slabs, n, self.proj.out_features), torch.float32)
            parts = self.proj.slabs(ctx, h, slabs)
            stride = slabs.stride(0)
            cos, sin = pos.prepare(ctx) if half else (None, None)
            cq = ctx.ws.alloc((n, self.Rq), rt.dtype)
            ops.mla_latents(slabs[0], self.Rq, self.q_norm, cq, self.kv_off, Rc, r, self.c_norm, self.eps, cos, sin,
                            half, cache, b.positions, b.row_seq, rt.status, n_partials=parts, partial_stride=stride,
                            pairing=pairing)
            qs = ctx.ws.alloc((ctx.max_slabs, n, H * (d + r)), torch.float32)
            q_parts = self.uq.slabs(ctx, cq, qs)
            q = ctx.ws.alloc((n, H * hd), rt.dtype)
            ops.head_linear(qs[0], d + r, self.uk_t, q, hd, n, n_partials=q_parts, partial_stride=qs.stride(0),
                            cos=cos, sin=sin, half=half, rot=r, pairing=pairing)
            a = ctx.ws.alloc((n, H * hd), rt.dtype)
            ops.paged_attention(ctx, q, a, cache, H, 1, hd, self.window, self.scale, vd=hd, weights_float32=True)
            og = ctx.ws.alloc((n, H * e), rt.dtype)
            ops.head_linear(a, hd, self.uv, og, e, n, gate=slabs[0] if self.gate else None, gate_off=self.gate_off,
                            gate_partials=parts, gate_partial_stride=stride)
            ctx.to_stream(self.o, og)


register_part("mixer", "latent_attention", LatentAttention)
