"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import KVRequirement, Mixer, TensorSpec
from .linear import Linear, concat_rows
from .spec import PartSpec, build_part, register_part


class PagedAttention(Mixer):
    """q, k, v = h Wq^T, h Wk^T, h Wv^T (no bias); position encoding on q and k
    after the projection and before the cache write; every query at position p
    attends to the cached keys [max(0, p-W+1), p] of its request (all of [0, p]
    when window == 0) with scores scale * q.k; o = a Wo^T.
    crates/forward/src/core/composites/standard_attn.rs:197-286 (projections),
    :355-399 (rotary), :418-420 (scale), :1261-1302 (output projection).

    Sizes are parameters: `num_heads * head_dim` need not equal `width`.
    `qk_norm` (optional, a norm PartSpec of width head_dim): a norm over every
    head of q and of k between the projection and the rotation, with weights
    `<prefix>q_norm.weight` and `<prefix>k_norm.weight` (the optional
    attn_q_norm / attn_k_norm of crates/forward/src/ctx.rs:368-369; the
    architecture built here has none).
    `distance_slopes` (optional, one number per query head): slope * (key
    position - query position) is added to every scaled score, a linear
    penalty on distance that a position scheme without rotation can be built
    from (the architecture built here has none; portions of prompts then run
    on the mma.sync kernel, which has the hook).
    `qk_norm_reach`: 'head' (the default: every head of q and of k is normalised alone, weights of head_dim) or
    'projection' (one norm over all of q and one over all of k before they are split into heads, weights of
    num_heads * head_dim and num_kv_heads * head_dim).
    `value_dim`: the size of a value row where it is not head_dim; the output projection then takes
    num_heads * value_dim columns.
    `sink` (bool): the softmax of every head has one more slot, a learned score per head (`<prefix><names.sink>`,
    [num_heads]) that is not scaled, has no key and no value, and counts once in the denominator.
    `weights_float32`: the softmax weights keep 16 bits of mantissa through the product with the values when serving
    in bfloat16 (two bfloat16 numbers a weight, two MMAs for one; the 32-bit mode has them in float32 anyway), for
    designs that say their attention weights are 32-bit numbers; otherwise they are rounded to bfloat16 for that
    product, as flash attention kernels do.
    `keep_first` (with a window): the keys at positions below this stay visible to every later query, each with the
    position it was written at (which its rotation and the window's distances use); the pages that hold them are kept
    while the request lives, whatever the window gives back behind them.
    `gate` (bool): the heads' outputs are multiplied element by element by sigmoid(Wg h) before the output projection
    (`<prefix><names.g>`, [num_heads * value_dim, width]; Wg reads the same input as the other projections and is
    part of their one product).
    `names`: what the tensors are called behind the prefix (keys q, k, v, o, q_norm, k_norm, sink, g), for checkpoints
    with other names than the defaults."""
    graph_safe = True

    DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                     "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "sink": "sinks", "g": "g_proj.weight"}

    def __init__(self, runtime=None, prefix="", *, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 window: int = 0, position: PartSpec | None = None, scale: float | None = None,
                 init_std: float = 0.02, qk_norm: PartSpec | None = None, distance_slopes=None,
                 qk_norm_reach: str = "head", value_dim: int | None = None, sink: bool = False, names=None,
                 weights_float32: bool = False, keep_first: int = 0, gate: bool = False):
        super().__init__(runtime, prefix)
        self.gate = bool(gate)
        self.width, self.nh, self.nkv, self.hd = int(width), int(num_heads), int(num_kv_heads), int(head_dim)
        self.vd = int(value_dim) if value_dim else self.hd
        self.sink = bool(sink)
        self.weights_float32 = bool(weights_float32)
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(names or {})
        if qk_norm_reach not in ("head", "projection"):
            raise ValueError(f"qk_norm_reach = {qk_norm_reach!r}: 'head' or 'projection'")
        self.qk_norm_reach = qk_norm_reach
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} query heads are not a multiple of {self.nkv} key/value heads")
        self.window = int(window or 0)
        self.keep_first = int(keep_first or 0) if self.window else 0
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        self.position = build_part(position, runtime) if position is not None else None
        self.q_norm = self.k_norm = None
        if qk_norm is not None:
            def norm_part(name, width_of_projection):
                # "<base>.<leaf>" behind the mixer's prefix: the norm part gets the prefix up to the last dot and
                # the leaf as the name of its weight
                params = dict(qk_norm.params)
                base, _, leaf = self.names[name].rpartition(".")
                params.setdefault("weight_name", leaf)
                if qk_norm_reach == "projection":
                    params["width"] = width_of_projection
                return build_part(PartSpec(qk_norm.category, qk_norm.kind, params,
                                           prefix + (base + "." if base else "")), runtime)
            self.q_norm = norm_part("q_norm", self.nh * self.hd)
            self.k_norm = norm_part("k_norm", self.nkv * self.hd)
        self.init_std = init_std
        self.distance_slopes = None
        if distance_slopes is not None:
            slopes = [float(x) for x in distance_slopes]
            if len(slopes) != self.nh:
                raise ValueError(f"{len(slopes)} distance slopes for {self.nh} query heads")
            self.distance_slopes = torch.tensor(slopes, dtype=torch.float32,
                                                device=runtime.device if runtime is not None else "cpu")
        self.qw, self.kvw, self.vw = self.nh * self.hd, self.nkv * self.hd, self.nkv * self.vd
        self.qkv = self.o = self.sinks = None

    def children(self):
        return [p for p in (self.position, self.q_norm, self.k_norm) if p is not None]

    def cache_requirement(self):
        return KVRequirement(self.nkv, self.hd, self.window, v_head_dim=self.vd if self.vd != self.hd else 0,
                             keep_first=self.keep_first)

    def own_tensor_specs(self):
        p, init = self.prefix, ("normal", self.init_std)
        nm = self.names
        specs = {
            p + nm["q"]: TensorSpec((self.qw, self.width), init=init),
            p + nm["k"]: TensorSpec((self.kvw, self.width), init=init),
            p + nm["v"]: TensorSpec((self.vw, self.width), init=init),
            p + nm["o"]: TensorSpec((self.width, self.nh * self.vd), init=init),
        }
        if self.sink:
            specs[p + nm["sink"]] = TensorSpec((self.nh,), init=("normal", 1.0))
        if self.gate:
            specs[p + nm["g"]] = TensorSpec((self.nh * self.vd, self.width), init=init)
        return specs

    def own_bind(self, tensors):
        p, nm = self.prefix, self.names
        stack = [tensors[p + nm["q"]], tensors[p + nm["k"]], tensors[p + nm["v"]]]
        self.gate_off = sum(t.shape[0] for t in stack)          # the gate's columns lie behind q, k and v
        if self.gate:
            stack.append(tensors[p + nm["g"]])
        rows = sum(t.shape[0] for t in stack)
        if rows % 8 and (self.q_norm is not None or self.vd != self.hd) and self._fused_norm_kernel():
            # rows of zeros up to a multiple of 8, so that the product's float32 rows stay 16-byte aligned
            stack.append(torch.zeros((8 - rows % 8, self.width), dtype=stack[0].dtype, device=stack[0].device))
        self.qkv = Linear(concat_rows(stack))
        self.o = Linear(tensors[p + nm["o"]])
        if self.sink:
            self.sinks = tensors[p + nm["sink"]].float().contiguous()      # scores are float32 in both modes

    def own_weights(self):
        return [self.qkv.weight, self.o.weight]

    def _fused_norm_kernel(self) -> bool:
        """Whether the kernel that normalises, rotates and writes the cache in one pass serves this mixer: the norms
        (if any) are the framework's RMS norm and the position encoding hands out its tables."""
        from .norms import RMSNorm
        pos = self.position
        if pos is not None and not getattr(pos, "fused_with_cache_write", False):
            return False
        return all(n is None or type(n) is RMSNorm for n in (self.q_norm, self.k_norm))

    def forward(self, ctx, h, out, call):
        n = ctx.n_tokens
        rt = self.runtime
        cache = ctx.cache(call)
        with ctx.ws.scope():
            # the projection stays float32 until after the rotation, so q and k are rounded once
            pos = self.position
            fused = pos is None or getattr(pos, "fused_with_cache_write", False)
            # the fused rotary kernel adds split-K shares of the projection itself; a position encoding with a
            # rotate() of its own gets whole rows
            if (self.q_norm is not None or self.vd != self.hd) and self._fused_norm_kernel():
                # one product for q, k and v; one kernel adds its shares, normalises q and k (every head alone or
                # the whole projection at once), rotates them, rounds q and fills the cache's pages
                cols = self.qkv.out_features
                slabs = ctx.ws.alloc((ctx.max_slabs, n, cols), torch.float32)
                parts = self.qkv.slabs(ctx, h, slabs)
                q = ctx.ws.alloc((n, self.qw), rt.dtype)
                cos, sin = pos.prepare(ctx) if pos is not None else (None, None)
                qn = self.q_norm
                ops.qk_norm_rope_kv_write(
                    slabs[0], qn.weight if qn is not None else None,
                    self.k_norm.weight if qn is not None else None, self.qk_norm_reach if qn is not None else None,
                    qn.eps if qn is not None else 0.0, qn.weight_offset if qn is not None else 0.0, cos, sin,
                    pos.half if pos is not None else 0, q, cache, ctx.batch.positions, ctx.batch.row_seq, self.nh,
                    self.nkv, self.hd, self.vd, rt.status, n_partials=parts, partial_stride=slabs.stride(0))
                a = ctx.ws.alloc((n, self.nh * self.vd), rt.dtype)
                hint = self.o.weight if ctx.l2_hints and n <= 64 else None
                ops.paged_attention(ctx, q, a, cache, self.nh, self.nkv, self.hd, self.window, self.scale,
                                    next_weight=hint, score_slopes=self.distance_slopes, sinks=self.sinks, vd=self.vd,
                                    weights_float32=self.weights_float32, keep_first=self.keep_first)
                if self.gate:
                    ops.sigmoid_gate(a, slabs[0][:, self.gate_off:self.gate_off + self.nh * self.vd], n, parts,
                                     slabs.stride(0))
                ctx.to_stream(self.o, a)
                return
            if self.vd != self.hd or self.qk_norm_reach != "head":
                raise ValueError("attention: value rows of their own width, or a norm over the whole projection, "
                                 "need the framework's RMS norm and a position encoding that hands out its tables")
            if self.gate and self.q_norm is not None:
                raise ValueError("attention: an output gate beside query/key norms needs the framework's RMS norm and a "
                                 "position encoding that hands out its tables")
            if self.q_norm is None:
                qkv_slabs = ctx.ws.alloc((ctx.max_slabs if fused else 1, n, self.qkv.out_features), torch.float32)
                parts = self.qkv.slabs(ctx, h, qkv_slabs)
                stride = qkv_slabs.stride(0)
                qkv = qkv_slabs[0]
                q_in = qkv[:, :self.qw]
                k = qkv[:, self.qw:self.qw + self.kvw]
                v = qkv[:, self.qw + self.kvw:self.qw + 2 * self.kvw]
            else:
                # un-fused: three products from row slices of the stacked weight, so that the heads of q and of k
                # lie as rows of their own; each head is normalised, then everything goes on as before
                parts, stride = 1, 0
                w = self.qkv.weight
                qn, kn = ctx.ws.alloc((n, self.qw), torch.float32), ctx.ws.alloc((n, self.kvw), torch.float32)
                q_in, k = ctx.ws.alloc((n, self.qw), torch.float32), ctx.ws.alloc((n, self.kvw), torch.float32)
                v = ctx.ws.alloc((n, self.kvw), torch.float32)
                ops.linear(h, w[:self.qw], qn, ctx)
                ops.linear(h, w[self.qw:self.qw + self.kvw], kn, ctx)
                ops.linear(h, w[self.qw + self.kvw:], v, ctx)
                self.q_norm.normalize(ctx, qn.view(n * self.nh, self.hd), q_in.view(n * self.nh, self.hd))
                self.k_norm.normalize(ctx, kn.view(n * self.nkv, self.hd), k.view(n * self.nkv, self.hd))
            q = ctx.ws.alloc((n, self.qw), rt.dtype)
            b = ctx.batch
            if fused:
                cos, sin = pos.prepare(ctx) if pos is not None else (None, None)
                half = pos.half if pos is not None else 0
                ops.rope_kv_write(q_in, q, k, v, cos, sin, half, b.positions, b.row_seq, cache.block_table,
                                  cache.k_pool, cache.v_pool, cache.page_size, self.nh, self.nkv, self.hd,
                                  cache.writable, rt.status, n_partials=parts, partial_stride=stride,
                                  table_base=cache.table_base, table_head=cache.table_head)
            else:
                pos.rotate(ctx, q_in, k if cache.writable else None)
                ops.rope_kv_write(q_in, q, k, v, None, None, 0, b.positions, b.row_seq, cache.block_table,
                                  cache.k_pool, cache.v_pool, cache.page_size, self.nh, self.nkv, self.hd,
                                  cache.writable, rt.status, table_base=cache.table_base,
                                  table_head=cache.table_head)
            a = ctx.ws.alloc((n, self.qw), rt.dtype)
            # few rows: the attention kernel fetches the start of the output projection's weights into L2 at its end
            hint = self.o.weight if ctx.l2_hints and n <= 64 else None
            ops.paged_attention(ctx, q, a, cache, self.nh, self.nkv, self.hd, self.window, self.scale,
                                next_weight=hint, score_slopes=self.distance_slopes, sinks=self.sinks,
                                weights_float32=self.weights_float32, keep_first=self.keep_first)
            if self.gate:
                ops.sigmoid_gate(a, qkv_slabs[0][:, self.gate_off:self.gate_off + self.qw], n, parts, stride)
            ctx.to_stream(self.o, a)


register_part("mixer", "attention", PagedAttention)
