"""Rotary position encodings: split-half pairs, and neighbouring pairs with stretched frequencies."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import PositionEncoding
from .spec import register_part


class RotaryHalf(PositionEncoding):
    """Pair i in [0, rot/2) of a head is (x[i], x[i + rot/2]); its angle is
    pos * theta^(-2i/rot) (crates/kernels-hip/src/kernels/
    rope_neox_partial_f16.cu:39-52).  `rotary_dim` < head_dim leaves the tail
    of the head untouched.  The cos/sin tables of a step are computed once and
    shared by every layer that uses equal parameters."""
    graph_safe = True

    fused_with_cache_write = True      # the attention mixer may hand the tables to its fused kernel
    pairing = "halves"                 # which dimensions form pair i (kernels.ops.ROTARY_PAIRING)

    def __init__(self, runtime=None, prefix="", *, head_dim: int, theta: float, rotary_dim: int | None = None):
        super().__init__(runtime, prefix)
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.half = self.rotary_dim // 2
        self._inv_freq = None

    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq is None:
            i = torch.arange(self.half, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rotary_dim)
            self._inv_freq = inv.to(self.runtime.device)
        return self._inv_freq

    def prepare(self, ctx):
        """(cos, sin), float32 [n, rot/2], for the rows of this step."""
        key = ("rotary_half", self.theta, self.rotary_dim)
        hit = ctx.shared.get(key)
        if hit is None:
            n = ctx.n_tokens
            cos = ctx.step_alloc((n, self.half), torch.float32)
            sin = ctx.step_alloc((n, self.half), torch.float32)
            ops.rope_table(ctx.batch.positions[:n], self.inv_freq(), cos, sin)
            hit = ctx.shared[key] = (cos, sin)
        return hit

    def rotate(self, ctx, q, k):
        """In place on q [n, heads*head_dim] and k [n, kv_heads*head_dim]."""
        cos, sin = self.prepare(ctx)
        for t in (q, k):
            if t is None:
                continue
            heads = t.shape[1] // self.head_dim
            ops.rope_kv_write(t, t, None, None, cos, sin, self.half, None, None, None, None, None, 0,
                              heads, 0, self.head_dim, False, self.runtime.status)


class RotaryNeighbours(PositionEncoding):
    """Pair i in [0, rot/2) of a head is (x[2i], x[2i+1]); its angle is pos * f_i with f_i = theta^(-2i/rot).
    `rotary_dim` < head_dim leaves the tail of the head untouched.

    `stretch` (optional: factor, original, fast, slow) lengthens the slow waves so that positions beyond `original`
    stay within the angles seen in training: with index(t) = rot * ln(original / (2 pi t)) / (2 ln theta) the pair
    index whose wave makes t turns over `original` positions, lo = max(floor(index(fast)), 0),
    hi = min(ceil(index(slow)), rot - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency of
    pair i becomes f_i / factor * ramp_i + f_i * (1 - ramp_i), and cos and sin are both multiplied by
    0.1 ln(factor) + 1.  Frequencies are formed in float64 on the host; the tables of a step (angles reduced in
    float64, the factor folded in) are computed once and shared by every layer that uses equal parameters."""
    graph_safe = True

    fused_with_cache_write = False     # the split-half kernels do not take these tables; mixers that do ask prepare()
    pairing = "neighbours"             # which dimensions form pair i (kernels.ops.ROTARY_PAIRING)

    def __init__(self, runtime=None, prefix="", *, head_dim: int, theta: float, rotary_dim: int | None = None,
                 stretch: dict | None = None):
        super().__init__(runtime, prefix)
        self.head_dim, self.theta = int(head_dim), float(theta)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.half = self.rotary_dim // 2
        self.stretch = dict(stretch) if stretch else None
        self.magnitude = 1.0
        freqs = [self.theta ** (-2.0 * i / self.rotary_dim) for i in range(self.half)]
        if self.stretch:
            factor, original = float(self.stretch["factor"]), float(self.stretch["original"])
            rot = self.rotary_dim

            def index(turns):
                return rot * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
            lo = max(math.floor(index(float(self.stretch["fast"]))), 0)
            hi = min(math.ceil(index(float(self.stretch["slow"]))), rot - 1)
            ramps = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(self.half)]
            freqs = [f / factor * ramp + f * (1.0 - ramp) for f, ramp in zip(freqs, ramps)]
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self.frequencies = freqs
        self._inv_freq = None

    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq is None:
            self._inv_freq = torch.tensor(self.frequencies, dtype=torch.float64).to(self.runtime.device)
        return self._inv_freq

    def prepare(self, ctx):
        """(cos, sin), float32 [n, rot/2], for the rows of this step, the stretch's factor folded in."""
        key = ("rotary_neighbours", self.theta, self.rotary_dim, tuple(sorted((self.stretch or {}).items())))
        hit = ctx.shared.get(key)
        if hit is None:
            n = ctx.n_tokens
            cos = ctx.step_alloc((n, max(self.half, 1)), torch.float32)
            sin = ctx.step_alloc((n, max(self.half, 1)), torch.float32)
            if self.half:
                ops.rope_table(ctx.batch.positions[:n], self.inv_freq(), cos, sin, self.magnitude)
            hit = ctx.shared[key] = (cos, sin)
        return hit

    def rotate(self, ctx, q, k):
        """In place on float32 q [n, heads*head_dim] and k [n, kv_heads*head_dim]."""
        cos, sin = self.prepare(ctx)
        for t in (q, k):
            if t is not None:
                ops.rope_neighbours(t, cos, sin, self.half, t.shape[1] // self.head_dim, self.head_dim)


register_part("position", "rotary_half", RotaryHalf)
register_part("position", "rotary_neighbours", RotaryNeighbours)
