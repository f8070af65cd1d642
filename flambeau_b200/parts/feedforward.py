"""Dense feed-forwards: gated (SiLU-gated in the architecture built here), and plain (one map, an activation, one map)."""
from __future__ import annotations

import os

import torch

from ..kernels import ops
from .base import FeedForward, TensorSpec
from .linear import Linear, interleave_rows
from .spec import register_part


class GatedMLP(FeedForward):
    """d = (act(h Wg^T) * (h Wu^T)) Wd^T, no bias, no routing
    (crates/forward/src/core/composites/dense_ffn.rs:116-186; act = SiLU
    there).  Gate and up weights are stacked at load, row by row alternately,
    so one product yields both and its epilogue can apply the activation to
    neighbouring outputs.  `activation` names one of the kernels' gate
    activations (kernels.ops.ACTIVATIONS)."""
    graph_safe = True

    DEFAULT_NAMES = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")

    def __init__(self, runtime=None, prefix="", *, width: int, inner: int, activation: str = "silu",
                 init_std: float = 0.02, names=DEFAULT_NAMES):
        super().__init__(runtime, prefix)
        self.names = tuple(names)                # what the gate, up and down tensors are called behind the prefix
        if len(self.names) != 3:
            raise ValueError("gated feed-forward: three tensor names wanted (gate, up, down)")
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"gated feed-forward: activation '{activation}' is not implemented "
                             f"({', '.join(sorted(ops.ACTIVATIONS))})")
        self.activation = activation
        self.width, self.inner, self.init_std = int(width), int(inner), init_std
        self.gate_up = self.down = None

    def own_tensor_specs(self):
        p, init = self.prefix, ("normal", self.init_std)
        gate, up, down = self.names
        return {
            p + gate: TensorSpec((self.inner, self.width), init=init),
            p + up: TensorSpec((self.inner, self.width), init=init),
            p + down: TensorSpec((self.width, self.inner), init=init),
        }

    def own_bind(self, tensors):
        p = self.prefix
        gate, up, down = self.names
        self.gate_up = Linear(interleave_rows(tensors[p + gate], tensors[p + up]))
        self.down = Linear(tensors[p + down])
        # Few rows (decoding): when the stacked matrix has at least as many 128-row tiles as the device has SMs,
        # one CTA per tile streams its rows over the whole of K and applies the activation in its epilogue; that
        # many CTAs draw the full memory bandwidth, and the separate activation kernel and the float32 shares it
        # would add are saved (measured on the 7B shape: 1 % of a step at 8 rows, 3 % at 64; a single row is no
        # faster that way and keeps the split).  Narrower matrices keep the split of K, which is what fills the
        # device for them.
        sms = torch.cuda.get_device_properties(self.gate_up.weight.device).multi_processor_count \
            if self.gate_up.weight.is_cuda else 0
        want = os.environ.get("FLAMBEAU_FFN_DECODE_EPILOGUE")
        self.decode_epilogue = (2 * self.inner // 128 >= sms > 0) if want is None else want != "0"

    def own_weights(self):
        return [self.gate_up.weight, self.down.weight]

    def forward(self, ctx, h, out):
        n = ctx.n_tokens
        with ctx.ws.scope():
            a = ctx.ws.alloc((n, self.inner), self.runtime.dtype)
            fused = ops.tc_supported(h, self.gate_up.weight, a)
            if n <= 64 and not (fused and self.decode_epilogue and n >= 2):
                # few rows: float32 split-K shares, added by the activation kernel
                gu = ctx.ws.alloc((ctx.max_slabs, n, 2 * self.inner), torch.float32)
                parts = self.gate_up.slabs(ctx, h, gu)
                ops.gate_mul(gu[0], a, n_partials=parts, partial_stride=gu.stride(0), activation=self.activation)
            elif fused:
                ops.gemm_tc_gated(h, self.gate_up.weight, a, self.runtime.status, self.activation)   # in the epilogue
            else:
                gu = ctx.ws.alloc((n, 2 * self.inner), self.runtime.dtype)
                self.gate_up(ctx, h, gu)
                ops.gate_mul(gu, a, activation=self.activation)
            ctx.to_stream(self.down, a)


class PlainMLP(FeedForward):
    """d = act(h Wu^T) Wd^T: no gate, no bias, no routing.  `activation` names one of the kernels' plain activations
    (kernels.ops.PLAIN_ACTIVATIONS: relu_squared, silu, gelu_tanh).  Over a prompt's portion the activation runs in
    the first product's epilogue; with few rows the product leaves float32 split-K shares and the activation kernel
    adds them.  `names`: what the up and down tensors are called behind the prefix."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, inner: int, activation: str = "relu_squared",
                 init_std: float = 0.02, names=("up", "down")):
        super().__init__(runtime, prefix)
        self.names = tuple(names)
        if len(self.names) != 2:
            raise ValueError("plain feed-forward: two tensor names wanted (up, down)")
        if activation not in ops.PLAIN_ACTIVATIONS or not ops.PLAIN_ACTIVATIONS[activation]:
            raise ValueError(f"plain feed-forward: activation '{activation}' is not implemented")
        self.activation = activation
        self.width, self.inner, self.init_std = int(width), int(inner), init_std
        self.up = self.down = None

    def own_tensor_specs(self):
        p, init = self.prefix, ("normal", self.init_std)
        up, down = self.names
        return {p + up: TensorSpec((self.inner, self.width), init=init),
                p + down: TensorSpec((self.width, self.inner), init=init)}

    def own_bind(self, tensors):
        up, down = self.names
        self.up = Linear(tensors[self.prefix + up])
        self.down = Linear(tensors[self.prefix + down])

    def own_weights(self):
        return [self.up.weight, self.down.weight]

    def forward(self, ctx, h, out):
        n = ctx.n_tokens
        with ctx.ws.scope():
            a = ctx.ws.alloc((n, self.inner), self.runtime.dtype)
            if n > 64 and ops.tc_supported(h, self.up.weight, a):
                ops.gemm_tc_act(h, self.up.weight, a, self.runtime.status, self.activation)       # in the epilogue
            else:
                z = ctx.ws.alloc((ctx.max_slabs, n, self.inner), torch.float32)
                parts = self.up.slabs(ctx, h, z)
                ops.activation(z[0], a, self.activation, n_partials=parts, partial_stride=z.stride(0))
            ctx.to_stream(self.down, a)


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "mlp", PlainMLP)
