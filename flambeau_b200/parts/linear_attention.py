"""Gated linear attention: a recurrent mixer with a matrix of state per head and a decay per key channel."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, StateRequirement, TensorSpec
from .linear import Linear, concat_rows
from .spec import register_part


class GatedLinearAttention(Mixer):
    """With H heads, key size dk and value size dv:

        q = Wq h * dk^-1/2,  k = Wk h  [H][dk];   v = Wv h  [H][dv]                      (no biases)
        alpha = sigmoid(W2 (W1 h) + b)^(1/tau)  [H][dk]        (a map through a narrow middle; one decay per key channel)
        per head, token by token:  S <- diag(alpha) S + k v^T;  o = S^T q
        o <- o / sqrt(mean(o^2) + eps) * norm * silu(Wg h)_head                        (norm [dv] shared by the heads)
        out = Wo [o_0 ; ... ; o_{H-1}]

    S [dk, dv] starts at zero and is carried from step to step in float32 in the request's state slot.  Decays (formed
    as exp(log sigmoid(z) / tau)), the recurrence and the head norm are float32 in both engine modes.  The five input
    maps (q, k, v, gate, W1) are one stacked product; W2 is applied to its float32 result.  The width of the middle
    is the size of the tensors a1 / a2 (no configuration key gives it; `decay_rank` is what the random-weights mode
    draws).

    Tensors behind the prefix: q, k, v, g, o, norm [dv], a1 [R, width], a2 [H*dk, R], a2.b [H*dk]."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, num_heads: int, key_dim: int, value_dim: int,
                 tau: float, eps: float = 1e-6, decay_rank: int = 16, init_std: float = 0.02):
        super().__init__(runtime, prefix)
        self.width, self.H, self.dk, self.dv = int(width), int(num_heads), int(key_dim), int(value_dim)
        self.tau, self.eps, self.rank, self.init_std = float(tau), float(eps), int(decay_rank), init_std
        if not self.tau > 0.0:
            raise ValueError("gated linear attention: tau must be positive")
        self.qk, self.vw = self.H * self.dk, self.H * self.dv
        self.state_floats = self.H * self.dk * self.dv
        self.proj = self.o = self.a2 = self.a2_b = self.norm = None

    def state_requirement(self):
        return StateRequirement((self.state_floats,), "float32")

    def own_tensor_specs(self):
        p, init = self.prefix, ("normal", self.init_std)
        return {
            p + "q": TensorSpec((self.qk, self.width), init=init),
            p + "k": TensorSpec((self.qk, self.width), init=init),
            p + "v": TensorSpec((self.vw, self.width), init=init),
            p + "g": TensorSpec((self.vw, self.width), init=init),
            p + "o": TensorSpec((self.width, self.vw), init=init),
            p + "norm": TensorSpec((self.dv,), init=("one_plus_normal", 0.1)),
            p + "a1": TensorSpec((self.rank, self.width), init=init, free_axes=(0,)),
            p + "a2": TensorSpec((self.qk, self.rank), init=("normal", 0.5), free_axes=(1,)),
            p + "a2.b": TensorSpec((self.qk,), init=("normal", 1.0)),
        }

    def own_bind(self, tensors):
        p = self.prefix
        a1, a2 = tensors[p + "a1"], tensors[p + "a2"]
        if a1.shape[0] != a2.shape[1]:
            raise ValueError(f"{p}a1 has {a1.shape[0]} outputs, {p}a2 takes {a2.shape[1]} inputs")
        self.rank = int(a1.shape[0])
        stack = [tensors[p + n] for n in ("q", "k", "v", "g", "a1")]
        rows = sum(t.shape[0] for t in stack)
        if rows % 8:          # rows of zeros up to a multiple of 8, so that the product's float32 rows stay 16-byte aligned
            stack.append(torch.zeros((8 - rows % 8, self.width), dtype=stack[0].dtype, device=stack[0].device))
        self.proj = Linear(concat_rows(stack))
        self.o = Linear(tensors[p + "o"])
        self.a2 = a2.contiguous()
        self.a2_b = tensors[p + "a2.b"].to(a2.dtype).contiguous()
        self.norm = tensors[p + "norm"]

    def own_weights(self):
        return [self.proj.weight, self.o.weight, self.a2]

    def forward(self, ctx, h, out, call):
        n = ctx.n_tokens
        rt, b = self.runtime, ctx.batch
        state = ctx.cache(call).state
        if state is None:
            raise ValueError("gated linear attention needs a state slot per request")
        state = state.view(state.shape[0], -1)
        H, dk, dv = self.H, self.dk, self.dv
        with ctx.ws.scope():
            slabs = ctx.ws.alloc((ctx.max_slabs, n, self.proj.out_features), torch.float32)
            parts = self.proj.slabs(ctx, h, slabs)
            stride = slabs.stride(0)
            qkv = ctx.ws.alloc((n, 2 * self.qk + self.vw), torch.float32)
            decay = ctx.ws.alloc((n, self.qk), torch.float32)
            ops.gla_prepare(slabs[0], self.a2, self.a2_b, self.tau, dk ** -0.5, qkv, decay, H, dk, dv,
                            n_partials=parts, partial_stride=stride)
            o = ctx.ws.alloc((n, self.vw), torch.float32)
            ops.gla_recurrent(qkv, decay, state, b, o, H, dk, dv)
            a = ctx.ws.alloc((n, self.vw), rt.dtype)
            ops.gdr_out_norm(o, slabs[0], 2 * self.qk + self.vw, self.norm, self.eps, a, H, dv, n_partials=parts,
                             partial_stride=stride)
            ctx.to_stream(self.o, a)


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
