"""Routed experts: a feed-forward of many small feed-forwards of which every token uses a few."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, TensorSpec
from .linear import Linear, concat_rows, interleave_rows
from .spec import PartSpec, build_part, register_part


class RoutedExperts(FeedForward):
    """d = sum over the token's `top` experts of share_e * expert_e(h)  (+ a shared expert)

    Router logits z = Wr h are float32.  Two rules turn them into a choice and shares:
      'softmax_of_chosen' (the default): the `top` experts with the largest z + br are chosen (the lower index wins a
        tie) and their shares are the softmax over the chosen logits only;
      'softmax_of_all': scores s = softmax(z) over all experts; the `top` largest of s + br are chosen (br only moves
        the choice); the shares are the chosen scores themselves over their sum (+ 1e-20), times `weight_scale`;
      'sigmoid': scores s = sigmoid(z), every logit by itself; the `top` largest of s + br are chosen; the shares are
        the chosen scores as they are, times `weight_scale`.
    `share_on_input`: the share multiplies what the expert reads instead of what it gives, d = sum expert_e(share_e h)
    (the rows are scaled as they are laid side by side in expert order; with experts that are not linear in their
    input this is another function than the weighted sum of outputs).
    An expert is Wdown act(Wup h) with `activation` one of kernels.ops.PLAIN_ACTIVATIONS, or, with `gated`,
    Wdown (act(Wgate h) * (Wup h)) with `activation` one of kernels.ops.ACTIVATIONS; experts have no biases.
    `identity` (a count): that many more router outputs, behind the experts', stand for experts without weights
    whose output is their input h itself (times the share).
    A shared expert runs for every token and is added: with `shared_inner`, one of the experts' plain form times
    sigmoid(w_sg . h), one number per token; with `shared` (a feed-forward PartSpec), that part's output as it is.

    Tensors behind the prefix: e<i>.up [inner, width], e<i>.down [width, inner] (gated: e<i>.gate as well), router
    [experts + identity, width], `bias_name` [experts + identity] (if router_bias), and with `shared_inner`
    shared.up, shared.down, shared.sg [1, width].

    How a step runs: the router's logits (and the shared expert's gate) as one product, the choice (one warp a token),
    a counting sort of the (token, choice) pairs into expert order
    with every expert's stretch padded to whole row tiles, two grouped products over that order (the first gathers
    the tokens' rows and applies the activation), and one kernel that brings the weighted outputs back to the
    tokens and adds the shared expert.  All sizes on the host are upper bounds, so nothing is read back and the
    step can be replayed from a CUDA graph."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, inner: int, experts: int, top: int,
                 activation: str = "relu_squared", shared_inner: int | None = None, router_bias: bool = True,
                 init_std: float = 0.02, router_std: float = 0.5, gated: bool = False,
                 rule: str = "softmax_of_chosen", weight_scale: float = 1.0, identity: int = 0,
                 bias_name: str = "router.b", shared: PartSpec | None = None, share_on_input: bool = False):
        super().__init__(runtime, prefix)
        self.width, self.inner, self.E, self.K = int(width), int(inner), int(experts), int(top)
        self.identity = int(identity)
        self.share_on_input = bool(share_on_input)
        if self.share_on_input and self.identity:
            raise ValueError("routed experts: shares on the experts' inputs and experts without weights do not go together")
        self.outputs = self.E + self.identity            # what the router tells apart
        if not 1 <= self.K <= self.outputs:
            raise ValueError(f"top = {self.K} of {self.outputs} experts")
        self.gated = bool(gated)
        if activation not in (ops.ACTIVATIONS if self.gated else ops.PLAIN_ACTIVATIONS):
            raise ValueError(f"routed experts: activation '{activation}' is not implemented")
        if rule not in ops.ROUTER_RULES:
            raise ValueError(f"routed experts: rule '{rule}' is not one of {sorted(ops.ROUTER_RULES)}")
        self.activation, self.rule, self.weight_scale = activation, rule, float(weight_scale)
        self.shared_inner = int(shared_inner) if shared_inner else 0
        if self.shared_inner and shared is not None:
            raise ValueError("routed experts: one shared expert, either of the experts' plain form or a part")
        if self.shared_inner and self.gated:
            raise ValueError("routed experts: beside gated experts the shared expert is a part of its own (`shared`)")
        self.shared = build_part(shared, runtime) if shared is not None else None
        self.router_bias, self.init_std, self.router_std = bool(router_bias), init_std, router_std
        self.bias_name = bias_name
        self.up = self.down = self.router = self.router_b = None
        self.shared_up = self.shared_down = None

    def children(self):
        return [self.shared] if self.shared is not None else []

    def own_tensor_specs(self):
        p, init = self.prefix, ("normal", self.init_std)
        specs = {}
        for e in range(self.E):
            if self.gated:
                specs[f"{p}e{e}.gate"] = TensorSpec((self.inner, self.width), init=init)
            specs[f"{p}e{e}.up"] = TensorSpec((self.inner, self.width), init=init)
            specs[f"{p}e{e}.down"] = TensorSpec((self.width, self.inner), init=init)
        specs[p + "router"] = TensorSpec((self.outputs, self.width), init=("normal", self.router_std))
        if self.router_bias:
            specs[p + self.bias_name] = TensorSpec((self.outputs,), init=("normal", 0.1))
        if self.shared_inner:
            specs[p + "shared.up"] = TensorSpec((self.shared_inner, self.width), init=init)
            specs[p + "shared.down"] = TensorSpec((self.width, self.shared_inner), init=init)
            specs[p + "shared.sg"] = TensorSpec((1, self.width), init=init)
        return specs

    def own_bind(self, tensors):
        p = self.prefix
        if self.gated:      # gate and up rows alternate, so that the product's epilogue finds a gate beside its up
            self.up = torch.stack([interleave_rows(tensors[f"{p}e{e}.gate"], tensors[f"{p}e{e}.up"])
                                   for e in range(self.E)]).contiguous()                           # [E, 2 inner, width]
        else:
            self.up = torch.stack([tensors[f"{p}e{e}.up"] for e in range(self.E)]).contiguous()    # [E, inner, width]
        self.down = torch.stack([tensors[f"{p}e{e}.down"] for e in range(self.E)]).contiguous()    # [E, width, inner]
        # the router and the shared expert's gate are one product: the gate's row lies behind the experts' rows
        # (then rows of zeros up to a multiple of 8, so that the product's float32 rows stay 16-byte aligned)
        rows = [tensors[p + "router"]]
        if self.shared_inner:
            rows.append(tensors[p + "shared.sg"].reshape(1, self.width).to(rows[0].dtype))
        have = sum(t.shape[0] for t in rows)
        if have % 8:
            rows.append(torch.zeros((8 - have % 8, self.width), dtype=rows[0].dtype, device=rows[0].device))
        self.router = Linear(concat_rows(rows))
        self.router_b = tensors[p + self.bias_name].to(rows[0].dtype).contiguous() if self.router_bias else None
        if self.shared_inner:
            self.shared_up = Linear(tensors[p + "shared.up"])
            self.shared_down = Linear(tensors[p + "shared.down"])

    def own_weights(self):
        # a step reads the router, the shared expert, and of the routed experts at most what its tokens choose
        w = [self.router.weight]
        if self.shared_inner:
            w += [self.shared_up.weight, self.shared_down.weight]
        return w

    def weight_bytes(self) -> int:
        per_expert = (self.up[0].numel() + self.down[0].numel()) * self.up.element_size()
        return super().weight_bytes() + self.K * per_expert         # one token's worth; a batch reads more experts

    def _shared_part(self, ctx, h, n):
        """The shared part's output: added to the stream by its own last product where that can be (None, 0, 0), else
        float32 shares in a buffer of its own (first share, how many, their stride)."""
        kept = (ctx.delta_slabs, ctx.delta, ctx.pending_slabs)
        sh = ctx.ws.alloc((ctx.max_slabs, n, self.width), torch.float32)
        ctx.delta_slabs, ctx.delta, ctx.pending_slabs = sh, sh[0], 1
        try:
            self.shared.forward(ctx, h, sh[0])
            parts = ctx.pending_slabs
        finally:
            ctx.delta_slabs, ctx.delta, ctx.pending_slabs = kept
        return (None, 1, 0) if parts == 0 else (sh[0], parts, sh.stride(0))

    def forward(self, ctx, h, out):
        n = ctx.n_tokens
        rt = self.runtime
        K, E, D = self.K, self.E, self.width
        pairs = n * K
        # (the second product's rows are the first one's output, whose width must suit the tensor cores too)
        on_tc = ops.grouped_tc_supported(h, self.up, h) and self.inner % 8 == 0
        tile = ops.grouped_tile(pairs, E, on_tc)
        max_tiles = ops.moe_max_tiles(pairs, E, tile)
        rows = max_tiles * tile
        with ctx.ws.scope():
            chosen = ctx.ws.alloc((n, K), torch.int32)
            share = ctx.ws.alloc((n, K), torch.float32)
            gate = ctx.ws.alloc((n,), torch.float32) if self.shared_inner else None
            z = ctx.ws.alloc((ctx.max_slabs, n, self.router.out_features), torch.float32)
            parts = self.router.slabs(ctx, h[:n], z)
            ops.moe_choose(z[0], self.router_b, self.outputs if self.shared_inner else -1, self.outputs, K, chosen,
                           share, gate, n_partials=parts, partial_stride=z.stride(0), rule=self.rule,
                           weight_scale=self.weight_scale)
            place_token = ctx.ws.alloc((rows,), torch.int32)
            pair_place = ctx.ws.alloc((pairs,), torch.int32)
            tile_expert = ctx.ws.alloc((max_tiles,), torch.int32)
            # (shares on the inputs: the gather wants to know which pair a place stands for)
            place_pair = ctx.ws.alloc((rows,), torch.int32) if self.share_on_input else None
            # (a choice beyond the experts that have weights gets no place: the combine hands the token's input on)
            ops.moe_sort(chosen, E, tile, place_token, pair_place, tile_expert, place_pair)
            act = ctx.ws.alloc((rows, self.inner), rt.dtype)
            scaled = dict(row_share=share.view(-1), row_pair=place_pair) if self.share_on_input else {}
            if self.gated:
                ops.grouped_gated_linear(h[:n], place_token, self.up, tile_expert, tile, act, self.activation, ctx,
                                         **scaled)
            else:
                ops.grouped_linear(h[:n], place_token, self.up, tile_expert, tile, act, self.activation, ctx, **scaled)
            y = ctx.ws.alloc((rows, D), torch.float32)
            ops.grouped_linear(act, None, self.down, tile_expert, tile, y, None, ctx)
            shared, shared_parts, shared_stride = None, 1, 0
            if self.shared_inner:
                z = ctx.ws.alloc((ctx.max_slabs, n, self.shared_inner), torch.float32)
                parts = self.shared_up.slabs(ctx, h[:n], z)
                a = ctx.ws.alloc((n, self.shared_inner), rt.dtype)
                ops.activation(z[0], a, self.activation, n_partials=parts, partial_stride=z.stride(0))
                sh = ctx.ws.alloc((ctx.max_slabs, n, D), torch.float32)
                shared_parts = self.shared_down.slabs(ctx, a, sh)
                shared, shared_stride = sh[0], sh.stride(0)
            elif self.shared is not None:
                shared, shared_parts, shared_stride = self._shared_part(ctx, h, n)
            ops.moe_combine(y, pair_place.view(n, K), None if self.share_on_input else share, shared, shared_parts,
                            shared_stride, gate, out, n, pass_on=h[:n] if self.identity else None)
        ctx.pending_slabs = 1


register_part("feed_forward", "routed_experts", RoutedExperts)
