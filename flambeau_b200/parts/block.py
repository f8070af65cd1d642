"""How a layer arranges its norms, mixer and feed-forward around the stream."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, StateRequirement, TensorSpec
from .spec import PartSpec, build_part, register_part


class ResidualStream:
    """The float32 stream x [n, width] plus the last part's output that has
    not been added yet (`pending`): the next norm adds it while it normalises,
    so the add costs no pass of its own.  `pending_slabs` > 1 says that the
    output is a sum of that many float32 slabs (split-K shares of the part's last
    product, ctx.delta_slabs[0..k)), which the norm adds as well; 0 says that the
    part's last product has added its result to x itself (ctx.to_stream), so the
    norm has nothing to add.  `pending_norm` (a norm part, or None) says that the pending output passes through that
    norm before it joins the stream; whoever adds the pending output applies it (Norm.add_norm(delta_norm=...)).
    `closer` (optional, set by a block arrangement that keeps the stream in another form, several copies of it, say):
    close(ctx) calls it once after the last block, and it leaves the stream as one x with nothing pending."""

    def __init__(self, x, pending=None, pending_slabs: int = 1, pending_norm=None):
        self.x, self.pending, self.pending_slabs, self.pending_norm = x, pending, pending_slabs, pending_norm
        self.closer = None

    def close(self, ctx) -> None:
        """After the last block: whatever form a block arrangement kept the stream in, it is one x again."""
        if self.closer is not None:
            closer, self.closer = self.closer, None
            closer(ctx, self)

    def settle(self, ctx) -> None:
        """Add what is pending to x now (through the pending norm's kernel, which then normalises nothing else), for
        a part that wants the whole stream rather than a normalised copy of it."""
        if self.pending is None or self.pending_slabs == 0:
            self.pending, self.pending_slabs, self.pending_norm = None, 0, None
            return
        if self.pending_norm is None:
            ops.add_slabs(self.x, self.pending, ctx.n_tokens, self.pending_slabs, ctx.delta_slabs.stride(0))
            self.pending, self.pending_slabs = None, 0
            return
        self.pending_norm.add_norm(ctx, self.x, self.pending, None, n_partials=self.pending_slabs,
                                   delta_norm=self.pending_norm)
        self.pending, self.pending_slabs, self.pending_norm = None, 0, None


class PreNormBlock(Part):
    """x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x))
    (crates/models/qwen35-v2/src/model.rs:25-42).  `feed_forward` (with its norm) may be None: the layer then ends
    behind the mixer.  `mixer_input` / `feed_forward_input` (parts of category 'input_map', optional): what the
    sublayer reads is made from the normalised rows by that part (a short convolution over time, say); the norm then
    leaves its rows in float32, so that the map's result is rounded once.  What such parts keep per request lies in
    the layer call's state slot behind the mixer's own state (float32 numbers: [mixer | mixer_input |
    feed_forward_input])."""
    graph_safe = True
    category = "block"

    def __init__(self, runtime=None, prefix="", *, mixer: PartSpec, mixer_norm: PartSpec,
                 feed_forward: PartSpec | None = None, feed_forward_norm: PartSpec | None = None,
                 mixer_input: PartSpec | None = None, feed_forward_input: PartSpec | None = None):
        super().__init__(runtime, prefix)
        self.mixer = build_part(mixer, runtime)
        self.mixer_norm = build_part(mixer_norm, runtime)
        self.mixer_input = build_part(mixer_input, runtime) if mixer_input is not None else None
        self.feed_forward = self.feed_forward_norm = self.feed_forward_input = None
        if feed_forward is not None:
            if feed_forward_norm is None:
                raise ValueError("a feed-forward behind a norm needs that norm")
            self.feed_forward = build_part(feed_forward, runtime)
            self.feed_forward_norm = build_part(feed_forward_norm, runtime)
            self.feed_forward_input = build_part(feed_forward_input, runtime) if feed_forward_input is not None else None
        elif feed_forward_input is not None:
            raise ValueError("an input map for a feed-forward that the layer does not have")
        # where the input maps' numbers begin in the layer call's state slot
        own = self.mixer.state_requirement()
        kept = [m.state_floats() for m in (self.mixer_input, self.feed_forward_input) if m is not None]
        self._state = own
        self._offsets = (0, 0)
        if sum(kept) > 0:
            if own is not None and (own.dtype != "float32" or len(own.shape) != 1):
                raise ValueError("input maps keep their numbers behind the mixer's state, which must then be one flat "
                                 "float32 array")
            base = own.shape[0] if own is not None else 0
            first = self.mixer_input.state_floats() if self.mixer_input is not None else 0
            self._offsets = (base, base + first)
            self._state = StateRequirement((base + sum(kept),), "float32")

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer_input, self.mixer, self.feed_forward_norm,
                            self.feed_forward_input, self.feed_forward) if p is not None]

    def state_requirement(self):
        return self._state

    def _normed_input(self, ctx, norm, input_map, offset, stream, call, h):
        """h = input_map(norm(x + pending)) (or the norm alone), the pending output added to the stream on the way."""
        if input_map is None:
            norm.add_norm(ctx, stream.x, stream.pending, h, n_partials=stream.pending_slabs,
                          delta_norm=stream.pending_norm)
            return
        with ctx.ws.scope():
            rows = ctx.ws.alloc((ctx.n_tokens, stream.x.shape[1]), torch.float32)
            norm.add_norm(ctx, stream.x, stream.pending, rows, n_partials=stream.pending_slabs,
                          delta_norm=stream.pending_norm)
            state = ctx.cache(call).state
            input_map.forward(ctx, rows, h, state.view(state.shape[0], -1) if state is not None else None, offset)

    def forward(self, ctx, stream: ResidualStream, call) -> None:
        h, delta = ctx.normed, ctx.delta
        ctx.stream_x = stream.x
        self._normed_input(ctx, self.mixer_norm, self.mixer_input, self._offsets[0], stream, call, h)
        stream.pending_norm = None
        ctx.pending_slabs = 1                 # a part that leaves split-K shares in ctx.delta_slabs says how many
        self.mixer.forward(ctx, h, delta, call)
        stream.pending, stream.pending_slabs = delta, ctx.pending_slabs
        if self.feed_forward is not None:
            self._normed_input(ctx, self.feed_forward_norm, self.feed_forward_input, self._offsets[1], stream, call, h)
            ctx.pending_slabs = 1
            self.feed_forward.forward(ctx, h, delta)
            stream.pending, stream.pending_slabs = delta, ctx.pending_slabs
        ctx.stream_x = None                   # another kind of block decides for itself whether parts may add to its stream


class DepthAveragedBlock(Part):
    """A block whose result is not handed on as it is: the model keeps what every block so far has produced, X_0 (the
    embedding output) to X_depth-1 (this block's result, the stream with everything added), and the next block reads
    x = sum_j w[j] X_j with this block's own learned weights `<prefix><weight_name>` [depth].  `block` is the block
    that does the layer's work; `depth` counts the kept results including this block's; `slots` is how many the
    model keeps in all (its layer calls + 1).  The kept results live for one step (float32 [slots, rows, width])."""
    graph_safe = True
    category = "block"
    HISTORY = "depth_average.history"

    def __init__(self, runtime=None, prefix="", *, block: PartSpec, depth: int, slots: int, width: int,
                 weight_name: str = "dwa"):
        super().__init__(runtime, prefix)
        self.inner = build_part(block, runtime)
        self.depth, self.slots, self.width, self.weight_name = int(depth), int(slots), int(width), weight_name
        if not 2 <= self.depth <= self.slots:
            raise ValueError(f"depth = {self.depth} of {self.slots} kept results")
        self.weight = None

    @property
    def mixer(self):
        return self.inner.mixer

    @property
    def feed_forward(self):
        return self.inner.feed_forward

    def state_requirement(self):
        inner = self.inner
        return inner.state_requirement() if hasattr(inner, "state_requirement") else inner.mixer.state_requirement()

    def children(self):
        return [self.inner]

    def own_tensor_specs(self):
        # (the newest result gets most of the weight, so that random weights still behave like a residual stream)
        return {self.prefix + self.weight_name: TensorSpec((self.depth,), init=("depth_mix", 0.1))}

    def own_bind(self, tensors):
        self.weight = tensors[self.prefix + self.weight_name].contiguous()

    def own_weights(self):
        return [self.weight]

    def forward(self, ctx, stream: ResidualStream, call) -> None:
        n = ctx.n_tokens
        history = ctx.shared.get(self.HISTORY)
        if history is None:
            stream.settle(ctx)
            history = ctx.shared[self.HISTORY] = ctx.step_alloc((self.slots, n, self.width), torch.float32)
            history[0].copy_(stream.x[:n])
        self.inner.forward(ctx, stream, call)
        if stream.pending_norm is not None:
            stream.settle(ctx)
        pending = stream.pending if stream.pending_slabs > 0 else None
        ops.depth_average(stream.x, pending, stream.pending_slabs if pending is not None else 0,
                          ctx.delta_slabs.stride(0), history, self.depth, self.weight, n)
        stream.pending, stream.pending_slabs, stream.pending_norm = None, 0, None


class SandwichNormBlock(Part):
    """A norm before and behind each sublayer:
        x = x + mixer_post_norm(mixer(mixer_norm(x)));  x = x + feed_forward_post_norm(feed_forward(feed_forward_norm(x)))
    `feed_forward` (with its two norms) may be None: the layer then ends behind the mixer.  A sublayer's output is
    left pending with its post norm; the next norm's kernel normalises it, adds it to the stream and normalises the
    stream for the next sublayer in one pass.  No product adds to the stream by itself here (ctx.stream_x stays
    None): what joins the stream is the normalised output, not the output."""
    graph_safe = True
    category = "block"

    def __init__(self, runtime=None, prefix="", *, mixer: PartSpec, mixer_norm: PartSpec, mixer_post_norm: PartSpec,
                 feed_forward: PartSpec | None = None, feed_forward_norm: PartSpec | None = None,
                 feed_forward_post_norm: PartSpec | None = None):
        super().__init__(runtime, prefix)
        self.mixer = build_part(mixer, runtime)
        self.mixer_norm = build_part(mixer_norm, runtime)
        self.mixer_post_norm = build_part(mixer_post_norm, runtime)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if feed_forward is not None:
            if feed_forward_norm is None or feed_forward_post_norm is None:
                raise ValueError("a feed-forward between two norms needs both of them")
            self.feed_forward = build_part(feed_forward, runtime)
            self.feed_forward_norm = build_part(feed_forward_norm, runtime)
            self.feed_forward_post_norm = build_part(feed_forward_post_norm, runtime)

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm,
                            self.feed_forward, self.feed_forward_post_norm) if p is not None]

    def forward(self, ctx, stream: ResidualStream, call) -> None:
        h, delta = ctx.normed, ctx.delta
        ctx.stream_x = None
        self.mixer_norm.add_norm(ctx, stream.x, stream.pending, h, n_partials=stream.pending_slabs,
                                 delta_norm=stream.pending_norm)
        ctx.pending_slabs = 1
        self.mixer.forward(ctx, h, delta, call)
        stream.pending, stream.pending_slabs, stream.pending_norm = delta, ctx.pending_slabs, self.mixer_post_norm
        if self.feed_forward is None:
            return
        self.feed_forward_norm.add_norm(ctx, stream.x, stream.pending, h, n_partials=stream.pending_slabs,
                                        delta_norm=stream.pending_norm)
        ctx.pending_slabs = 1
        self.feed_forward.forward(ctx, h, delta)
        stream.pending, stream.pending_slabs, stream.pending_norm = delta, ctx.pending_slabs, self.feed_forward_post_norm


class HyperConnectionBlock(Part):
    """A pre-norm layer on S copies of the residual stream (hyper-connections).  All copies start as the stream the
    first such block finds.  Sublayer q (the mixer, then the feed-forward) with its learned weights in_q [S],
    mix_q [S, S] (indexed [from, to]) and out_q [S]:

        u = sum_s in_q[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + out_q[t] y   for all t at once

    After the last block the stream is the sum of the copies.  The copies are float32 and live for the step
    ([S, rows, width]); one kernel per sublayer does the write of the sublayer before it (whose output is left
    pending, as split-K shares where its last product left them), this sublayer's read and its RMS norm; a norm of
    another kind gets the read as float32 rows and normalises them itself.  No product adds to a stream by itself here
    (ctx.stream_x stays None): what joins a copy is out_q[t] times the output.  `feed_forward` (with its norm) may be
    None.  Tensors behind the prefix: `<names[0]>in`, `<names[0]>mix`, `<names[0]>out` for the mixer and the same
    under names[1] for the feed-forward."""
    graph_safe = True
    category = "block"
    STREAMS = "hyper_connections.streams"

    def __init__(self, runtime=None, prefix="", *, streams: int, width: int, mixer: PartSpec, mixer_norm: PartSpec,
                 feed_forward: PartSpec | None = None, feed_forward_norm: PartSpec | None = None,
                 names=("hc1.", "hc2.")):
        super().__init__(runtime, prefix)
        self.S, self.width, self.names = int(streams), int(width), tuple(names)
        if not 1 <= self.S <= 8:
            raise ValueError(f"hyper-connections: {self.S} streams (1 to 8)")
        self.mixer = build_part(mixer, runtime)
        self.mixer_norm = build_part(mixer_norm, runtime)
        self.feed_forward = self.feed_forward_norm = None
        if feed_forward is not None:
            if feed_forward_norm is None:
                raise ValueError("a feed-forward behind a norm needs that norm")
            self.feed_forward = build_part(feed_forward, runtime)
            self.feed_forward_norm = build_part(feed_forward_norm, runtime)
        self.weights = {}                   # (sublayer, 'in' | 'mix' | 'out') -> float32 tensor

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def _sublayers(self):
        return self.names if self.feed_forward is not None else self.names[:1]

    def own_tensor_specs(self):
        # (close to one plain residual stream per copy: reads average the copies, writes reach every copy, the mix is
        # near the identity, so that random weights still behave like a residual network)
        specs = {}
        for name in self._sublayers():
            p = self.prefix + name
            specs[p + "in"] = TensorSpec((self.S,), init=("normal_around", 1.0 / self.S, 0.1))
            specs[p + "out"] = TensorSpec((self.S,), init=("normal_around", 1.0, 0.1))
            specs[p + "mix"] = TensorSpec((self.S, self.S), init=("identity_plus_normal", 0.1))
        return specs

    def own_bind(self, tensors):
        for name in self._sublayers():
            for leaf in ("in", "mix", "out"):
                self.weights[(name, leaf)] = tensors[self.prefix + name + leaf].float().contiguous()   # float32 in both modes

    def own_weights(self):
        return list(self.weights.values())

    def _read(self, ctx, xs, stream, name, norm, h):
        """The pending output joins the copies, then h = norm(sum_s in[s] x_s)."""
        from .norms import RMSNorm
        n = ctx.n_tokens
        y, parts, written_by = stream.pending, stream.pending_slabs, getattr(stream, "pending_writer", None)
        if y is None or written_by is None:
            y, mix, out_w = None, None, None
        else:
            mix, out_w = written_by
        stride = ctx.delta_slabs.stride(0) if parts > 1 else 0
        in_w = self.weights[(name, "in")]
        if type(norm) is RMSNorm:
            ops.hc_step(xs, y, parts, stride, mix, out_w, in_w, norm.weight, norm.eps, norm.weight_offset, h, n)
        else:
            with ctx.ws.scope():
                u = ctx.ws.alloc((n, self.width), torch.float32)
                ops.hc_step(xs, y, parts, stride, mix, out_w, in_w, None, 0.0, 0.0, u, n)
                norm.normalize(ctx, u, h)
        stream.pending, stream.pending_slabs, stream.pending_writer = None, 0, None

    def _leave(self, ctx, stream, name, delta):
        stream.pending, stream.pending_slabs = delta, ctx.pending_slabs
        stream.pending_writer = (self.weights[(name, "mix")], self.weights[(name, "out")])

    @classmethod
    def _close(cls, ctx, stream):
        """x = the sum of the copies, the last sublayer's output written into them first."""
        xs = ctx.shared.pop(cls.STREAMS)
        y, parts, writer = stream.pending, stream.pending_slabs, getattr(stream, "pending_writer", None)
        mix, out_w = writer if (y is not None and writer is not None) else (None, None)
        if mix is None:
            y = None
        stride = ctx.delta_slabs.stride(0) if parts > 1 else 0
        ops.hc_step(xs, y, parts, stride, mix, out_w, None, None, 0.0, 0.0, stream.x, ctx.n_tokens, write_back=False)
        stream.pending, stream.pending_slabs, stream.pending_norm, stream.pending_writer = None, 0, None, None

    def forward(self, ctx, stream: ResidualStream, call) -> None:
        n = ctx.n_tokens
        xs = ctx.shared.get(self.STREAMS)
        if xs is None:
            # the first block of a step that keeps copies: every copy starts as the stream it finds
            stream.settle(ctx)
            xs = ctx.shared[self.STREAMS] = ctx.step_alloc((self.S, n, self.width), torch.float32)
            xs.copy_(stream.x[:n].unsqueeze(0).expand(self.S, n, self.width))
            stream.closer = HyperConnectionBlock._close
            stream.pending_writer = None
        elif xs.shape[0] != self.S:
            raise ValueError(f"hyper-connections: this block keeps {self.S} copies of the stream, the step has {xs.shape[0]}")
        h, delta = ctx.normed, ctx.delta
        ctx.stream_x = None
        self._read(ctx, xs, stream, self.names[0], self.mixer_norm, h)
        ctx.pending_slabs = 1
        self.mixer.forward(ctx, h, delta, call)
        self._leave(ctx, stream, self.names[0], delta)
        if self.feed_forward is not None:
            self._read(ctx, xs, stream, self.names[1], self.feed_forward_norm, h)
            ctx.pending_slabs = 1
            self.feed_forward.forward(ctx, h, delta)
            self._leave(ctx, stream, self.names[1], delta)


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "hyper_connections", HyperConnectionBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
register_part("block", "depth_averaged", DepthAveragedBlock)
