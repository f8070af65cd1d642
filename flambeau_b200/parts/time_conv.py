"""A short convolution over time in front of a sublayer."""
from __future__ import annotations

from ..kernels import ops
from .base import Part, TensorSpec
from .spec import register_part


class TimeConvResidual(Part):
    """out_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j): every channel of a sublayer's input is joined by a causal
    convolution of itself over the last `taps` tokens (its own weights per channel, no bias, the last tap the current
    token's, zeros before the request's first token).  The last taps - 1 inputs of a request are its state here
    (float32), so that a portion continues where the one before ended; one tap keeps nothing.  The sum is float32
    and is rounded once, to the engine's dtype.  The tensor is `<prefix><weight_name>` [width, taps]."""
    graph_safe = True
    category = "input_map"

    def __init__(self, runtime=None, prefix="", *, width: int, taps: int, weight_name: str = "conv",
                 init_std: float | None = None):
        super().__init__(runtime, prefix)
        self.width, self.taps, self.weight_name = int(width), int(taps), weight_name
        if self.taps < 1:
            raise ValueError("a convolution over time needs at least one tap")
        self.init_std = float(init_std) if init_std is not None else 0.5 / self.taps ** 0.5
        self.weight = self.weight_t = None

    def state_floats(self) -> int:
        return (self.taps - 1) * self.width

    def own_tensor_specs(self):
        return {self.prefix + self.weight_name: TensorSpec((self.width, self.taps), init=("normal", self.init_std))}

    def own_bind(self, tensors):
        self.weight = tensors[self.prefix + self.weight_name].contiguous()
        # tap by tap in float32 (exact), so that neighbouring channels' weights of one tap lie side by side
        self.weight_t = self.weight.t().float().contiguous()

    def own_weights(self):
        return [self.weight]

    def forward(self, ctx, h, out, state, offset: int) -> None:
        """h: float32 [n, width] normalised rows; out: [n, width] engine dtype; state: float32 [slots, floats] whose
        numbers from `offset` on are this part's."""
        ops.time_conv(h, self.weight_t, state, offset, ctx.batch, out, ctx.n_tokens)


register_part("input_map", "time_conv", TimeConvResidual)
