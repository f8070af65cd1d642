"""Norms with the residual add fused in front of them: RMSNorm, and a LayerNorm without bias."""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, TensorSpec
from .spec import register_part


class RMSNorm(Norm):
    """y = v * (w + weight_offset) / sqrt(mean(v^2) + eps) with v = x + delta.  The
    architecture built here uses the plain weight (weight_offset 0,
    crates/kernels-hip/src/kernels/rmsnorm_f16.cu:41-85); weight_offset 1 is
    the "1 + w" form some architectures store.  The sum, the mean and the
    product are float32; the stream x stays float32."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, eps: float, init=("one_plus_normal", 0.02),
                 weight_offset: float = 0.0, weight_name: str = "weight"):
        super().__init__(runtime, prefix)
        self.width, self.eps, self.init = int(width), float(eps), tuple(init)
        self.weight_offset = float(weight_offset)
        self.weight_name = weight_name           # the tensor is `<prefix><weight_name>`
        self.weight = None

    def own_tensor_specs(self):
        return {self.prefix + self.weight_name: TensorSpec((self.width,), init=self.init)}

    def own_bind(self, tensors):
        self.weight = tensors[self.prefix + self.weight_name]

    def own_weights(self):
        return [self.weight]

    def add_norm(self, ctx, x, delta, out, rows=None, n_partials: int = 1, delta_norm=None):
        """delta_norm (an RMSNorm, optional): the delta is normalised by it before it joins the stream, in the same
        kernel (blocks that put a norm behind each sublayer).  out = None: the stream is updated and nothing else."""
        if n_partials == 0 or delta is None:     # the stream already holds the sum
            delta, delta_norm = None, None
        stride = ctx.delta_slabs.stride(0) if n_partials > 1 else 0
        if delta_norm is not None:
            ops.norm_add_rms_norm(x, delta, delta_norm.weight, delta_norm.eps, delta_norm.weight_offset,
                                  self.weight if out is not None else None, self.eps, out, rows=rows,
                                  n_partials=n_partials, n_rows=ctx.n_tokens, partial_stride=stride,
                                  weight_offset=self.weight_offset)
            return
        if out is None:
            raise ValueError("add_norm without an output needs a delta that passes through a norm of its own")
        ops.add_rms_norm(x, delta, self.weight, self.eps, out, rows=rows, n_partials=n_partials,
                         n_rows=ctx.n_tokens, partial_stride=stride, weight_offset=self.weight_offset)

    def normalize(self, ctx, x, out):
        ops.add_rms_norm(x, None, self.weight, self.eps, out, n_rows=x.shape[0], weight_offset=self.weight_offset)


class LayerNorm(Norm):
    """y = (v - mean v) / sqrt(mean (v - mean v)^2 + eps) * w with v = x + delta: a norm that takes the mean off, with
    a weight and no bias.  Mean, variance (from the deviations) and the product are float32; the stream stays
    float32.  The tensor is `<prefix><weight_name>`."""
    graph_safe = True

    def __init__(self, runtime=None, prefix="", *, width: int, eps: float, init=("one_plus_normal", 0.02),
                 weight_name: str = "weight"):
        super().__init__(runtime, prefix)
        self.width, self.eps, self.init, self.weight_name = int(width), float(eps), tuple(init), weight_name
        self.weight = None

    def own_tensor_specs(self):
        return {self.prefix + self.weight_name: TensorSpec((self.width,), init=self.init)}

    def own_bind(self, tensors):
        self.weight = tensors[self.prefix + self.weight_name]

    def own_weights(self):
        return [self.weight]

    def add_norm(self, ctx, x, delta, out, rows=None, n_partials: int = 1, delta_norm=None):
        if delta_norm is not None:
            raise ValueError("the centring norm adds a part's output as it is; a norm behind the part is not fused here")
        if n_partials == 0 or delta is None:     # the stream already holds the sum
            delta = None
        stride = ctx.delta_slabs.stride(0) if n_partials > 1 else 0
        ops.add_layer_norm(x, delta, self.weight, self.eps, out, rows=rows, n_partials=n_partials,
                           n_rows=ctx.n_tokens, partial_stride=stride)

    def normalize(self, ctx, x, out):
        ops.add_layer_norm(x, None, self.weight, self.eps, out, n_rows=x.shape[0])


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
