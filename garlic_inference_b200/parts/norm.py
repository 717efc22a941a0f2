"""Norms, each fused with the residual add that precedes it.

`rms_norm`: y = x * rsqrt(mean(x^2) + eps) * weight, the weight used as it is
(src/src-cuda/norm.cu:3-49; the add: norm.cu:51-101).  `size` and `eps` are
parameters; sums are float32.

`dyt_norm`, Dynamic Tanh: y = tanh(alpha x) * weight + bias with one learned
number alpha; it takes no mean and no variance, so a row's elements do not
depend on each other.  Upstream has no such norm.

`layer_norm`: y = (x - mean(x)) / sqrt(var(x) + eps) * weight (+ bias), var the
mean of the squared deviations.  Upstream has no such norm.

All take `delta_scale`, a factor per channel on the pending delta (blocks
with a learned layer scale), and `delta2`, a second pending result that joins
the stream with the first (blocks whose sublayers run side by side); the
layer norm adds both in its own kernel, the others settle the second first."""
from __future__ import annotations

from ..ops import kernels
from ..weights.loader import TensorWant
from .base import Norm, register_part


class RMSNorm(Norm):
    kind = "rms_norm"
    graph_safe = True
    takes_offset = True

    @classmethod
    def wanted(cls, params):
        return {"weight": TensorWant((params["size"],), "norm")}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = load("weight")

    def add_norm(self, delta, residual, rows=None, write_residual=True, delta_scale=None, delta2=None, offset=None):
        """normed(residual + delta (+ offset)) in the activation type.  The float32 sum is written back to
        `residual` unless `rows` picks rows or `write_residual` is False; `delta` may be None.  A scaled delta
        is added to the stream by a kernel of its own first (then the stream is written whatever was asked).
        `offset` [size] joins every row in the same kernel."""
        if delta2 is not None:
            kernels.residual_add(delta2, residual)
        if delta is not None and delta_scale is not None:
            kernels.residual_add_scaled(delta, delta_scale, residual)
            delta = None
        return kernels.add_rmsnorm(delta, residual, self.weight, self.eps, self.rt.dtype, rows=rows,
                                   write_residual=write_residual, offset=offset)


class DynamicTanhNorm(Norm):
    kind = "dyt_norm"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        n = params["size"]
        return {"weight": TensorWant((n,), "norm"), "bias": TensorWant((n,)), "alpha": TensorWant((), "norm")}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.size = int(params["size"])
        dtype = load.dtype("weight", "bias", "alpha")
        self.weight, self.bias = load("weight").to(dtype), load("bias").to(dtype)
        self.alpha = load("alpha").to(dtype).reshape(1)

    def add_norm(self, delta, residual, rows=None, write_residual=True, delta_scale=None, delta2=None):
        if delta2 is not None:
            kernels.residual_add(delta2, residual)
        return kernels.add_dyt(delta, delta_scale, residual, self.weight, self.bias, self.alpha, self.rt.dtype,
                               rows=rows, write_residual=write_residual)


class LayerNorm(Norm):
    kind = "layer_norm"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        w = {"weight": TensorWant((params["size"],), "norm")}
        if params.get("bias", False):
            w["bias"] = TensorWant((params["size"],))
        return w

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = load("weight")
        self.bias = load("bias").to(self.weight.dtype) if params.get("bias", False) else None

    def add_norm(self, delta, residual, rows=None, write_residual=True, delta_scale=None, delta2=None):
        """normed(residual + delta + delta2) in the activation type; the float32 sum goes back into `residual` unless
        `rows` picks rows or `write_residual` is False.  A scaled delta is added by a kernel of its own first."""
        if delta is not None and delta_scale is not None:
            kernels.residual_add_scaled(delta, delta_scale, residual)
            delta = None
        return kernels.add_layernorm(delta, residual, self.weight, self.bias, self.eps, self.rt.dtype, rows=rows,
                                     write_residual=write_residual, delta2=delta2)


register_part(RMSNorm.kind, RMSNorm)
register_part(LayerNorm.kind, LayerNorm)
register_part(DynamicTanhNorm.kind, DynamicTanhNorm)
