"""Feed-forwards.

`xielu_mlp`: down( a(up(x)) ), no biases, with the xIELU activation
    a(z) = softplus(p) z^2 + z/2                         for z > 0
           (1/2 + softplus(q)) (e^z - 1 - z) + z/2       for z <= 0
whose two numbers (p, q) are a tensor of the layer; float32 inside, one
rounding.  Upstream has no such feed-forward.

`swiglu_mlp`, the SwiGLU feed-forward: down( silu(gate(x)) * up(x) ), no biases
(src/models/qwen3/qwen3.cpp:186-203).  gate and up are packed into one weight
at load time (one product instead of two); silu and the product are one kernel
in float32 with a single rounding (upstream rounds after silu and again after
the product, src/src-cuda/activations/silu.cu:35-67, hadamard.cu:48-67).

`glu_mlp`: down( act(gate(x)) * up(x) ) with `activation` "silu", "gelu_tanh" (the tanh form of gelu,
0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))) or "swish" (z sigmoid(`swish_alpha` z)); gate and up packed
like SwiGLU's.  Optional limits make it down( act(min(gate x, `gate_max`)) * (clamp(up x, -`up_limit`, `up_limit`)
+ `up_shift`) ).  With "silu" and no limits it runs SwiGLU's fused products.  `pre_output` hands over what goes
into the down projection, for arrangements that join it with another product."""
from __future__ import annotations

import torch

from ..ops import glu_product, kernels, linear, swiglu_product
from ..weights.loader import TensorWant
from .base import FeedForward, register_part


class SwiGLUMLP(FeedForward):
    kind = "swiglu_mlp"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        h, i = params["hidden_size"], params["intermediate_size"]
        return {"gate_proj": TensorWant((i, h)), "up_proj": TensorWant((i, h)), "down_proj": TensorWant((h, i))}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.w_gate_up = torch.empty((2 * self.inter, self.hidden), dtype=load.dtype("gate_proj", "up_proj"),
                                     device=rt.device)
        load("gate_proj", out=self.w_gate_up[:self.inter])
        load("up_proj", out=self.w_gate_up[self.inter:])
        self.w_down = load("down_proj")

    def step(self, x, ctx):
        return linear(swiglu_product(x, self.w_gate_up), self.w_down)


class GluMLP(FeedForward):
    kind = "glu_mlp"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        h, i = params["hidden_size"], params["intermediate_size"]
        return {"gate": TensorWant((i, h)), "up": TensorWant((i, h)), "down": TensorWant((h, i))}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.activation = params.get("activation", "silu")
        if self.activation not in kernels.GLU_KINDS:
            raise ValueError(f"glu_mlp activation {self.activation!r} is none of {sorted(kernels.GLU_KINDS)}")
        self.unit = kernels.glu_shape(self.activation, params.get("swish_alpha", 1.0), params.get("gate_max"),
                                      params.get("up_limit"), params.get("up_shift", 0.0))
        self.plain_silu = self.unit == kernels.glu_shape("silu")
        self.w_gate_up = torch.empty((2 * self.inter, self.hidden), dtype=load.dtype("gate", "up"), device=rt.device)
        load("gate", out=self.w_gate_up[:self.inter])
        load("up", out=self.w_gate_up[self.inter:])
        self.w_down = load("down")

    def pre_output(self, x, ctx, out=None):
        """unit(gate x, up x): [n, intermediate_size] in the activation type, into `out` (columns of a wider matrix)
        when given."""
        if self.plain_silu and out is None:
            return swiglu_product(x, self.w_gate_up)
        return glu_product(x, self.w_gate_up, self.unit, out=out)

    def step(self, x, ctx):
        return linear(self.pre_output(x, ctx), self.w_down)


class XieluMLP(FeedForward):
    kind = "xielu_mlp"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        h, i = params["hidden_size"], params["intermediate_size"]
        return {"up": TensorWant((i, h)), "down": TensorWant((h, i)), "act": TensorWant((2,), std_scale=10.0)}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.w_up, self.w_down, self.act = load("up"), load("down"), load("act")

    def step(self, x, ctx):
        return linear(kernels.xielu(linear(x, self.w_up), self.act), self.w_down)


register_part(SwiGLUMLP.kind, SwiGLUMLP)
register_part(GluMLP.kind, GluMLP)
register_part(XieluMLP.kind, XieluMLP)
