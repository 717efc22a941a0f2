"""The recurrent block with a real-gated linear recurrent unit (RG-LRU), as a mixer with one number of state per
channel.

    y = gelu_tanh(Wy x + by)                                        the gate branch
    u = conv(Wx x + bx)                                             a causal convolution per channel over time
                                                                    (`conv_taps` taps, the last on the present token,
                                                                    bias `conv.b`, no activation)
    per block b of `blocks` equal blocks of channels:  r = sigmoid(Ra[b] u_b + ra),  i = sigmoid(Ri[b] u_b + ri)
    a = exp(-`decay_scale` r softplus(lam));   S_t = a S_(t-1) + sqrt(1 - a^2) (i u),   S = 0 before the first token
    out = Wo (S * y)

Both branches are one packed product.  Everything behind the convolution is float32: its output, the gate
products (this package's own kernel, the matrices kept transposed so that a warp reads whole lines), decays,
softplus, exponentials and the state; the scan multiplies by the gate branch and rounds once.  The state row of a
slot holds S and, behind it, the last conv_taps - 1 inputs of the convolution.  One scan kernel walks a
sequence's rows in order for prompts, portions and single tokens alike.
NikolayBlagoev/garlic-inference has no recurrent mixer.
"""
from __future__ import annotations

import torch

from ..cache import StateRequirement
from ..ops import kernels, linear
from ..weights.loader import TensorWant
from .base import Mixer, register_part, seq_spans_array
from .linear_attention import pack_rows


class RGLRU(Mixer):
    kind = "rglru"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        hid, W, B, K = (int(params[k]) for k in ("hidden_size", "width", "blocks", "conv_taps"))
        bw = W // max(B, 1)
        return {"y": TensorWant((W, hid)), "y.b": TensorWant((W,)), "x": TensorWant((W, hid)), "x.b": TensorWant((W,)),
                "conv": TensorWant((W, K), std_scale=8.0), "conv.b": TensorWant((W,)),
                "ra": TensorWant((B, bw, bw), std_scale=2.0), "ra.b": TensorWant((B, bw)),
                "ri": TensorWant((B, bw, bw), std_scale=2.0), "ri.b": TensorWant((B, bw)),
                "lam": TensorWant((W,), std_scale=20.0), "o": TensorWant((hid, W))}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden, self.W, self.B, self.K = (int(params[k]) for k in ("hidden_size", "width", "blocks", "conv_taps"))
        if self.B <= 0 or self.W % self.B:
            raise ValueError(f"{self.W} channels do not fall into {self.B} equal blocks")
        if not 1 <= self.K <= 16:
            raise ValueError(f"{self.K} taps are outside this library's 1 to 16")
        self.decay_scale = float(params.get("decay_scale", 8.0))
        self.w_in, (self.y_off, self.x_off) = pack_rows(load, [("y", self.W), ("x", self.W)], self.hidden, rt)
        f32 = lambda n: load(n).to(torch.float32).reshape(-1).contiguous()
        self.y_bias, self.x_bias, self.conv_bias = f32("y.b"), f32("x.b"), f32("conv.b")
        self.taps = load("conv")
        # [blocks, out, in] as stored -> [blocks, in, out]: thread o of a block reads w[k][o], a whole line per warp
        self.wa_t = load("ra").transpose(1, 2).contiguous()
        self.wi_t = load("ri").transpose(1, 2).contiguous()
        self.ba, self.bi, self.lam = f32("ra.b"), f32("ri.b"), f32("lam")
        self.w_o = load("o")
        self.state_floats = -(-(self.K * self.W) // 4) * 4          # S, then the last K - 1 inputs

    def cache_requirement(self):
        return StateRequirement((self.state_floats,), torch.float32)

    def step_arrays(self, shape, cache):
        return {} if shape.all_single else {"seq_spans": lambda: seq_spans_array(shape)}

    def pre_output(self, x, ctx, cache, position, writes_cache=True, out=None, out_mul=1.0):
        """S * gelu(gate branch): [n, width] in the activation type, into `out` when given."""
        if not writes_cache:
            raise ValueError("a mixer with state of its own cannot read another layer's")
        if out_mul != 1.0:
            raise ValueError("the recurrent block's result takes no factor")
        proj = linear(x, self.w_in)
        conv_in = proj[:, self.x_off:self.x_off + self.W]
        conv_state = cache.state[:, self.W:] if self.K > 1 else cache.state      # one tap: no inputs are kept
        u = kernels.causal_conv_silu(conv_in, self.taps, conv_state, ctx.tok_slot, activation="none",
                                     renew_state=ctx.all_single, in_bias=self.x_bias, out_bias=self.conv_bias)
        if not ctx.all_single and self.K > 1:
            kernels.conv_state_update(conv_in, self.K, conv_state, ctx.tok_slot, in_bias=self.x_bias)
        a, b = kernels.rglru_gates(u, self.wa_t, self.wi_t, self.ba, self.bi, self.lam, self.decay_scale)
        return kernels.rglru_scan(a, b, proj[:, self.y_off:self.y_off + self.W], self.y_bias, cache.state,
                                  ctx.seq_spans(), ctx.tok_slot, out=out)

    def step(self, x, ctx, cache, position, writes_cache=True):
        return linear(self.pre_output(x, ctx, cache, position, writes_cache), self.w_o)


register_part(RGLRU.kind, RGLRU)
