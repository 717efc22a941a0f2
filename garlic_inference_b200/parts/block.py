"""Arrangements of a layer's parts, and the two ends of the model.

`pre_norm_residual` (src/models/qwen3/qwen3.cpp:225-248):
    r = h;  x = norm_in(h);  r = mixer(x) + r;  x = norm_post(r);  h = ffn(x) + r
The residual stream is float32; each add happens inside the norm that
follows it, so the block takes and returns a pending `delta` (see base.py).
The feed-forward may be absent (then the mixer's result is returned pending).
A vector that the schedule adds to the stream before the layer
(`ctx.stream_offset`, a row of a `stream_offset` table) rides in the first
norm's kernel; the other arrangements add it with a kernel of its own.

`post_norm_gated_residual` (no upstream counterpart): the sublayers read the
stream itself and the norm sits on each sublayer's result, behind a gate that
is made from the sublayer's input:
    h += norm_mixer( sigmoid(G1 h + b1) * mixer(h) );  h += norm_ff( sigmoid(G2 h + b2) * ffn(h) )
Gate, norm and add are one float32 kernel, which also leaves the new stream
in the activation type for the products that read it next; nothing is pending
when the block returns.  The feed-forward and either gate may be absent.

`pre_norm_scaled_residual` (no upstream counterpart): pre-norm with a learned factor per channel (layer
scale) on each sublayer's result:
    h += s1 * mixer(norm_in(h));  h += s2 * ffn(norm_post(h))
The scaled add happens inside the norm that follows, in float32; the block returns its last result pending and
leaves the factor it still has to be multiplied by in `ctx.delta_scale`.  The feed-forward may be absent.

`parallel_residual` (no upstream counterpart): one norm, read by the mixer and the feed-forward alike, whose
results join the stream together:
    x = norm_in(h);  h += mixer(x) + ffn(x)
Both results stay pending (`ctx.delta_extra` carries the second) and the next norm adds them in float32.  When
both sublayers end in an output projection and can hand over what goes into it (`pre_output` with `w_o` /
`w_down`), the two projections and the sum are one product over activations and weights laid side by side, summed
in float32 inside the product.  The feed-forward may be absent.
"""
from __future__ import annotations

import torch

from ..ops import kernels, linear
from ..weights.loader import TensorWant
from .base import Block, Embedding, Gate, Head, StreamOffset, register_part


def settle_scaled(delta, residual, ctx):
    """A pending delta that still carries a factor per channel (left by a block with layer scale) is added to the
    stream now; returns what is still pending.  Blocks whose norms take no such factor call this first."""
    if delta is not None and ctx.delta_scale is not None:
        kernels.residual_add_scaled(delta, ctx.delta_scale, residual)
        delta = None
    ctx.delta_scale = None
    settle_extra(residual, ctx)
    return delta


def settle_offset(residual, ctx):
    """A vector that joins every row of the stream before this block (set by the model from the schedule) is added
    now, by arrangements whose first norm does not take it along."""
    if ctx.stream_offset is not None:
        kernels.residual_add_row(ctx.stream_offset, residual)
        ctx.stream_offset = None


def settle_extra(residual, ctx):
    """A second pending result (left by a block whose sublayers run side by side) is added to the stream now."""
    if ctx.delta_extra is not None:
        kernels.residual_add(ctx.delta_extra, residual)
        ctx.delta_extra = None


class PreNormResidualBlock(Block):
    kind = "pre_norm_residual"
    norm_names = ("input", "post_mixer")

    def __init__(self, mixer, feed_forward, norms, position, rt):
        self.rt = rt
        self.mixer, self.feed_forward, self.position = mixer, feed_forward, position
        need = self.norm_names if feed_forward is not None else self.norm_names[:1]
        missing = [n for n in need if n not in norms]
        if missing:
            raise ValueError(f"block 'pre_norm_residual' needs norms {need}; missing {missing}")
        self.norm_in, self.norm_post = norms["input"], norms.get("post_mixer")

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    @property
    def graph_safe(self):
        parts = (self.mixer, self.feed_forward, self.norm_in, self.norm_post, self.position)
        return all(p.graph_safe for p in parts if p is not None)

    def step_arrays(self, shape, cache):
        ff = self.feed_forward.step_arrays(shape, cache) if self.feed_forward is not None else {}
        return {**self.mixer.step_arrays(shape, cache), **ff}

    def step(self, delta, residual, ctx, cache, writes_cache=True):
        ctx.residual_act = None                     # this block changes the stream and keeps no rounded copy
        delta = settle_scaled(delta, residual, ctx)
        offset = {}
        if ctx.stream_offset is not None and self.norm_in.takes_offset:
            offset, ctx.stream_offset = {"offset": ctx.stream_offset}, None
        settle_offset(residual, ctx)
        x = self.norm_in.add_norm(delta, residual, **offset)
        a = self.mixer.step(x, ctx, cache, self.position, writes_cache)
        if self.feed_forward is None:
            return a
        x = self.norm_post.add_norm(a, residual)
        return self.feed_forward.step(x, ctx)


class SigmoidGate(Gate):
    """A gate on a sublayer's result, one number per channel: sigmoid(W x + b) with x the sublayer's input.
    This part owns W and b and makes the logits; the arrangement's kernel adds b and applies the sigmoid in
    float32 where it multiplies."""
    kind = "sigmoid_gate"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        h = params["hidden_size"]
        return {"weight": TensorWant((h, h)), "bias": TensorWant((h,), std_scale=10.0)}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.weight, self.bias = load("weight"), load("bias")

    def logits(self, x):
        return linear(x, self.weight)


class PostNormGatedResidualBlock(Block):
    kind = "post_norm_gated_residual"

    def __init__(self, mixer, feed_forward, norms, position, rt, gates=None):
        self.rt = rt
        self.mixer, self.feed_forward, self.position = mixer, feed_forward, position
        gates = gates or {}
        need = ["post_mixer"] + (["post_ff"] if feed_forward is not None else [])
        missing = [n for n in need if n not in norms]
        if missing:
            raise ValueError(f"block 'post_norm_gated_residual' needs norms {need}; missing {missing}")
        self.norm_mixer, self.norm_ff = norms["post_mixer"], norms.get("post_ff")
        self.gate_mixer, self.gate_ff = gates.get("mixer"), gates.get("ff")

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    @property
    def graph_safe(self):
        parts = (self.mixer, self.feed_forward, self.norm_mixer, self.norm_ff, self.gate_mixer, self.gate_ff,
                 self.position)
        return all(p.graph_safe for p in parts if p is not None)

    def step_arrays(self, shape, cache):
        ff = self.feed_forward.step_arrays(shape, cache) if self.feed_forward is not None else {}
        return {**self.mixer.step_arrays(shape, cache), **ff}

    def _join(self, y, gate, norm, x, residual, want_copy):
        g = gate.logits(x) if gate is not None else None
        return kernels.gate_norm_add(y, g, gate.bias if gate is not None else None, norm.weight, norm.eps, residual,
                                     want_copy)

    def step(self, delta, residual, ctx, cache, writes_cache=True):
        act = self.rt.dtype
        delta = settle_scaled(delta, residual, ctx)
        if ctx.stream_offset is not None:
            ctx.residual_act = None
        settle_offset(residual, ctx)
        if delta is not None:                       # a block before this one left its result pending
            kernels.residual_add(delta, residual)
            ctx.residual_act = None
        # the stream in the activation type: the stream itself under float32, else the copy the last
        # gate-norm-add kernel wrote, else a cast
        copies = act != torch.float32
        x = residual if not copies else (ctx.residual_act if ctx.residual_act is not None
                                         else kernels.cast(residual, act))
        y = self.mixer.step(x, ctx, cache, self.position, writes_cache)
        x2 = self._join(y, self.gate_mixer, self.norm_mixer, x, residual, copies)
        x = x2 if copies else residual
        if self.feed_forward is not None:
            y = self.feed_forward.step(x, ctx)
            x2 = self._join(y, self.gate_ff, self.norm_ff, x, residual, copies)
        ctx.residual_act = x2 if copies else None
        return None


class ChannelScale(Gate):
    """A learned factor per channel on a sublayer's result (layer scale).  It does not depend on the input: the
    arrangement hands `weight` to the kernel that adds the result to the stream."""
    kind = "channel_scale"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        return {"weight": TensorWant((params["hidden_size"],), "norm")}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.weight = load("weight")


class PreNormScaledResidualBlock(Block):
    kind = "pre_norm_scaled_residual"

    def __init__(self, mixer, feed_forward, norms, position, rt, gates=None):
        self.rt = rt
        self.mixer, self.feed_forward, self.position = mixer, feed_forward, position
        gates = gates or {}
        need = ["input"] + (["post_mixer"] if feed_forward is not None else [])
        missing = [n for n in need if n not in norms]
        if missing:
            raise ValueError(f"block 'pre_norm_scaled_residual' needs norms {need}; missing {missing}")
        self.norm_in, self.norm_post = norms["input"], norms.get("post_mixer")
        self.scale_mixer, self.scale_ff = gates.get("mixer"), gates.get("ff")

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    @property
    def graph_safe(self):
        parts = (self.mixer, self.feed_forward, self.norm_in, self.norm_post, self.scale_mixer, self.scale_ff,
                 self.position)
        return all(p.graph_safe for p in parts if p is not None)

    def step_arrays(self, shape, cache):
        ff = self.feed_forward.step_arrays(shape, cache) if self.feed_forward is not None else {}
        return {**self.mixer.step_arrays(shape, cache), **ff}

    def step(self, delta, residual, ctx, cache, writes_cache=True):
        ctx.residual_act = None
        settle_extra(residual, ctx)
        settle_offset(residual, ctx)
        scale = lambda g: g.weight if g is not None else None
        x = self.norm_in.add_norm(delta, residual, delta_scale=ctx.delta_scale if delta is not None else None)
        y = self.mixer.step(x, ctx, cache, self.position, writes_cache)
        ctx.delta_scale = scale(self.scale_mixer)
        if self.feed_forward is not None:
            x = self.norm_post.add_norm(y, residual, delta_scale=ctx.delta_scale)
            y = self.feed_forward.step(x, ctx)
            ctx.delta_scale = scale(self.scale_ff)
        return y


class ParallelResidualBlock(Block):
    kind = "parallel_residual"

    def __init__(self, mixer, feed_forward, norms, position, rt):
        self.rt = rt
        self.mixer, self.feed_forward, self.position = mixer, feed_forward, position
        if "input" not in norms:
            raise ValueError("block 'parallel_residual' needs the norm 'input'")
        self.norm_in = norms["input"]
        # one output product for both sublayers when each can hand over what goes into its own
        self.w_out = None
        ff = feed_forward
        if ff is not None and hasattr(mixer, "pre_output") and getattr(mixer, "w_o", None) is not None and \
                hasattr(ff, "pre_output") and getattr(ff, "w_down", None) is not None and \
                mixer.w_o.dtype == ff.w_down.dtype and mixer.w_o.shape[1] % 8 == 0:
            self.k_mixer = mixer.w_o.shape[1]
            self.w_out = torch.cat([mixer.w_o, ff.w_down], dim=1).contiguous()
            mixer.w_o = ff.w_down = None             # the sublayers' own copies are let go: only pre_output runs

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in (self.mixer, self.feed_forward, self.norm_in, self.position) if p is not None)

    def step_arrays(self, shape, cache):
        ff = self.feed_forward.step_arrays(shape, cache) if self.feed_forward is not None else {}
        return {**self.mixer.step_arrays(shape, cache), **ff}

    def step(self, delta, residual, ctx, cache, writes_cache=True):
        ctx.residual_act = None
        if delta is not None and ctx.delta_scale is not None:
            kernels.residual_add_scaled(delta, ctx.delta_scale, residual)
            delta = None
        ctx.delta_scale = None
        settle_offset(residual, ctx)
        extra, ctx.delta_extra = ctx.delta_extra, None
        x = self.norm_in.add_norm(delta, residual, **({"delta2": extra} if extra is not None else {}))
        if self.w_out is not None:
            acts = torch.empty((x.shape[0], self.w_out.shape[1]), dtype=self.rt.dtype, device=x.device)
            self.mixer.pre_output(x, ctx, cache, self.position, writes_cache, out=acts[:, :self.k_mixer])
            self.feed_forward.pre_output(x, ctx, out=acts[:, self.k_mixer:])
            return linear(acts, self.w_out)
        y = self.mixer.step(x, ctx, cache, self.position, writes_cache)
        if self.feed_forward is None:
            return y
        ctx.delta_extra = y
        return self.feed_forward.step(x, ctx)


class TokenEmbedding(Embedding):
    """h[t] = table[id[t]] * scale (src/src-cuda/embedding.cu:29-53, which has no scale: the default 1), written
    as float32."""
    kind = "token_embedding"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        return {"weight": TensorWant((params["vocab_size"], params["hidden_size"]), "table")}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.weight = load("weight")
        self.scale = float(params.get("scale", 1.0))

    def step(self, ctx):
        return kernels.embedding(ctx.tokens, self.weight, scale=self.scale)


class LinearHead(Head):
    """logits = normed . W^T as float32 (src/models/qwen3/qwen3.cpp:302-303), on the rows asked for only.  With
    `softcap` c the logits become c * tanh(logits / c) (upstream has no cap)."""
    kind = "linear_head"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        return {"weight": TensorWant((params["vocab_size"], params["hidden_size"]), "table")}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.weight = load("weight")
        self.softcap = float(params["softcap"]) if params.get("softcap") else None

    def step(self, normed):
        logits = linear(normed, self.weight, out_dtype=torch.float32)
        return kernels.softcap_(logits, self.softcap) if self.softcap else logits


class StreamOffsetTable(StreamOffset):
    """A table of learned vectors [rows, hidden]; the schedule names the row that joins every token's residual stream
    before a layer run (a vector per pass of layers that run several times, for instance).  Upstream has none."""
    kind = "stream_offset"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        return {"weight": TensorWant((params["rows"], params["hidden_size"]))}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        table = load("weight")
        # a tensor per row, so that each starts on an allocation's boundary (the norm kernel reads 16 bytes at a time)
        self.rows = [table[i].clone().contiguous() for i in range(table.shape[0])]

    def row(self, i: int):
        return self.rows[i]


register_part(StreamOffsetTable.kind, StreamOffsetTable)
register_part(PreNormResidualBlock.kind, PreNormResidualBlock)
register_part(PostNormGatedResidualBlock.kind, PostNormGatedResidualBlock)
register_part(PreNormScaledResidualBlock.kind, PreNormScaledResidualBlock)
register_part(ParallelResidualBlock.kind, ParallelResidualBlock)
register_part(SigmoidGate.kind, SigmoidGate)
register_part(ChannelScale.kind, ChannelScale)
register_part(TokenEmbedding.kind, TokenEmbedding)
register_part(LinearHead.kind, LinearHead)
