"""Softmax attention with the options that grouped-query attention proper does not have, as a mixer.

    q = Wq x, k = Wk x, v = Wv x                    `n_heads` query heads, `n_kv_heads` key/value heads; keys of
                                                    `key_dim`, values of `value_dim` (they may differ)
    conv_taps K > 0:  q, k, v <- causal convolution over time per channel (K taps, no bias, no activation); the
                      last K - 1 projected values of a sequence are part of its state
    a position part:  its rotation on q and k (any layout, any number of rotated dimensions)
    mask:             "causal"; "window" (the last `size` keys); "chunk" (the keys j <= i with floor(j / size) =
                      floor(i / size), chunks counted from position 0)
    maps = 2:         differential attention.  Wq and Wk make two maps per head, laid out head by head as
                      [map 1, map 2]; each is a softmax of its own over the same values, and
                      o = a_1 - lam a_2,  lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff     (one number per layer)
    sub_norm_eps:     o <- o / sqrt(mean(o^2) + eps) per head (no weight), times `out_mul`
    head_gate:        o <- o * sigmoid(Wg x)_head, one number per head, from the mixer's own input
    qkv_bias:         q, k, v <- q + bq, k + bk, v + bv (tensors `q.b`, `k.b`, `v.b`), before everything else
    projection_norm_eps:  q <- q / sqrt(mean(q^2) + eps) * wq over ALL query columns of the token at once (not per
                      head), k likewise with wk (tensors `q.norm`, `k.norm`, a weight per column, used as they are)
    query_temperature {coef, every}:  q at position p times 1 + coef ln(floor((p + 1) / every) + 1)
    sink s:           the softmax's denominator also holds exp(s): a key that every query sees and that has no
                      value (s = 0 adds one to the denominator)
    distance_bias {rows B, max_distance D}:  the scaled score of key j for the query at position i gets
                      rel[bucket(i - j), head] added (tensor `rel` [B, heads]; the scale does not touch it), with
                      bucket(n) = n for n < B/2, else min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(D / (B/2)) (B - B/2)))
    y = Wo concat(o)
Bias, norm, temperature and rotation are float32 inside the kernel that also appends keys and values to the cache;
sinks and distance biases (one map per head only) are taken by all three attention kernels below.

Query head h reads key/value head h // (n_heads // n_kv_heads).  With `own_kv` False the layer has no key and
value tensors: the schedule points it at another layer's cache entry, whose keys and values (as that cache holds
them: after convolution and rotation) it reads with its own queries, mask and everything else.

All projections that read x are one packed product.  Which attention runs: in bfloat16, with key and value
sizes that the tensor-core kernels take (multiples of 16 up to 128, equal or one twice the other; one map with
keys and values of 128 and pages of a multiple of 64 tokens: the tcgen05 prompt kernel): the flash
kernel for steps that bring several tokens of a sequence and the split-KV kernel for decode steps, once per map,
with the chunk mask in them (float32 scores, softmax and sums; the weights rounded to bfloat16 as the second
product's operand).  Everything else (float32, other sizes): the exact-order kernel, whose result at a position does not depend on how the tokens were cut into steps.  What
comes out is combined, normed and gated in float32 and rounded once.  Upstream has grouped-query attention only
(src/models/qwen3/qwen3.cpp:140-179).
"""
from __future__ import annotations

import math

import torch

from ..cache import EntryRequirement, KVRequirement, StateRequirement
from ..ops import kernels, linear
from ..weights.loader import TensorWant
from .attention import query_runs
from .base import Mixer, register_part
from .linear_attention import pack_rows


class MaskedAttention(Mixer):
    kind = "masked_attention"
    graph_safe = True

    @staticmethod
    def _sizes(params):
        H, G, d, dv = (int(params[k]) for k in ("n_heads", "n_kv_heads", "key_dim", "value_dim"))
        maps = int(params.get("maps", 1))
        return H, G, d, dv, maps, int(params.get("conv_taps", 0) or 0), bool(params.get("own_kv", True))

    @classmethod
    def wanted(cls, params):
        hid = params["hidden_size"]
        H, G, d, dv, maps, K, own = cls._sizes(params)
        w = {"q": TensorWant((H * maps * d, hid)), "o": TensorWant((hid, H * dv))}
        if own:
            w["k"], w["v"] = TensorWant((G * maps * d, hid)), TensorWant((G * dv, hid))
        if K:
            taps = lambda rows: TensorWant((rows, K), std_scale=8.0)
            w["q.conv"] = taps(H * maps * d)
            if own:
                w["k.conv"], w["v.conv"] = taps(G * maps * d), taps(G * dv)
        if maps == 2:
            for n in ("lq1", "lk1", "lq2", "lk2"):
                w[n] = TensorWant((d,), std_scale=5.0)
        if params.get("head_gate", False):
            w["g"] = TensorWant((H, hid))
        if params.get("qkv_bias", False):
            w["q.b"] = TensorWant((H * maps * d,), std_scale=5.0)
            if own:
                w["k.b"], w["v.b"] = TensorWant((G * maps * d,), std_scale=5.0), TensorWant((G * dv,), std_scale=5.0)
        if params.get("projection_norm_eps") is not None:
            w["q.norm"] = TensorWant((H * maps * d,), "norm")
            if own:
                w["k.norm"] = TensorWant((G * maps * d,), "norm")
        if params.get("distance_bias"):
            w["rel"] = TensorWant((int(params["distance_bias"]["rows"]), H), std_scale=10.0)
        return w

    @staticmethod
    def distance_buckets(rows: int, max_distance: int) -> torch.Tensor:
        """bucket(n) for n = 0 .. max_distance (every larger distance reads the last row, as max_distance itself
        does): int64 [max_distance + 1].  The logarithms are float64."""
        half = rows // 2
        n = torch.arange(max_distance + 1, dtype=torch.float64)
        if half == 0:
            return torch.zeros(max_distance + 1, dtype=torch.long)
        far = half + torch.floor(torch.log(torch.clamp(n, min=1.0) / half) / math.log(max_distance / half) * (rows - half))
        return torch.where(n < half, n, torch.clamp(far, max=rows - 1)).to(torch.long)

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden = int(params["hidden_size"])
        self.H, self.G, self.d, self.dv, self.maps, self.K, self.own_kv = self._sizes(params)
        if self.H % self.G:
            raise ValueError(f"{self.H} query heads are no multiple of {self.G} key/value heads")
        if self.maps not in (1, 2):
            raise ValueError(f"{self.maps} softmax maps per head: one, or two (differential attention)")
        self.scale = float(params.get("softmax_scale", self.d ** -0.5))
        mask = params.get("mask") or {"kind": "causal"}
        if mask["kind"] not in ("causal", "window", "chunk"):
            raise ValueError(f"mask kind {mask['kind']!r} is none of 'causal', 'window', 'chunk'")
        self.window = int(mask["size"]) if mask["kind"] == "window" else 0
        self.chunk = int(mask["size"]) if mask["kind"] == "chunk" else 0
        self.sub_norm_eps = params.get("sub_norm_eps")
        self.out_mul = float(params.get("out_mul", 1.0))
        self.head_gate = bool(params.get("head_gate", False))
        self.Cq = self.H * self.maps * self.d
        self.Ck, self.Cv = (self.G * self.maps * self.d, self.G * self.dv) if self.own_kv else (0, 0)
        self.C = self.Cq + self.Ck + self.Cv
        packed = [("q", self.Cq)] + ([("k", self.Ck), ("v", self.Cv)] if self.own_kv else []) + \
                 ([("g", self.H)] if self.head_gate else [])
        self.w_in, offs = pack_rows(load, packed, self.hidden, rt)
        self.g_off = offs[-1] if self.head_gate else None
        self.w_o = load("o")
        self.taps = None
        if self.K:
            names = ["q.conv"] + (["k.conv", "v.conv"] if self.own_kv else [])
            self.taps = torch.cat([load(n) for n in names]).contiguous()
        self.lam = None
        if self.maps == 2:
            f = lambda n: load(n).to(torch.float32)
            self.lam = (torch.exp((f("lq1") * f("lk1")).sum()) - torch.exp((f("lq2") * f("lk2")).sum())
                        + float(params.get("diff", 0.0))).reshape(1).contiguous()
        self.state_floats = -(-((self.K - 1) * self.C) // 4) * 4 if self.K > 1 else 0
        self._no_state = None
        f32 = lambda t: t.to(torch.float32)
        own_names = lambda stem: [stem.format("q")] + ([stem.format("k")] if self.own_kv else [])
        self.bias = None
        if params.get("qkv_bias", False):
            self.bias = torch.cat([f32(load(n)) for n in own_names("{}.b") + (["v.b"] if self.own_kv else [])]).contiguous()
        self.norm_eps = params.get("projection_norm_eps")
        self.norm_w = None
        if self.norm_eps is not None:
            self.norm_w = torch.cat([f32(load(n)) for n in own_names("{}.norm")]).contiguous()
        temp = params.get("query_temperature") or {}
        self.temp_coef, self.temp_every = float(temp.get("coef", 0.0)), int(temp.get("every", 0))
        if temp and self.temp_every <= 0:
            raise ValueError(f"query_temperature.every must be positive, found {self.temp_every}")
        self.sinks = None
        if params.get("sink") is not None:
            self.sinks = torch.full((self.H,), float(params["sink"]), dtype=torch.float32, device=rt.device)
        self.dist_bias = None
        if params.get("distance_bias"):
            rows, far = int(params["distance_bias"]["rows"]), int(params["distance_bias"]["max_distance"])
            if rows < 1 or far <= rows // 2:
                raise ValueError(f"a distance bias of {rows} rows up to distance {far}: the distance must pass half the rows")
            # the table by distance, [max_distance + 1, heads] float32: what the kernels index with min(i - j, last)
            self.dist_bias = f32(load("rel"))[self.distance_buckets(rows, far).to(rt.device)].contiguous()
        if (self.sinks is not None or self.dist_bias is not None) and self.maps != 1:
            raise ValueError("a sink and a distance bias come with one softmax map per head")
        if (self.bias is not None or self.norm_w is not None or self.temp_every) and self.K:
            raise ValueError("biases, the projection norm and the query temperature are not combined with the short filters")

    def cache_requirement(self):
        kv = KVRequirement(self.G * self.maps, self.d, None, 2, value_heads=self.G, value_dim=self.dv)
        if not self.state_floats:
            return kv
        return EntryRequirement(kv, StateRequirement((self.state_floats,), torch.float32))

    def _tensor_cores(self) -> bool:
        return kernels.mma_attention_takes(self.rt.dtype, self.d, self.dv)

    def _run_rows(self, kv) -> int:
        """Height of the query runs of the prompt kernel that takes this mixer: 128 (tcgen05: one map, keys and
        values of 128, pages of a multiple of 64), 64 (mma.sync), 0 (the exact-order kernel, which needs none)."""
        if self.maps == 1 and self.d == self.dv and self.dist_bias is None and \
                kernels.tcgen05_attention_takes(self.rt.dtype, self.d, kv.page_size):
            return 128
        return 64 if self._tensor_cores() else 0

    def step_arrays(self, shape, cache):
        rows = 0 if shape.all_single else self._run_rows(cache.kv)
        return {f"query_runs_{rows}": lambda: query_runs(shape, rows)} if rows else {}

    def _rotation(self, position):
        if position is None:
            return None, 0, False
        freq, magnitude, n_rot, layout = position.rotary_frequencies()
        if magnitude != 1.0:
            raise ValueError("masked_attention turns q and k by plain angles: a rotation that scales cos and sin is "
                             "not computed here")
        if n_rot > self.d:
            raise ValueError(f"{n_rot} rotated dimensions of heads of {self.d}")
        return freq, n_rot, layout == "half"

    def step(self, x, ctx, cache, position, writes_cache=True):
        return linear(self.pre_output(x, ctx, cache, position, writes_cache), self.w_o)

    def pre_output(self, x, ctx, cache, position, writes_cache=True, out=None, out_mul=1.0):
        """Everything before the output projection: [n, n_heads * value_dim] in the activation type, times
        `out_mul`, written into `out` (columns of a wider matrix) when given."""
        kv = cache.kv
        if self.own_kv != bool(writes_cache):
            raise ValueError("a layer with keys and values of its own writes its cache entry, and one without reads "
                             "another layer's: the schedule says otherwise")
        proj = linear(x, self.w_in)
        src = proj
        if self.K:
            conv_in = proj[:, :self.C]
            if self.K > 1:
                src = kernels.causal_conv_silu(conv_in, self.taps, cache.state, ctx.tok_slot, activation="none",
                                               renew_state=ctx.all_single)
                if not ctx.all_single:
                    kernels.conv_state_update(conv_in, self.K, cache.state, ctx.tok_slot)
            else:                                     # one tap: a factor per channel, no state
                if self._no_state is None:
                    self._no_state = torch.zeros((cache.kv.block_table.shape[0] + 1, 4), dtype=torch.float32, device=x.device)
                src = kernels.causal_conv_silu(conv_in, self.taps, self._no_state, ctx.tok_slot, activation="none")
        freq, n_rot, half = self._rotation(position)
        q = kernels.attn_prepare(src, 0, self.Cq if self.own_kv else -1, self.Cq + self.Ck, freq, n_rot, half,
                                 ctx.tok_pos, ctx.tok_slot, kv.block_table, kv.k_pool, kv.v_pool, self.H * self.maps,
                                 self.d, self.rt.dtype, ctx.status, append=writes_cache, bias=self.bias,
                                 norm_weight=self.norm_w, norm_eps=float(self.norm_eps or 0.0), temp_coef=self.temp_coef,
                                 temp_every=self.temp_every)
        extras = dict(sinks=self.sinks, dist_bias=self.dist_bias)
        if ctx.all_single and self._tensor_cores() and self.H // self.G <= 16:
            att = kernels.attention_decode_masked_bf16(q, kv.k_pool, kv.v_pool, kv.block_table, ctx.tok_pos, ctx.tok_slot,
                                                       self.scale, window=self.window, chunk=self.chunk, maps=self.maps,
                                                       **extras)
        elif not ctx.all_single and ctx.seq_lens and self._run_rows(kv):
            rows = self._run_rows(kv)
            runs = ctx.arrays.get(f"query_runs_{rows}")
            if runs is None:                      # a context put together by hand: cut and copy here
                runs = ctx.arrays[f"query_runs_{rows}"] = torch.from_numpy(query_runs(ctx, rows)).to(x.device)
            covered = ctx.n_tokens == sum(ctx.seq_lens)
            if rows == 128:
                att = kernels.attention_prefill_tcgen05(q, kv.k_pool, kv.v_pool, kv.block_table, runs, self.scale,
                                                        self.window, rows_covered=covered, chunk=self.chunk,
                                                        sinks=self.sinks)
            else:
                att = kernels.attention_prefill_masked_bf16(q, kv.k_pool, kv.v_pool, kv.block_table, runs, self.scale,
                                                            window=self.window, chunk=self.chunk, maps=self.maps,
                                                            rows_covered=covered, **extras)
        else:
            att = kernels.attention_masked(q, kv.k_pool, kv.v_pool, kv.block_table, ctx.tok_pos, ctx.tok_slot,
                                           self.scale, ctx.status, window=self.window, chunk=self.chunk,
                                           maps=self.maps, out_float32=True, **extras)
        gate = proj[:, self.g_off:self.g_off + self.H] if self.head_gate else None
        if self.maps == 1 and gate is None and self.sub_norm_eps is None and self.out_mul * out_mul == 1.0 and \
                out is None and att.dtype == self.rt.dtype:
            return att                                # one map, nothing to combine, norm or gate: it is the result
        return kernels.attn_finish(att, self.H, self.maps, self.lam, self.sub_norm_eps, self.out_mul * out_mul, gate,
                                   self.rt.dtype, out=out)


register_part(MaskedAttention.kind, MaskedAttention)
