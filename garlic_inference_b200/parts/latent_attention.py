"""Attention whose keys and values are expanded from a cached low-rank latent, as a mixer.

    q = Wq x = per head [ plain_dim unrotated | rot_dim rotated ]
        with `q_rank`:  q = Wuq ( rmsnorm(Wdq x) * w ), the queries through a normed latent of their own
    [c | kr] = Wdkv x;  c <- rmsnorm(c) * w  (kv_rank);  kr (rot_dim): one rotated key part shared by all heads
    head h:  key = [ Wuk,h c | rot(kr) ],  value = Wuv,h c
    score = (q_plain . Wuk,h c + rot(q_rot) . rot(kr)) * softmax_scale,  causal
    softmax whose denominator also holds exp(sink_h) (optional, one learned number per head)
    o_h = sum_j p_j Wuv,h c_j;  with `head_gate`:  o_h <- o_h * sigmoid(Wg x)_h, one number per head from the mixer's input
    y = Wo concat_h( o_h )

With `own_kv` False the layer has no Wdkv: the schedule points it at another layer's cache entry, whose rows (the
normed latent and the rotated key part as that layer cached them) it reads with its own Wuk, Wuv and queries.

Only c and rot(kr) are cached: one row per position in a single-plane paged entry.  The expansion is never
materialised: q'_h = Wuk,h^T q_plain,h is made by a per-head product, attention runs over the cached rows for
all heads (score q'_h . c_j + rot(q_rot) . rot(kr_j), values c_j), and Wuv,h is applied to the result.

Which attention runs.  Everything under float32, and short portions: the exact-order kernel (scores, softmax
and weighted sum float32, one block per token and head).  Decode steps in bfloat16: the shared-rows kernel,
which stages the cached rows in shared memory once for 32 heads (asynchronous copies, a chunk ahead), cuts the
keys into slices and does both products on tensor cores (mma.sync; float32 scores, softmax and sums, the
weights rounded to bfloat16 as the second product's operand).  Portions of `PRODUCT_MIN_ROWS`
tokens and more in bfloat16: because all heads share the cached rows, the scores of a block of tokens are one
matrix product [tokens x heads, row] . [row, keys] with float32 results, the softmax (causal, with the sink,
float32) is this package's kernel, and the weighted sum is a second product [tokens x heads, keys] . [keys,
kv_rank]; the sequence's rows are gathered from its pages once per step and the tokens are cut into blocks
whose scores fit `SCORE_BYTES`.  Tensor cores do both products; the weights are rounded to bfloat16 only as
the second product's operand.
The rotation is the position part's (its frequencies, magnitude and layout: pairs (2i, 2i+1), or halves (i,
i + n/2)).  Upstream has grouped-query attention only (src/models/qwen3/qwen3.cpp:140-179).
"""
from __future__ import annotations

import torch

from ..cache import KVRequirement
from ..ops import kernels, linear, per_head_linear
from ..weights.loader import TensorWant
from .base import Mixer, register_part
from .linear_attention import pack_rows


# From how many new tokens of a sequence on a bfloat16 step runs attention as product - softmax - product.
PRODUCT_MIN_ROWS = 32
SCORE_BYTES = 256 << 20        # float32 scores of one block of tokens (all heads, all keys)


class LatentAttention(Mixer):
    kind = "latent_attention"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        hid, H, d, dr, dv, r = (params[k] for k in ("hidden_size", "n_heads", "plain_dim", "rot_dim", "value_dim",
                                                    "kv_rank"))
        w = {"uk": TensorWant((H * d, r)), "uv": TensorWant((H * dv, r)), "o": TensorWant((hid, H * dv))}
        if params.get("q_rank"):
            qr = params["q_rank"]
            w.update({"dq": TensorWant((qr, hid)), "dq.norm": TensorWant((qr,), "norm"), "uq": TensorWant((H * (d + dr), qr))})
        else:
            w["q"] = TensorWant((H * (d + dr), hid))
        if params.get("own_kv", True):
            w.update({"dkv": TensorWant((r + dr, hid)), "dkv.norm": TensorWant((r,), "norm")})
        if params.get("head_gate", False):
            w["g"] = TensorWant((H, hid))
        if params.get("sink", False):
            w["sink"] = TensorWant((H,), std_scale=20.0)
        return w

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden, self.H = int(params["hidden_size"]), int(params["n_heads"])
        self.d, self.dr, self.dv, self.rank = (int(params[k]) for k in ("plain_dim", "rot_dim", "value_dim", "kv_rank"))
        self.scale, self.eps = float(params["softmax_scale"]), float(params["eps"])
        self.q_rank = int(params.get("q_rank") or 0)
        self.own_kv, self.head_gate = bool(params.get("own_kv", True)), bool(params.get("head_gate", False))
        self.row = -(-(self.rank + self.dr) // 8) * 8             # a cache row, padded for the kernel's 16-byte loads
        # everything that reads the mixer's input is one product: [queries or their latent | latent and key part | gates]
        packed = [("dq", self.q_rank) if self.q_rank else ("q", self.H * (self.d + self.dr))]
        packed += [("dkv", self.rank + self.dr)] if self.own_kv else []
        packed += [("g", self.H)] if self.head_gate else []
        self.w_in, offs = pack_rows(load, packed, self.hidden, rt)
        self.q_off = offs[0]
        self.c_off = offs[1] if self.own_kv else None
        self.g_off = offs[-1] if self.head_gate else None
        self.q_norm, self.w_uq = (load("dq.norm"), load("uq")) if self.q_rank else (None, None)
        self.c_norm = load("dkv.norm") if self.own_kv else None
        # Wuk per head as [rank, plain_dim]: the product q'_h = Wuk,h^T q_h in the [out, in] form of the others
        self.w_uk_t = load("uk").view(self.H, self.d, self.rank).transpose(1, 2).contiguous()
        self.w_uv = load("uv").view(self.H, self.dv, self.rank)
        self.w_o = load("o")
        self.sink = load("sink") if params.get("sink", False) else None
        self._no_rotation = None

    def cache_requirement(self):
        return KVRequirement(1, self.row, None, planes=1)

    def _rotation(self, position, device):
        if position is not None:
            freq, magnitude, n_rot, layout = position.rotary_frequencies()
            if n_rot > self.dr:
                raise ValueError(f"{n_rot} rotated dimensions of a key part of {self.dr}")
            return freq, magnitude, n_rot, layout == "half"
        if self._no_rotation is None:
            self._no_rotation = torch.zeros(0, dtype=torch.float32, device=device)
        return self._no_rotation, 1.0, 0, False

    def step(self, x, ctx, cache, position, writes_cache=True):
        return linear(self.pre_output(x, ctx, cache, position, writes_cache), self.w_o)

    def pre_output(self, x, ctx, cache, position, writes_cache=True, out=None, out_mul=1.0):
        """Everything before the output projection: [n, n_heads * value_dim] in the activation type, times
        `out_mul`, written into `out` (columns of a wider matrix) when given."""
        kv = cache.kv
        if self.own_kv != bool(writes_cache):
            raise ValueError("a layer with a latent of its own writes its cache entry, and one without reads another "
                             "layer's: the schedule says otherwise")
        n = x.shape[0]
        freq, magnitude, n_rot, half = self._rotation(position, x.device)
        proj = linear(x, self.w_in)
        if self.q_rank:
            q_src, q_off = linear(kernels.rmsnorm_rows(proj[:, self.q_off:self.q_off + self.q_rank], self.q_norm, self.eps),
                                  self.w_uq), 0
        else:
            q_src, q_off = proj, self.q_off
        q = q_src[:, q_off:q_off + self.H * (self.d + self.dr)].view(n, self.H, self.d + self.dr)
        q_lat = per_head_linear(q[:, :, :self.d], self.w_uk_t)                       # [n, H, rank]
        q_rows = kernels.latent_prepare(q_src, q_off, proj if self.own_kv else None, self.c_off or 0, q_lat, self.c_norm,
                                        self.eps, freq, magnitude, n_rot, ctx.tok_pos, ctx.tok_slot, kv.block_table,
                                        kv.k_pool, self.H, self.d, self.dr, self.rank, ctx.status, append=writes_cache,
                                        half_layout=half)
        o_lat = self.attend(q_rows, kv, ctx)
        plain = not self.head_gate and out is None and out_mul == 1.0
        # with a gate (or a factor, or columns to write into) the values leave their product in float32 and are
        # rounded once, after the gate
        o = per_head_linear(o_lat.view(n, self.H, self.rank), self.w_uv,
                            out_dtype=None if plain else torch.float32)             # [n, H, value_dim]
        if plain:
            return o.view(n, self.H * self.dv)
        gate = proj[:, self.g_off:self.g_off + self.H] if self.head_gate else None
        return kernels.attn_finish(o.view(n, self.H * self.dv), self.H, 1, None, None, out_mul, gate, self.rt.dtype, out=out)

    def attend(self, q_rows, kv, ctx):
        """Attention of q_rows [n, H, row] over the cached rows; returns [n, H * kv_rank]."""
        by_products = (q_rows.dtype == torch.bfloat16 and not ctx.all_single and not ctx.captured and ctx.seq_lens
                       and max(ctx.seq_lens) >= PRODUCT_MIN_ROWS)
        if ctx.all_single and kernels.latent_decode_takes(q_rows.dtype, q_rows.shape[2], self.rank, self.H):
            return kernels.latent_decode(q_rows, kv.k_pool, kv.block_table, ctx.tok_pos, ctx.tok_slot, self.scale,
                                         self.sink, self.rank, ctx.status)
        if not by_products:
            return kernels.attention_generic(q_rows, kv.k_pool, kv.k_pool, kv.block_table, ctx.tok_pos, ctx.tok_slot,
                                             self.scale, 0, ctx.status, sinks=self.sink, value_dim=self.rank)
        n, H, row = q_rows.shape
        out = torch.empty((n, H * self.rank), dtype=q_rows.dtype, device=q_rows.device)
        page = kv.page_size
        pool = kv.k_pool.view(kv.k_pool.shape[0], page, row)
        short = [(s, st, m, p) for s, st, m, p in zip(ctx.seq_slots, ctx.seq_starts, ctx.seq_lens, ctx.seq_past)
                 if m < PRODUCT_MIN_ROWS]
        for slot, start, n_new, past in zip(ctx.seq_slots, ctx.seq_starts, ctx.seq_lens, ctx.seq_past):
            if n_new < PRODUCT_MIN_ROWS:
                continue
            n_pages = -(-(past + n_new) // page)
            rows = pool.index_select(0, kv.block_table[slot, :n_pages].long()).view(n_pages * page, row)
            block = max(1, min(n_new, SCORE_BYTES // (4 * H * n_pages * page)))
            for q0 in range(0, n_new, block):
                tq = min(block, n_new - q0)
                keys = min(-(-(past + q0 + tq) // 8) * 8, n_pages * page)      # what this block sees, padded to 8
                q = q_rows[start + q0:start + q0 + tq].view(tq * H, row)
                scores = torch.mm(q, rows[:keys].t(), out_dtype=torch.float32)
                weights = kernels.causal_sink_softmax(scores, H, past + q0, self.scale, self.sink, q_rows.dtype)
                out[start + q0:start + q0 + tq] = torch.mm(weights, rows[:keys, :self.rank]).view(tq, H * self.rank)
        if short:                                  # sequences that bring a few tokens: the exact-order kernel
            idx = torch.cat([torch.arange(st, st + m) for _, st, m, _ in short]).to(q_rows.device)
            part = kernels.attention_generic(q_rows.index_select(0, idx).contiguous(), kv.k_pool, kv.k_pool,
                                             kv.block_table, ctx.tok_pos.index_select(0, idx).contiguous(),
                                             ctx.tok_slot.index_select(0, idx).contiguous(), self.scale, 0,
                                             ctx.status, sinks=self.sink, value_dim=self.rank)
            out.index_copy_(0, idx, part)
        return out


register_part(LatentAttention.kind, LatentAttention)
