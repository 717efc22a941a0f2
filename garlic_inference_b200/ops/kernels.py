"""Python faces of the CUDA entry points.

Each function checks that its tensors are on the GPU, dense and of the types
the kernel is written for, allocates the output, and launches on torch's
current stream.  Sizes a kernel cannot take come back as `KernelError` with
the kernel's own message.
"""
from __future__ import annotations

from typing import Optional

import torch

from .library import KernelError, check, counters, require_gpu
from .library import counters as counters_mod

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


def code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is neither float32 nor bfloat16") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dense(t: torch.Tensor, name: str, dtype=None) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on the GPU only")
    if not t.is_contiguous():
        raise KernelError(f"{name} of shape {tuple(t.shape)} and strides {t.stride()} is not dense")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} is {t.dtype}, the kernel wants {dtype}")
    return t


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def set_dependent_launch(on: bool) -> None:
    """Whether the launches that follow carry the attribute for programmatic dependent launch (the next
    kernel may be launched, and fetch its weights, while this one still runs)."""
    require_gpu().gi_set_pdl(1 if on else 0)


def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """float32 rows of `table` for int32 `ids`, times `scale`: the start of the residual stream."""
    l = require_gpu()
    _dense(ids, "ids", torch.int32)
    _dense(table, "table")
    n, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _dense(out, "out", torch.float32)
    check(l.gi_embedding(_ptr(ids), _ptr(table), code(table.dtype), _ptr(out), n, vocab, hidden, float(scale), _stream()), l)
    return out


def add_rmsnorm(delta: Optional[torch.Tensor], residual: torch.Tensor, weight: torch.Tensor, eps: float,
                act_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                write_residual: bool = True, out: Optional[torch.Tensor] = None,
                offset: Optional[torch.Tensor] = None) -> torch.Tensor:
    """normed = rmsnorm(residual (+ delta) (+ offset)) * weight in `act_dtype`; with `write_residual` the
    float32 sum goes back into `residual`.  `rows` (int32) picks input rows (then nothing is written back).
    `offset` [dim]: a vector that joins every row."""
    l = require_gpu()
    _dense(residual, "residual", torch.float32)
    _dense(weight, "weight")
    dim = residual.shape[-1]
    if weight.numel() != dim:
        raise KernelError(f"norm weight has {weight.numel()} elements for rows of {dim}")
    if delta is not None:
        _dense(delta, "delta", act_dtype)
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} and residual {tuple(residual.shape)} differ")
    if rows is not None:
        _dense(rows, "rows", torch.int32)
        n_rows, write_residual = rows.numel(), False
    else:
        n_rows = residual.numel() // dim
    if offset is not None:
        _dense(offset, "offset")
        if offset.numel() != dim:
            raise KernelError(f"an offset of {offset.numel()} elements for rows of {dim}")
    if out is None:
        out = torch.empty((n_rows, dim), dtype=act_dtype, device=residual.device)
    _dense(out, "out", act_dtype)
    check(l.gi_add_rmsnorm(_ptr(delta), _ptr(residual), _ptr(weight), code(weight.dtype), _ptr(out),
                           code(act_dtype), _ptr(rows), n_rows, dim, float(eps), int(write_residual), _ptr(offset),
                           code(offset.dtype) if offset is not None else F32, _stream()), l)
    return out


def add_layernorm(delta: Optional[torch.Tensor], residual: torch.Tensor, weight: torch.Tensor,
                  bias: Optional[torch.Tensor], eps: float, act_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                  write_residual: bool = True, delta2: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(s - mean(s)) / sqrt(var(s) + eps) * weight (+ bias) for s = residual (+ delta (+ delta2)), in `act_dtype`; the
    float32 sum goes back into `residual` unless `rows` (int32) picks rows or `write_residual` is False."""
    l = require_gpu()
    _dense(residual, "residual", torch.float32), _dense(weight, "weight")
    dim = residual.shape[-1]
    if weight.numel() != dim or (bias is not None and _dense(bias, "bias", weight.dtype).numel() != dim):
        raise KernelError(f"norm weight of {weight.numel()} elements for rows of {dim}")
    for d, name in ((delta, "delta"), (delta2, "delta2")):
        if d is not None and _dense(d, name, act_dtype).shape != residual.shape:
            raise KernelError(f"{name} {tuple(d.shape)} and residual {tuple(residual.shape)} differ")
    if rows is not None:
        _dense(rows, "rows", torch.int32)
        n_rows, write_residual = rows.numel(), False
    else:
        n_rows = residual.numel() // dim
    out = torch.empty((n_rows, dim), dtype=act_dtype, device=residual.device)
    check(l.gi_add_layernorm(_ptr(delta), _ptr(delta2), _ptr(residual), _ptr(weight), _ptr(bias), code(weight.dtype),
                             _ptr(out), code(act_dtype), _ptr(rows), n_rows, dim, float(eps), int(write_residual),
                             _stream()), l)
    return out


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight for the rows of x, which may be columns of a wider matrix; dense result in
    x's type, float32 inside."""
    l = require_gpu()
    _rows(x, "x"), _dense(weight, "weight")
    n, dim = x.shape
    if weight.numel() != dim:
        raise KernelError(f"norm weight of {weight.numel()} elements for rows of {dim}")
    out = torch.empty((n, dim), dtype=x.dtype, device=x.device)
    check(l.gi_rmsnorm_rows(_ptr(x), x.stride(0), _ptr(weight), code(weight.dtype), _ptr(out), code(x.dtype), n, dim,
                            float(eps), _stream()), l)
    return out


def softcap_(z: torch.Tensor, cap: float) -> torch.Tensor:
    """z <- cap * tanh(z / cap) in place (float32)."""
    l = require_gpu()
    _dense(z, "z", torch.float32)
    check(l.gi_softcap(_ptr(z), z.numel(), float(cap), _stream()), l)
    return z


def residual_add(delta: torch.Tensor, residual: torch.Tensor) -> None:
    l = require_gpu()
    _dense(delta, "delta")
    _dense(residual, "residual", torch.float32)
    if delta.shape != residual.shape:
        raise KernelError(f"delta {tuple(delta.shape)} and residual {tuple(residual.shape)} differ")
    check(l.gi_residual_add(_ptr(delta), code(delta.dtype), _ptr(residual), residual.numel(), _stream()), l)


def residual_add_row(vec: torch.Tensor, residual: torch.Tensor) -> None:
    """residual[r, :] += vec for every row (float32 sums)."""
    l = require_gpu()
    _dense(vec, "vec"), _dense(residual, "residual", torch.float32)
    dim = residual.shape[-1]
    if vec.numel() != dim:
        raise KernelError(f"a vector of {vec.numel()} elements for rows of {dim}")
    check(l.gi_residual_add_row(_ptr(vec), code(vec.dtype), _ptr(residual), residual.numel() // dim, dim, _stream()), l)


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(gate) * up for [n, 2*inter] rows holding the gate first, then up."""
    l = require_gpu()
    _dense(gate_up, "gate_up")
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError(f"gate_up rows of {two_i} columns cannot hold a gate and an up half")
    if out is None:
        out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _dense(out, "out", gate_up.dtype)
    check(l.gi_swiglu(_ptr(gate_up), _ptr(out), code(gate_up.dtype), n, two_i // 2, _stream()), l)
    return out


def cast(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if src.dtype == dtype:
        return src
    l = require_gpu()
    _dense(src, "src")
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    check(l.gi_cast(_ptr(src), code(src.dtype), _ptr(out), code(dtype), src.numel(), _stream()), l)
    return out


def random_normal(out: torch.Tensor, key: int, mean: float, std: float) -> torch.Tensor:
    """Fill `out` (float32 or bfloat16, dense) with mean + std * z_i, z_i a standard normal variate that
    depends on (key, i) alone; `weights/random_init.py` holds the same arithmetic for the host."""
    l = require_gpu()
    _dense(out, "out")
    check(l.gi_random_normal(_ptr(out), code(out.dtype), out.numel(), key & 0xFFFFFFFFFFFFFFFF, float(mean),
                             float(std), _stream()), l)
    return out


def qk_norm_rope_append(qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                        cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int,
                        tok_pos: torch.Tensor, tok_slot: torch.Tensor,
                        k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                        status: torch.Tensor, append: bool = True) -> torch.Tensor:
    """Norm and rotate q and k of packed projections [n, (n_q + 2 n_kv) d]; returns q [n, n_q, d]
    and (with `append`) writes k and v of every token with a slot into the paged pools."""
    l = require_gpu()
    act = qkv.dtype
    _dense(qkv, "qkv")
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError(f"qkv rows have {qkv.shape[1]} columns, not (n_q + 2 n_kv) * head_dim = "
                          f"{(n_q + 2 * n_kv) * head_dim}")
    for t, name in ((k_pool, "k_pool"), (v_pool, "v_pool")):
        _dense(t, name, act)
    n_pages, pool_kv, page_size, pool_d = k_pool.shape
    if (pool_kv, pool_d) != (n_kv, head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit "
                          f"{n_kv} key/value heads of {head_dim}")
    _dense(cos, "cos", torch.float32), _dense(sin, "sin", torch.float32)
    if cos.shape != sin.shape or cos.shape[1] * 2 != rotary_dim:
        raise KernelError(f"rotary tables {tuple(cos.shape)} do not fit rotary_dim {rotary_dim}")
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table"), (status, "status")):
        _dense(t, name, torch.int32)
    if tok_pos.numel() < n or tok_slot.numel() < n:
        raise KernelError("tok_pos / tok_slot are shorter than the token rows")
    w_code = F32
    if q_weight is not None:
        _dense(q_weight, "q_weight"), _dense(k_weight, "k_weight", q_weight.dtype)
        if q_weight.numel() != head_dim or k_weight.numel() != head_dim:
            raise KernelError("q/k norm weights must have head_dim elements")
        w_code = code(q_weight.dtype)
    q_out = torch.empty((n, n_q, head_dim), dtype=act, device=qkv.device)
    check(l.gi_qk_norm_rope_append(
        _ptr(qkv), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), code(act), _ptr(q_weight), _ptr(k_weight), w_code,
        float(eps), _ptr(cos), _ptr(sin), rotary_dim, _ptr(tok_pos), _ptr(tok_slot), _ptr(block_table),
        n, n_q, n_kv, head_dim, page_size, block_table.shape[1], n_pages, cos.shape[0], int(append),
        _ptr(status), _stream()), l)
    return q_out


def attention_generic(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                      tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float, window: int,
                      status: torch.Tensor, sinks: Optional[torch.Tensor] = None,
                      value_dim: Optional[int] = None) -> torch.Tensor:
    """Exact-order attention of q [n, n_q, d] over the paged cache; returns [n, n_q * value_dim] (value_dim = d
    unless given: the first columns of the value rows).  `sinks` [n_q]: a number per head that joins the
    softmax's denominator as exp(sink), without a value."""
    l = require_gpu()
    _dense(q, "q")
    n, n_q, d = q.shape
    d_v = d if value_dim is None else int(value_dim)
    if sinks is not None:
        _dense(sinks, "sinks")
        if sinks.numel() != n_q:
            raise KernelError(f"{sinks.numel()} sinks for {n_q} query heads")
    _dense(k_pool, "k_pool", q.dtype), _dense(v_pool, "v_pool", q.dtype)
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    if pool_d != d or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not fit head_dim {d}")
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table"), (status, "status")):
        _dense(t, name, torch.int32)
    out = torch.empty((n, n_q * d_v), dtype=q.dtype, device=q.device)
    check(l.gi_attention_generic(_ptr(q), _ptr(k_pool), _ptr(v_pool), code(q.dtype), _ptr(block_table),
                                 _ptr(tok_pos), _ptr(tok_slot), _ptr(out), n, n_q, n_kv, d, page_size,
                                 block_table.shape[1], n_pages, int(window or 0), float(scale), _ptr(sinks),
                                 code(sinks.dtype) if sinks is not None else F32, d_v, _ptr(status), _stream()), l)
    return out


def attention_masked(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                     tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float, status: torch.Tensor, window: int = 0,
                     chunk: int = 0, maps: int = 1, out_float32: bool = False, sinks: Optional[torch.Tensor] = None,
                     dist_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exact-order attention of q [n, rows, d] over keys [pages, key heads, page, d] and values [pages, value
    heads, page, dv] of their own shape.  `sinks` [rows]: a score per query row that joins the softmax's denominator
    without a value.  `dist_bias` float32 [n_dist, rows]: added to the scaled score of key j for the query at
    position i at row min(i - j, n_dist - 1).  `chunk` > 0: a query sees the keys of its own chunk of positions only
    (chunks counted from position 0).  `maps` > 1: the rows of a token are [head][map] and the key heads [key
    head][map]; every map is a softmax of its own over the head's values.  Returns [n, rows * dv], float32 when
    asked, else q's type."""
    l = require_gpu()
    _dense(q, "q"), _dense(k_pool, "k_pool", q.dtype), _dense(v_pool, "v_pool", q.dtype)
    n, n_q, d = q.shape
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    v_pages, n_vh, v_page, dv = v_pool.shape
    if pool_d != d or (v_pages, v_page) != (n_pages, page_size):
        raise KernelError(f"cache pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit queries of {d}")
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table"), (status, "status")):
        _dense(t, name, torch.int32)
    n_dist = _check_sinks_bias(sinks, dist_bias, n_q)
    out = torch.empty((n, n_q * dv), dtype=torch.float32 if out_float32 else q.dtype, device=q.device)
    check(l.gi_attention_masked(_ptr(q), _ptr(k_pool), _ptr(v_pool), code(q.dtype), _ptr(block_table), _ptr(tok_pos),
                                _ptr(tok_slot), None if out_float32 else _ptr(out), n, n_q, n_kv, d, page_size,
                                block_table.shape[1], n_pages, int(window or 0), float(scale), _ptr(sinks), F32, dv,
                                _ptr(status), int(chunk or 0), n_vh, dv, int(maps), _ptr(out) if out_float32 else None,
                                _ptr(dist_bias), n_dist, _stream()), l)
    return out


def _check_sinks_bias(sinks: Optional[torch.Tensor], dist_bias: Optional[torch.Tensor], rows: int) -> int:
    """Checks a sink vector [rows] and a distance-bias table [n_dist, rows] (both float32); returns n_dist."""
    if sinks is not None:
        _dense(sinks, "sinks", torch.float32)
        if sinks.numel() != rows:
            raise KernelError(f"{sinks.numel()} sinks for {rows} query rows")
    if dist_bias is None:
        return 0
    _dense(dist_bias, "dist_bias", torch.float32)
    if dist_bias.dim() != 2 or dist_bias.shape[1] != rows or dist_bias.shape[0] < 1:
        raise KernelError(f"a distance bias {tuple(dist_bias.shape)} for {rows} query rows")
    return int(dist_bias.shape[0])


def attn_prepare(src: torch.Tensor, q_off: int, k_off: int, v_off: int, freq: Optional[torch.Tensor], n_rot: int,
                 half_layout: bool, tok_pos: torch.Tensor, tok_slot: torch.Tensor, block_table: Optional[torch.Tensor],
                 k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], n_q_rows: int, d: int,
                 act_dtype: torch.dtype, status: torch.Tensor, append: bool = True,
                 bias: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 0.0,
                 temp_coef: float = 0.0, temp_every: int = 0) -> torch.Tensor:
    """Between projections (or convolutions) and attention: the queries of `src` [n, >= columns] at `q_off` come
    back as [n, n_q_rows, d] in `act_dtype`, their first `n_rot` dimensions turned by position x `freq`; with
    `k_off` >= 0 the keys (turned alike) and values at `k_off` / `v_off` go into the token's cache page.  Before the
    rotation, in float32: `bias` (a number per column, [queries | keys | values]) is added; with `norm_weight`
    ([queries | keys]) all of a token's query columns are divided by their root mean square (eps inside the root)
    and multiplied by their weights, and its key columns likewise; with `temp_every` > 0 the queries at position p
    are multiplied by 1 + temp_coef ln(floor((p + 1) / temp_every) + 1)."""
    l = require_gpu()
    _rows(src, "src")
    n = src.shape[0]
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (status, "status")):
        _dense(t, name, torch.int32)
    if n_rot:
        _dense(freq, "freq", torch.float32)
        if freq.numel() * 2 != n_rot:
            raise KernelError(f"{freq.numel()} frequencies for {n_rot} rotated dimensions")
    n_kh = n_vh = dv = page_size = max_pages = n_pages = 0
    if k_off >= 0:
        _dense(k_pool, "k_pool", act_dtype), _dense(v_pool, "v_pool", act_dtype), _dense(block_table, "block_table", torch.int32)
        n_pages, n_kh, page_size, pool_d = k_pool.shape
        _, n_vh, _, dv = v_pool.shape
        max_pages = block_table.shape[1]
        if pool_d != d:
            raise KernelError(f"key pool rows of {pool_d} for heads of {d}")
    cols_qk = n_q_rows * d + (n_kh * d if k_off >= 0 else 0)
    if bias is not None:
        _dense(bias, "bias")
        if bias.numel() != cols_qk + (n_vh * dv if k_off >= 0 else 0):
            raise KernelError(f"a bias of {bias.numel()} elements for {cols_qk} query and key columns and the values")
    if norm_weight is not None:
        _dense(norm_weight, "norm_weight")
        if norm_weight.numel() != cols_qk or not norm_eps > 0:
            raise KernelError(f"a norm weight of {norm_weight.numel()} elements for {cols_qk} query and key columns, eps {norm_eps}")
    q_out = torch.empty((n, n_q_rows, d), dtype=act_dtype, device=src.device)
    check(l.gi_attn_prepare(_ptr(src), code(src.dtype), src.stride(0), q_off, k_off, v_off, _ptr(freq) if n_rot else None,
                            n_rot, int(half_layout), _ptr(tok_pos), _ptr(tok_slot), _ptr(block_table) if k_off >= 0 else None,
                            _ptr(k_pool) if k_off >= 0 else None, _ptr(v_pool) if k_off >= 0 else None, _ptr(q_out),
                            code(act_dtype), n, n_q_rows, n_kh, n_vh, d, max(dv, 1), page_size, max_pages, n_pages,
                            int(append), _ptr(status), _ptr(bias), code(bias.dtype) if bias is not None else F32,
                            _ptr(norm_weight), code(norm_weight.dtype) if norm_weight is not None else F32,
                            float(norm_eps), float(temp_coef), int(temp_every), _stream()), l)
    return q_out


def attn_finish(att: torch.Tensor, heads: int, maps: int, lam: Optional[torch.Tensor], norm_eps: Optional[float],
                mul: float, gate: Optional[torch.Tensor], act_dtype: torch.dtype,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """att [n, heads * maps * dv] -> [n, heads * dv] in `act_dtype`: a_1 - lam a_2 for two maps, divided by its root
    mean square per head when `norm_eps` is given, times `mul`, times sigmoid(gate[:, head]).  `out` may be columns
    of a wider matrix."""
    l = require_gpu()
    _dense(att, "att")
    n = att.shape[0]
    dv = att.shape[1] // (heads * maps)
    if gate is not None:
        _rows(gate, "gate", act_dtype)
    if lam is not None:
        _dense(lam, "lam", torch.float32)
    if out is None:
        out = torch.empty((n, heads * dv), dtype=act_dtype, device=att.device)
    _rows(out, "out", act_dtype)
    if out.shape != (n, heads * dv):
        raise KernelError(f"out {tuple(out.shape)} for a result of {(n, heads * dv)}")
    check(l.gi_attn_finish(_ptr(att), code(att.dtype), maps, _ptr(lam), float(norm_eps or 0.0), int(norm_eps is not None),
                           float(mul), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out), out.stride(0),
                           code(act_dtype), n, heads, dv, _stream()), l)
    return out


def add_dyt(delta: Optional[torch.Tensor], delta_scale: Optional[torch.Tensor], residual: torch.Tensor,
            weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor, act_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, write_residual: bool = True) -> torch.Tensor:
    """tanh(alpha s) * weight + bias for s = residual (+ delta * delta_scale), in `act_dtype`; the float32 sum goes
    back into `residual` unless `rows` (int32) picks rows or `write_residual` is False."""
    l = require_gpu()
    _dense(residual, "residual", torch.float32), _dense(weight, "weight"), _dense(bias, "bias", weight.dtype)
    _dense(alpha, "alpha", weight.dtype)
    dim = residual.shape[-1]
    if weight.numel() != dim or bias.numel() != dim or alpha.numel() != 1:
        raise KernelError(f"norm tensors of {weight.numel()}, {bias.numel()} and {alpha.numel()} elements for rows of {dim}")
    if delta is not None:
        _dense(delta, "delta", act_dtype)
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} and residual {tuple(residual.shape)} differ")
    if delta_scale is not None and _dense(delta_scale, "delta_scale").numel() != dim:
        raise KernelError(f"a factor per channel has {delta_scale.numel()} elements for rows of {dim}")
    if rows is not None:
        _dense(rows, "rows", torch.int32)
        n_rows, write_residual = rows.numel(), False
    else:
        n_rows = residual.numel() // dim
    out = torch.empty((n_rows, dim), dtype=act_dtype, device=residual.device)
    check(l.gi_add_dyt(_ptr(delta), _ptr(delta_scale), code(delta_scale.dtype) if delta_scale is not None else F32,
                       _ptr(residual), _ptr(weight), _ptr(bias), _ptr(alpha), code(weight.dtype), _ptr(out),
                       code(act_dtype), _ptr(rows), n_rows, dim, int(write_residual and delta is not None), _stream()), l)
    return out


def residual_add_scaled(delta: torch.Tensor, delta_scale: Optional[torch.Tensor], residual: torch.Tensor) -> None:
    """residual += delta * delta_scale (a factor per channel; None: 1)."""
    l = require_gpu()
    _dense(delta, "delta"), _dense(residual, "residual", torch.float32)
    if delta.shape != residual.shape:
        raise KernelError(f"delta {tuple(delta.shape)} and residual {tuple(residual.shape)} differ")
    n, dim = residual.shape
    check(l.gi_residual_add_scaled(_ptr(delta), code(delta.dtype), _ptr(delta_scale),
                                   code(delta_scale.dtype) if delta_scale is not None else F32, _ptr(residual), n, dim,
                                   _stream()), l)


GLU_KINDS = {"silu": 0, "gelu_tanh": 1, "swish": 2}


def glu_shape(activation: str, swish_alpha: float = 1.0, gate_max: Optional[float] = None,
              up_limit: Optional[float] = None, up_shift: float = 0.0) -> tuple:
    """The gated unit act(min(gate, gate_max)) * (clamp(up, -up_limit, up_limit) + up_shift) as the kernels take it:
    (kind, alpha, gate_max, up_limit, up_shift); a limit of None is none."""
    if activation not in GLU_KINDS:
        raise KernelError(f"gated-unit activation {activation!r} is none of {sorted(GLU_KINDS)}")
    inf = float("inf")
    return (GLU_KINDS[activation], float(swish_alpha), inf if gate_max is None else float(gate_max),
            inf if up_limit is None else float(up_limit), float(up_shift))


def glu(gate_up: torch.Tensor, activation, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """unit(gate, up) for rows [gate | up]; `activation` is "silu", "gelu_tanh" or "swish" (plain act(gate) * up), or a
    `glu_shape` tuple with limits and a shift.  `out` may be columns of a wider matrix."""
    l = require_gpu()
    _rows(gate_up, "gate_up")
    n, two_i = gate_up.shape
    shape = glu_shape(activation) if isinstance(activation, str) else activation
    if out is None:
        out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _rows(out, "out", gate_up.dtype)
    if out.shape != (n, two_i // 2):
        raise KernelError(f"out {tuple(out.shape)} for a result of {(n, two_i // 2)}")
    check(l.gi_glu(_ptr(gate_up), gate_up.stride(0), _ptr(out), out.stride(0), code(gate_up.dtype), n, two_i // 2, *shape,
                   _stream()), l)
    return out


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    l = require_gpu()
    _dense(z, "z")
    out = torch.empty_like(z)
    check(l.gi_relu_squared(_ptr(z), _ptr(out), code(z.dtype), z.numel(), _stream()), l)
    return out


def scaled_sum(a: torch.Tensor, ca: float, b: torch.Tensor, cb: float) -> torch.Tensor:
    """a * ca + b * cb, float32 inside."""
    l = require_gpu()
    _dense(a, "a"), _dense(b, "b", a.dtype)
    if a.shape != b.shape:
        raise KernelError(f"{tuple(a.shape)} and {tuple(b.shape)} differ")
    out = torch.empty_like(a)
    check(l.gi_scaled_sum(_ptr(a), float(ca), _ptr(b), float(cb), _ptr(out), code(a.dtype), a.numel(), _stream()), l)
    return out


def router_logits(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [n, hidden] . w[experts, hidden]^T as float32, for a float32 weight and activations of either type."""
    l = require_gpu()
    _rows(x, "x"), _dense(w, "w", torch.float32)
    n, hidden = x.shape
    if w.shape[1] != hidden:
        raise KernelError(f"router weight {tuple(w.shape)} for rows of {hidden}")
    z = torch.empty((n, w.shape[0]), dtype=torch.float32, device=x.device)
    check(l.gi_router_logits(_ptr(x), x.stride(0), code(x.dtype), _ptr(w), _ptr(z), n, w.shape[0], hidden, _stream()), l)
    return z


def router_topk(logits: torch.Tensor, top: int):
    """(chosen experts int32 [n, top] in falling order of their logits, softmax over the chosen logits float32)."""
    l = require_gpu()
    _rows(logits, "logits", torch.float32)
    n, E = logits.shape
    idx = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    wt = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    check(l.gi_router_topk(_ptr(logits), logits.stride(0), E, int(top), _ptr(idx), _ptr(wt), n, _stream()), l)
    return idx, wt


def router_select(logits: torch.Tensor, top: int, groups: int, keep: int, scale: float, sigmoid: bool = False,
                  correction: Optional[torch.Tensor] = None, group_top: int = 1, normalize: bool = False):
    """Scores = softmax of the float32 `logits` over all experts (or, with `sigmoid`, the sigmoid of each); of
    `groups` equal groups of neighbouring experts the `keep` with the largest best score (or sum of the two best, with
    `group_top` 2) stay; (the `top` experts with the largest scores among those int32 [n, top] in falling order, their
    scores times `scale` float32).  `correction` float32 [experts] is added to the scores that choose groups and
    experts, not to the weights; `normalize` divides the weights by their sum (+ 1e-20) before the factor."""
    l = require_gpu()
    _rows(logits, "logits", torch.float32)
    n, E = logits.shape
    idx = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    wt = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    if correction is not None:
        _dense(correction, "correction", torch.float32)
        if correction.numel() != E:
            raise KernelError(f"a correction of {correction.numel()} elements for {E} experts")
    check(l.gi_router_select(_ptr(logits), logits.stride(0), E, int(top), int(groups), int(keep), float(scale), _ptr(idx),
                             _ptr(wt), n, int(sigmoid), _ptr(correction), int(group_top), int(normalize), _stream()), l)
    return idx, wt


def moe_rowwise(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, idx: torch.Tensor, wt: torch.Tensor,
                activation, add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(add[t] +) sum_j wt[t, j] W_down[idx[t, j]] act(W_up[idx[t, j]] x[t]) with the chosen experts read from device memory:
    w_up [E, ff, hidden] and `activation` "relu_squared" or "silu", or w_up [E, 2 ff, hidden] (gate rows, then up
    rows) and a `glu_shape` tuple; w_down [E, hidden, ff]; one row of x at a time (decode steps)."""
    l = require_gpu()
    _rows(x, "x"), _dense(w_up, "w_up", x.dtype), _dense(w_down, "w_down", x.dtype)
    _dense(idx, "idx", torch.int32), _dense(wt, "wt", torch.float32)
    n, hidden = x.shape
    E, _, ff = w_down.shape
    top = idx.shape[1]
    gated = not isinstance(activation, str)
    if w_up.shape != (E, (2 if gated else 1) * ff, hidden):
        raise KernelError(f"expert matrices {tuple(w_up.shape)} and {tuple(w_down.shape)} do not fit each other")
    a = torch.empty((n, top, ff), dtype=x.dtype, device=x.device)
    part = torch.empty((n * top, hidden), dtype=x.dtype, device=x.device)
    act = 2 if gated else {"relu_squared": 0, "silu": 1}[activation]
    unit = activation if gated else glu_shape("silu")
    check(l.gi_moe_up(_ptr(x), x.stride(0), _ptr(w_up), _ptr(idx), _ptr(a), code(x.dtype), n, top, E, ff, hidden, act,
                      *unit, _stream()), l)
    check(l.gi_moe_down(_ptr(a), _ptr(w_down), _ptr(idx), _ptr(part), code(x.dtype), n, top, E, ff, hidden, _stream()), l)
    return moe_combine(part, None, wt, add)


def moe_group(idx: torch.Tensor, x: torch.Tensor, n_experts: int):
    """The (token, choice) pairs of idx [n, top] in the order of their experts (stable): returns (where int32 [n, top],
    each pair's row; ends int32 [n_experts], each expert's last row + 1; rows [n * top, hidden], x's rows in that
    order)."""
    l = require_gpu()
    _dense(idx, "idx", torch.int32), _rows(x, "x")
    n, top = idx.shape
    hidden = x.shape[1]
    where = torch.empty((n, top), dtype=torch.int32, device=x.device)
    ends = torch.empty((n_experts,), dtype=torch.int32, device=x.device)
    rows = torch.empty((n * top, hidden), dtype=x.dtype, device=x.device)
    scratch = torch.empty((-(-(n * top) // 1024) * n_experts,), dtype=torch.int32, device=x.device)
    check(l.gi_moe_group(_ptr(idx), _ptr(x), x.stride(0), code(x.dtype), _ptr(where), _ptr(ends), _ptr(rows), _ptr(scratch),
                         n, top, n_experts, hidden, _stream()), l)
    counters.launches += 3
    return where, ends, rows


def moe_combine(buf: torch.Tensor, where: Optional[torch.Tensor], wt: torch.Tensor,
                add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t] = (add[t] +) sum_j wt[t, j] buf[where[t, j]] (float32 sums in the order of j); without `where`: row
    t * top + j."""
    l = require_gpu()
    _dense(buf, "buf"), _dense(wt, "wt", torch.float32)
    if where is not None:
        _dense(where, "where", torch.int32)
    n, top = wt.shape
    if add is not None:
        _dense(add, "add", buf.dtype)
        if add.shape != (n, buf.shape[1]):
            raise KernelError(f"an addend {tuple(add.shape)} for a result of {(n, buf.shape[1])}")
    y = torch.empty((n, buf.shape[1]), dtype=buf.dtype, device=buf.device)
    check(l.gi_moe_combine(_ptr(buf), _ptr(where), _ptr(wt), _ptr(y), code(buf.dtype), n, top, buf.shape[1], _ptr(add),
                           _stream()), l)
    return y


def _rows(t: torch.Tensor, name: str, dtype=None) -> torch.Tensor:
    """A 2-D tensor whose rows are dense but may lie apart (columns of a wider product's output)."""
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} of shape {tuple(t.shape)} and strides {t.stride()} is no matrix of dense rows on the GPU")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} is {t.dtype}, the kernel wants {dtype}")
    return t


def gate_norm_add(y: torch.Tensor, gate: Optional[torch.Tensor], bias: Optional[torch.Tensor], weight: torch.Tensor,
                  eps: float, residual: torch.Tensor, want_copy: bool) -> Optional[torch.Tensor]:
    """residual += rmsnorm(y * sigmoid(gate + bias)) * weight, all in float32 (without `gate`: the norm of y
    itself).  With `want_copy` returns the new residual rounded to y's type, for the next products."""
    l = require_gpu()
    act = y.dtype
    _rows(y, "y"), _dense(residual, "residual", torch.float32), _dense(weight, "weight")
    n, dim = y.shape
    if residual.shape != (n, dim) or weight.numel() != dim:
        raise KernelError(f"y {tuple(y.shape)}, residual {tuple(residual.shape)} and a norm weight of {weight.numel()} differ")
    if gate is not None:
        _rows(gate, "gate", act)
        if gate.shape != (n, dim) or (bias is not None and _dense(bias, "bias").numel() != dim):
            raise KernelError(f"gate {tuple(gate.shape)} / bias do not fit rows of {dim}")
    copy = torch.empty((n, dim), dtype=act, device=y.device) if want_copy else None
    check(l.gi_gate_norm_add(_ptr(y), y.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(bias),
                             code(bias.dtype) if bias is not None else F32, _ptr(weight), code(weight.dtype),
                             _ptr(residual), _ptr(copy), code(act), n, dim, float(eps), _stream()), l)
    return copy


def xielu(z: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    """softplus(p) z^2 + z/2 for z > 0, (1/2 + softplus(q)) (e^z - 1 - z) + z/2 otherwise; pq = [p, q] on the device."""
    l = require_gpu()
    _rows(z, "z"), _dense(pq, "pq")
    if pq.numel() != 2:
        raise KernelError(f"xielu takes two numbers, not {pq.numel()}")
    n, cols = z.shape
    out = torch.empty((n, cols), dtype=z.dtype, device=z.device)
    check(l.gi_xielu(_ptr(z), z.stride(0), _ptr(out), code(z.dtype), _ptr(pq), code(pq.dtype), n, cols, _stream()), l)
    return out


def gated_group_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, groups: int,
                        gate_kind: str, mul: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """o float32 [n, groups * gs]: each group divided by its root mean square, times weight (one per column, or
    one per column of a group), times sigmoid(gate) or silu(gate), times `mul`; returns gate's type.  `out` may be
    columns of a wider matrix."""
    l = require_gpu()
    _dense(o, "o", torch.float32), _rows(gate, "gate"), _dense(weight, "weight")
    n, cols = o.shape
    if cols % groups or gate.shape != (n, cols):
        raise KernelError(f"o {tuple(o.shape)} in {groups} groups, gate {tuple(gate.shape)}")
    if out is None:
        out = torch.empty((n, cols), dtype=gate.dtype, device=o.device)
    _rows(out, "out", gate.dtype)
    if out.shape != (n, cols):
        raise KernelError(f"out {tuple(out.shape)} for a result of {(n, cols)}")
    check(l.gi_gated_group_rmsnorm(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), code(weight.dtype), weight.numel(),
                                   _ptr(out), code(gate.dtype), n, groups, cols // groups, float(eps),
                                   {"sigmoid": 0, "silu": 1}[gate_kind], float(mul), out.stride(0), _stream()), l)
    return out


def scan_state_floats(key_dim: int, value_dim: int) -> int:
    """Floats of one head's recurrent state as the scan kernels lay it out (keys padded for their loads)."""
    from .library import lib
    n = lib().gi_scan_state_floats(int(key_dim), int(value_dim))
    if n < 0:
        raise KernelError(f"a key dimension of {key_dim} is beyond the scan kernels' 256")
    return int(n)


def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, tok_slot: torch.Tensor,
                     activation: str = "silu", renew_state: bool = False, in_bias: Optional[torch.Tensor] = None,
                     out_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu (or, with activation "none", the plain sum) of the causal convolution over time of x [n, C] (rows may lie apart) with taps [C, K], the K-1 inputs
    before the step's first token of a sequence taken from `state` [slots, >= (K-1) C] (a view of float32 state
    rows); returns float32 [n, C].  Call `conv_state_update` afterwards, or pass `renew_state` when no two rows of
    the step belong to one sequence (a decode step): the same launch then renews the state."""
    l = require_gpu()
    _rows(x, "x"), _dense(taps, "taps"), _rows(state, "state", torch.float32), _dense(tok_slot, "tok_slot", torch.int32)
    n, C = x.shape
    out = torch.empty((n, C), dtype=torch.float32, device=x.device)
    bias_dtype = _bias_pair(in_bias, out_bias, C)
    check(l.gi_causal_conv_biased(_ptr(x), x.stride(0), code(x.dtype), C, _ptr(taps), code(taps.dtype), taps.shape[1],
                                  _ptr(state), state.stride(0), _ptr(tok_slot), _ptr(out), n, 2 if renew_state else 0,
                                  {"none": 0, "silu": 1}[activation], _ptr(in_bias), _ptr(out_bias), bias_dtype,
                                  _stream()), l)
    return out


def _bias_pair(in_bias, out_bias, C: int) -> int:
    """The one dtype code of a convolution's two optional biases [C]."""
    given = [b for b in (in_bias, out_bias) if b is not None]
    for b in given:
        _dense(b, "bias")
        if b.numel() != C or b.dtype != given[0].dtype:
            raise KernelError(f"a bias of {b.numel()} {b.dtype} elements for {C} channels (both biases share a type)")
    return code(given[0].dtype) if given else F32


def conv_state_update(x: torch.Tensor, n_taps: int, state: torch.Tensor, tok_slot: torch.Tensor,
                      in_bias: Optional[torch.Tensor] = None) -> None:
    """Each sequence's state becomes the last K-1 inputs it has seen (this step's rows, then what the state held);
    `in_bias` [C] is added to the step's rows as the convolution adds it."""
    l = require_gpu()
    _rows(x, "x"), _rows(state, "state", torch.float32), _dense(tok_slot, "tok_slot", torch.int32)
    if n_taps <= 1:
        return
    check(l.gi_causal_conv_biased(_ptr(x), x.stride(0), code(x.dtype), x.shape[1], None, F32, n_taps, _ptr(state),
                                  state.stride(0), _ptr(tok_slot), None, x.shape[0], 1, 1, _ptr(in_bias), None,
                                  _bias_pair(in_bias, None, x.shape[1]), _stream()), l)


def rglru_gates(u: torch.Tensor, wa_t: torch.Tensor, wi_t: torch.Tensor, ba: torch.Tensor, bi: torch.Tensor,
                lam: torch.Tensor, decay_scale: float):
    """The decay and the gated input of a real-gated linear recurrent unit from its input u float32 [n, width]:
    per block of channels r = sigmoid(Wa u + ba), i = sigmoid(Wi u + bi) with the matrices given transposed
    ([blocks, in, out]); a = exp(-decay_scale r softplus(lam)), b = sqrt(1 - a^2) i u.  Returns (a, b) float32."""
    l = require_gpu()
    _dense(u, "u", torch.float32), _dense(wa_t, "wa_t"), _dense(wi_t, "wi_t", wa_t.dtype)
    n, width = u.shape
    blocks, bw, bw2 = wa_t.shape
    if bw != bw2 or blocks * bw != width or wi_t.shape != wa_t.shape:
        raise KernelError(f"gate matrices {tuple(wa_t.shape)} / {tuple(wi_t.shape)} for {width} channels")
    for v, name in ((ba, "ba"), (bi, "bi"), (lam, "lam")):
        _dense(v, name, ba.dtype)
        if v.numel() != width:
            raise KernelError(f"{name} has {v.numel()} elements for {width} channels")
    a = torch.empty((n, width), dtype=torch.float32, device=u.device)
    b = torch.empty((n, width), dtype=torch.float32, device=u.device)
    check(l.gi_rglru_gates(_ptr(u), _ptr(wa_t), _ptr(wi_t), code(wa_t.dtype), _ptr(ba), _ptr(bi), _ptr(lam), code(ba.dtype),
                           float(decay_scale), _ptr(a), _ptr(b), n, width, blocks, _stream()), l)
    return a, b


def rglru_scan(a: torch.Tensor, b: torch.Tensor, y: torch.Tensor, y_bias: Optional[torch.Tensor], state: torch.Tensor,
               spans: Optional[torch.Tensor], tok_slot: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """S <- a_t S + b_t along every sequence's rows from and into `state` (float32 rows per slot, the first `width`
    columns); returns S_t * gelu_tanh(y_t + y_bias) in y's type.  y and `out` may be columns of wider matrices."""
    l = require_gpu()
    _dense(a, "a", torch.float32), _dense(b, "b", torch.float32), _rows(y, "y"), _rows(state, "state", torch.float32)
    n, width = a.shape
    if y.shape != (n, width) or b.shape != a.shape:
        raise KernelError(f"a {tuple(a.shape)}, b {tuple(b.shape)} and y {tuple(y.shape)} differ")
    if y_bias is not None:
        _dense(y_bias, "y_bias")
    if out is None:
        out = torch.empty((n, width), dtype=y.dtype, device=y.device)
    _rows(out, "out", y.dtype)
    spans, n_seqs = _scan_args(spans, tok_slot, n)
    check(l.gi_rglru_scan(_ptr(a), _ptr(b), _ptr(y), y.stride(0), code(y.dtype), _ptr(y_bias),
                          code(y_bias.dtype) if y_bias is not None else F32, _ptr(state), state.stride(0), _ptr(spans),
                          _ptr(tok_slot), _ptr(out), out.stride(0), n_seqs, width, _stream()), l)
    return out


def _scan_args(spans: Optional[torch.Tensor], tok_slot: torch.Tensor, n_rows: int):
    _dense(tok_slot, "tok_slot", torch.int32)
    if spans is None:
        return None, n_rows
    _dense(spans, "spans", torch.int32)
    if spans.dim() != 2 or spans.shape[1] != 3:
        raise KernelError(f"spans of shape {tuple(spans.shape)}, not [sequences, 3]")
    return spans, spans.shape[0]


def decay_scan(qkv: torch.Tensor, offsets: tuple, decay: torch.Tensor, state: torch.Tensor,
               spans: Optional[torch.Tensor], tok_slot: torch.Tensor, n_heads: int, key_dim: int,
               value_dim: int) -> torch.Tensor:
    """Linear attention with a fixed decay per head over the step's rows, from and to `state` [slots, floats]:
    S = decay S + silu(k) silu(v)^T, o = S^T silu(q).  q, k, v are columns of `qkv` at `offsets`.  `spans`
    [n_seq, 3] = {slot, first row, rows}; None: every row is a sequence of its own (slot from tok_slot).
    Returns float32 [n, n_heads * value_dim]."""
    l = require_gpu()
    _rows(qkv, "qkv"), _dense(decay, "decay", torch.float32), _rows(state, "state", torch.float32)
    n = qkv.shape[0]
    spans, n_seq = _scan_args(spans, tok_slot, n)
    out = torch.empty((n, n_heads * value_dim), dtype=torch.float32, device=qkv.device)
    check(l.gi_decay_scan(_ptr(qkv), qkv.stride(0), code(qkv.dtype), *map(int, offsets), _ptr(decay), _ptr(state),
                          state.stride(0), _ptr(spans), _ptr(tok_slot), _ptr(out), n_seq, n_heads, key_dim, value_dim,
                          _stream()), l)
    return out


def delta_scan(qkv: torch.Tensor, offsets: tuple, ab: torch.Tensor, ab_offsets: tuple, A_log: torch.Tensor,
               dt_bias: torch.Tensor, state: torch.Tensor, spans: Optional[torch.Tensor], tok_slot: torch.Tensor,
               n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, unit_eps: float,
               channel_decay: bool = False, decay_logits: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The gated delta rule over the step's rows, from and to `state`.  `qkv` float32 [n, C] holds q, k (per key
    head) and v (per head) at `offsets`; `ab` float32 holds the logits of beta and of the decay at `ab_offsets`
    (one column per head; with `channel_decay` the decay has one column per head and key channel, and dt_bias as
    many elements).  `decay_logits`: the decay's logits as a float32 matrix of their own (its column
    ab_offsets[1] is the first).  Returns float32 [n, n_heads * value_dim]."""
    l = require_gpu()
    _rows(qkv, "qkv", torch.float32), _rows(ab, "ab", torch.float32), _rows(state, "state", torch.float32)
    _dense(A_log, "A_log"), _dense(dt_bias, "dt_bias", A_log.dtype)
    n = qkv.shape[0]
    spans, n_seq = _scan_args(spans, tok_slot, n)
    out = torch.empty((n, n_heads * value_dim), dtype=torch.float32, device=qkv.device)
    if decay_logits is not None:
        _rows(decay_logits, "decay_logits", torch.float32)
    check(l.gi_delta_scan(_ptr(qkv), qkv.stride(0), *map(int, offsets), _ptr(ab), ab.stride(0),
                          *map(int, ab_offsets), _ptr(decay_logits),
                          decay_logits.stride(0) if decay_logits is not None else 0, _ptr(A_log), _ptr(dt_bias), code(A_log.dtype), _ptr(state),
                          state.stride(0), _ptr(spans), _ptr(tok_slot), _ptr(out), n_seq, n_heads, n_kv_heads,
                          key_dim, value_dim, float(unit_eps), float(key_dim) ** -0.5, int(channel_decay), _stream()), l)
    return out


def causal_sink_softmax(scores: torch.Tensor, heads: int, first_pos: int, scale: float,
                        sinks: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """Softmax over the rows of float32 `scores` [tokens * heads, keys]: row t * heads + h belongs to the query at
    position first_pos + t and sees keys 0 .. first_pos + t; `scale` multiplies the scores; exp(sinks[h]) joins the
    denominator.  Returns the weights [tokens * heads, keys] in `out_dtype`, zeros beyond each row's position."""
    l = require_gpu()
    _rows(scores, "scores", torch.float32)
    n, keys = scores.shape
    if sinks is not None and _dense(sinks, "sinks").numel() != heads:
        raise KernelError(f"{sinks.numel()} sinks for {heads} heads")
    out = torch.empty((n, keys), dtype=out_dtype, device=scores.device)
    check(l.gi_causal_sink_softmax(_ptr(scores), scores.stride(0), _ptr(out), keys, code(out_dtype), n, heads,
                                   int(first_pos), keys, float(scale), _ptr(sinks),
                                   code(sinks.dtype) if sinks is not None else F32, _stream()), l)
    return out


def latent_decode_takes(dtype: torch.dtype, row: int, rank: int, heads: int) -> bool:
    """Whether the shared-rows decode kernel takes these sizes (bfloat16, rows a multiple of 8, at most 512 value
    columns, and shared memory for a group of heads beside 32 rows)."""
    group = 8 * (4 if heads > 16 else (2 if heads > 8 else 1))
    return (dtype == torch.bfloat16 and row % 8 == 0 and 0 < rank <= min(row, 512)
            and group * row * 4 + 32 * (row // 2 + 1) * 4 <= 220 * 1024)


def latent_decode(q: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor, tok_pos: torch.Tensor,
                  tok_slot: torch.Tensor, scale: float, sinks: Optional[torch.Tensor], rank: int,
                  status: torch.Tensor, n_splits: Optional[int] = None) -> torch.Tensor:
    """Attention of one new token per sequence, q [n, heads, row] bfloat16, over latent rows shared by all heads
    (`pool` [pages, 1, page_size, row]); values are the rows' first `rank` columns.  Returns [n, heads * rank]."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(pool, "pool", torch.bfloat16)
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table"), (status, "status")):
        _dense(t, name, torch.int32)
    n, heads, row = q.shape
    n_pages, one, page_size, pool_row = pool.shape
    if one != 1 or pool_row != row:
        raise KernelError(f"a pool {tuple(pool.shape)} does not hold rows of {row} shared by all heads")
    if n_splits is None:
        # Slices of the keys: about 256 blocks in all, at most 16 slices.  Measured at 32 heads over rows of 576 with
        # 2,048 cached tokens (us at 4 / 8 / 16 / 32 slices): 1 sequence 108 / 69 / 52 / 52, 8 sequences
        # 108 / 69 / 54 / 73, 64 sequences 210 / 228 / 245 / 329.
        groups = -(-heads // 32)
        n_splits = max(1, min(16, 256 // max(1, n * groups)))
    part = torch.empty((n, n_splits, heads, rank + 2), dtype=torch.float32, device=q.device)
    out = torch.empty((n, heads * rank), dtype=torch.bfloat16, device=q.device)
    check(l.gi_latent_decode(_ptr(q), _ptr(pool), _ptr(block_table), _ptr(tok_pos), _ptr(tok_slot), _ptr(part),
                             _ptr(out), n, heads, row, rank, page_size, block_table.shape[1], n_pages, n_splits,
                             float(scale), _ptr(sinks), code(sinks.dtype) if sinks is not None else F32,
                             _ptr(status), _stream()), l)
    counters.launches += 1                     # two kernels behind one entry point
    return out


def latent_prepare(q_src: torch.Tensor, q_off: int, kv_src: Optional[torch.Tensor], c_off: int, q_lat: torch.Tensor,
                   norm_w: Optional[torch.Tensor], eps: float, freq: torch.Tensor, magnitude: float, n_rot: int,
                   tok_pos: torch.Tensor, tok_slot: torch.Tensor, block_table: torch.Tensor, pool: torch.Tensor,
                   n_heads: int, plain_dim: int, rot_dim: int, rank: int, status: torch.Tensor, append: bool = True,
                   half_layout: bool = False) -> torch.Tensor:
    """Latent attention between projections and attention: writes each token's cache row [normed latent | rotated
    shared key part | zeros] into `pool` [pages, 1, page_size, row] from columns c_off .. of `kv_src` (None for a
    layer that reads rows another layer cached) and returns the queries [n, heads, row] = [q' | rotated part |
    zeros], q' = `q_lat` [n, heads, rank], the rotated part from `q_src`'s columns (heads of plain_dim + rot_dim from
    q_off on).  `half_layout`: dimension i turns with i + n_rot/2 instead of 2i with 2i + 1."""
    l = require_gpu()
    act = q_src.dtype
    _rows(q_src, "q_src"), _dense(q_lat, "q_lat", act), _dense(freq, "freq", torch.float32)
    _dense(pool, "pool", act)
    if kv_src is not None:
        _rows(kv_src, "kv_src", act), _dense(norm_w, "norm_w")
    elif append:
        raise KernelError("latent_prepare: nothing to append without a latent")
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table"), (status, "status")):
        _dense(t, name, torch.int32)
    n = q_src.shape[0]
    n_pages, one, page_size, row_w = pool.shape
    if one != 1 or q_lat.shape != (n, n_heads, rank) or freq.numel() * 2 != n_rot or \
            (kv_src is not None and norm_w.numel() != rank):
        raise KernelError("latent_prepare: the pool, q_lat, the norm weight or the frequencies do not fit the sizes")
    q_out = torch.empty((n, n_heads, row_w), dtype=act, device=q_src.device)
    check(l.gi_latent_prepare(_ptr(q_src), q_src.stride(0), q_off, _ptr(kv_src), kv_src.stride(0) if kv_src is not None else 0,
                              c_off, int(half_layout), _ptr(q_lat), code(act), _ptr(norm_w),
                              code(norm_w.dtype) if norm_w is not None else F32, float(eps), _ptr(freq), float(magnitude),
                              n_rot, _ptr(tok_pos), _ptr(tok_slot), _ptr(block_table), _ptr(pool), _ptr(q_out), n, n_heads,
                              plain_dim, rot_dim, rank, row_w, page_size, block_table.shape[1], n_pages,
                              int(append and kv_src is not None), _ptr(status), _stream()), l)
    return q_out


def sgemm_nt(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M,K] . w[N,K]^T in true float32."""
    l = require_gpu()
    _dense(a, "a", torch.float32), _dense(w, "w", torch.float32)
    (m, k), (n, k2) = a.shape, w.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: a {tuple(a.shape)}, w {tuple(w.shape)}")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    _dense(out, "out", torch.float32)
    check(l.gi_sgemm_nt(_ptr(a), _ptr(w), _ptr(out), m, n, k, k, n, _stream()), l)
    return out


def sgemm_nt_strided(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """a [M,K] . w[N,K]^T in true float32 into `out` [M,N]; the rows of a and of out may lie apart."""
    l = require_gpu()
    _rows(a, "a", torch.float32), _dense(w, "w", torch.float32), _rows(out, "out", torch.float32)
    (m, k), (n, k2) = a.shape, w.shape
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"a {tuple(a.shape)}, w {tuple(w.shape)} and out {tuple(out.shape)} do not fit")
    check(l.gi_sgemm_nt(_ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(0) if m > 1 else k,
                        out.stride(0) if m > 1 else n, _stream()), l)
    return out


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [M<=8, K] . w[N,K]^T, bfloat16 operands, float32 accumulation."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w, "w", torch.bfloat16)
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w.shape)}")
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    check(l.gi_gemv_bf16(_ptr(x), _ptr(w), _ptr(out), code(out_dtype), m, n, k, _stream()), l)
    return out


def gemm_skinny_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, n_split: int = 0,
                     wide: int = -1) -> torch.Tensor:
    """x [M<=16, K] . w[N,K]^T on the tensor cores with W streamed once.  K is shared by a cluster of
    `n_split` CTAs (1 to 8; 0: chosen from the sizes); `wide` picks 64 (1) or 32 (0) rows of W per
    CTA (-1: chosen from the sizes)."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w, "w", torch.bfloat16)
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w.shape)}")
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    check(l.gi_gemm_skinny_bf16(_ptr(x), _ptr(w), _ptr(out), code(out_dtype), m, n, k, n_split, wide, _stream()), l)
    return out


def gemv_swiglu_bf16(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for one row x [1, K]: the bandwidth kernel with a gate and an up row per warp
    and the activation at its end.  Returns [1, I] bfloat16, the bits of `swiglu(gemv_bf16(x, w_gate_up))`."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w_gate_up, "w_gate_up", torch.bfloat16)
    (m, k), (n2, k2) = x.shape, w_gate_up.shape
    if m != 1 or k != k2:
        raise KernelError(f"gemv_swiglu_bf16 takes one row: x {tuple(x.shape)}, w {tuple(w_gate_up.shape)}")
    out = torch.empty((1, n2 // 2), dtype=torch.bfloat16, device=x.device)
    check(l.gi_gemv_swiglu_bf16(_ptr(x), _ptr(w_gate_up), _ptr(out), n2, k, _stream()), l)
    return out


def gemm_skinny_swiglu_bf16(x: torch.Tensor, w_gate_up: torch.Tensor, n_split: int = 0, wide: int = -1) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for x [M<=16, K] and w_gate_up = [Wg; Wu] ([2 I, K], the gate first) with the
    activation in the last step of the skinny product.  Returns [M, I] bfloat16: `swiglu(gemm_skinny_bf16(x,
    w_gate_up))` up to the rounding of the sums (the kernels walk K in different orders)."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w_gate_up, "w_gate_up", torch.bfloat16)
    (m, k), (n2, k2) = x.shape, w_gate_up.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w_gate_up.shape)}")
    out = torch.empty((m, n2 // 2), dtype=torch.bfloat16, device=x.device)
    check(l.gi_gemm_skinny_swiglu_bf16(_ptr(x), _ptr(w_gate_up), _ptr(out), m, n2, k, n_split, wide, _stream()), l)
    return out


def _glu_out(x, w_gate_up, out):
    _dense(x, "x", torch.bfloat16), _dense(w_gate_up, "w_gate_up", torch.bfloat16)
    (m, k), (n2, k2) = x.shape, w_gate_up.shape
    if k != k2 or n2 % 2:
        raise KernelError(f"x {tuple(x.shape)} does not fit a gate and an up half {tuple(w_gate_up.shape)}")
    if out is None:
        out = torch.empty((m, n2 // 2), dtype=torch.bfloat16, device=x.device)
    _rows(out, "out", torch.bfloat16)
    if out.shape != (m, n2 // 2):
        raise KernelError(f"out {tuple(out.shape)} for a result of {(m, n2 // 2)}")
    return m, n2, k, out


def gemm_skinny_glu_bf16(x: torch.Tensor, w_gate_up: torch.Tensor, unit: tuple, out: Optional[torch.Tensor] = None,
                         n_split: int = 0, wide: int = -1) -> torch.Tensor:
    """unit(x . Wg^T, x . Wu^T) for x [M<=16, K] and w_gate_up = [Wg; Wu] with the gated unit (a `glu_shape` tuple) in
    the last step of the skinny product; `out` may be columns of a wider matrix.  `glu(gemm_skinny_bf16(x,
    w_gate_up), unit)` up to the rounding of the sums."""
    l = require_gpu()
    m, n2, k, out = _glu_out(x, w_gate_up, out)
    check(l.gi_gemm_skinny_glu_bf16(_ptr(x), _ptr(w_gate_up), _ptr(out), out.stride(0), m, n2, k, *unit, n_split, wide,
                                    _stream()), l)
    return out


def gemm_tcgen05_glu_bf16(x: torch.Tensor, w_gate_up: torch.Tensor, unit: tuple,
                          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """unit(x . Wg^T, x . Wu^T) with the gated unit (a `glu_shape` tuple) in the epilogue of the tcgen05 product
    (pairs of CTAs); `out` may be columns of a wider matrix that start on 16 bytes.  The bits of
    `glu(gemm_tcgen05_bf16(x, w_gate_up), unit)`."""
    l = require_gpu()
    m, n2, k, out = _glu_out(x, w_gate_up, out)
    check(l.gi_gemm_tcgen05_glu_bf16(_ptr(x), _ptr(w_gate_up), _ptr(out), out.stride(0), m, n2, k, *unit,
                                     _ptr(tcgen05_error_flag(x.device)), _stream()), l)
    return out


_tcgen05_flag: dict = {}


def tcgen05_error_flag(device) -> torch.Tensor:
    """The int32 on `device` that the tcgen05 product sets when one of its bounded waits runs out."""
    key = torch.device(device).index or 0
    if key not in _tcgen05_flag:
        _tcgen05_flag[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tcgen05_flag[key]


class WaitRanOut(RuntimeError):
    """A kernel gave up one of its bounded waits; what it was writing is unspecified."""


def check_bounded_waits(device) -> None:
    """Raise `WaitRanOut` if a tcgen05 kernel launched on `device` since the last check gave up a bounded wait
    (synchronises).  The flag is cleared and the stream-K product's hand-over flags are zeroed, since a kernel
    that gave up may have left some of them set: the next call starts clean."""
    flag = tcgen05_error_flag(device)
    code = int(flag.item())
    if code:
        flag.zero_()
        key = torch.device(device).index or 0
        if key in _streamk_space:
            _streamk_space[key][1].zero_()
        raise WaitRanOut(f"a tcgen05 kernel gave up a bounded wait (code {code}: 11-13 product, 21-23 attention, "
                         "24 unmapped page, 31-33 stream-K product, 34 a partial sum that was never announced)")


def streamk_test_unanswered_flags(limit: int) -> None:
    """For the test of the bounded wait: with `limit` > 0 the stream-K product's hand-over flags are held back
    and the wait for them gives up after `limit` polls (see the kernel file); 0 restores the product."""
    require_gpu().gi_gemm_streamk_test_unanswered_flags(int(limit))


def gemm_tcgen05_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [M, K] . w[N, K]^T for many rows on tcgen05 tensor cores (TMA-fed, accumulators in tensor memory)."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w, "w", torch.bfloat16)
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w.shape)}")
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    check(l.gi_gemm_tcgen05_bf16(_ptr(x), _ptr(w), _ptr(out), code(out_dtype), m, n, k,
                                 _ptr(tcgen05_error_flag(x.device)), _stream()), l)
    return out


_streamk_space: dict = {}


def _streamk_workspace(device):
    """Per device: the float32 slots through which the CTAs of the stream-K product hand over partial tiles,
    and their flags (zero between calls: every call clears what it set)."""
    key = torch.device(device).index or 0
    if key not in _streamk_space:
        l = require_gpu()
        _streamk_space[key] = (torch.empty(l.gi_gemm_streamk_workspace_floats(), dtype=torch.float32, device=device),
                               torch.zeros(l.gi_gemm_streamk_flags(), dtype=torch.int32, device=device))
    return _streamk_space[key]


def gemm_streamk_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [M<=64, K] . w[N,K]^T on tcgen05 with W cut evenly over the SMs (TMA-fed, operands swapped: the rows of
    W fill the 128-row side of the instruction).  Calls on one device share a work space, so they must not
    overlap (they do not on one stream)."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w, "w", torch.bfloat16)
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w.shape)}")
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    partials, flags = _streamk_workspace(x.device)
    check(l.gi_gemm_streamk_bf16(_ptr(x), _ptr(w), _ptr(out), code(out_dtype), m, n, k, _ptr(partials), _ptr(flags),
                                 _ptr(tcgen05_error_flag(x.device)), _stream()), l)
    return out


def gemm_tcgen05_swiglu_bf16(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for w_gate_up = [Wg; Wu] ([2 I, K], the gate first): the gate/up product of
    a SwiGLU feed-forward with the activation in the epilogue of the tcgen05 product (pairs of CTAs).
    Returns [M, I] bfloat16, the bits of `swiglu(gemm_tcgen05_bf16(x, w_gate_up))`."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w_gate_up, "w_gate_up", torch.bfloat16)
    (m, k), (n2, k2) = x.shape, w_gate_up.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w_gate_up.shape)}")
    out = torch.empty((m, n2 // 2), dtype=torch.bfloat16, device=x.device)
    check(l.gi_gemm_tcgen05_swiglu_bf16(_ptr(x), _ptr(w_gate_up), _ptr(out), m, n2, k,
                                        _ptr(tcgen05_error_flag(x.device)), _stream()), l)
    return out


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], streams: Optional[torch.Tensor],
           counters: Optional[torch.Tensor], seed: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [n, vocab]: greedy where temperature <= 0 (or None),
    else a draw from softmax(logits / temperature) keyed by (seed, streams[row], counters[row])."""
    l = require_gpu()
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logits must be [rows, vocab] with dense rows")
    if not logits.is_cuda or logits.dtype != torch.float32:
        raise KernelError("logits must be float32 on the GPU")
    n, vocab = logits.shape
    if temperature is not None:
        _dense(temperature, "temperature", torch.float32)
    if streams is not None:
        _dense(streams, "streams", torch.int64)
    if counters is not None:
        _dense(counters, "counters", torch.int32)
    for t, name in ((temperature, "temperature"), (streams, "streams"), (counters, "counters")):
        if t is not None and t.numel() < n:
            raise KernelError(f"{name} has fewer entries than logits has rows")
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _dense(out, "out", torch.int32)
    n_chunks = l.gi_sample_chunks(vocab)
    part_v = torch.empty((n * n_chunks,), dtype=torch.float32, device=logits.device)
    part_i = torch.empty((n * n_chunks,), dtype=torch.int32, device=logits.device)
    check(l.gi_sample(_ptr(logits), logits.stride(0), n, vocab, _ptr(temperature), _ptr(streams), _ptr(counters),
                      int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(part_v), _ptr(part_i), _ptr(out), _stream()), l)
    counters_mod.launches += 1                               # the second pass
    return out


def mma_attention_takes(dtype: torch.dtype, head_dim: int, value_dim: Optional[int] = None) -> bool:
    """Whether the tensor-core attention kernels take this element type and head size (with `value_dim`: keys of
    `head_dim` and values of `value_dim`, which the general entry points take when one is twice the other)."""
    if value_dim is None or value_dim == head_dim:
        return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128
    from .library import lib
    return dtype == torch.bfloat16 and bool(lib().gi_attention_mma_takes(int(head_dim), int(value_dim)))


def attention_prefill_bf16(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                           q_tiles: torch.Tensor, scale: float, window: int, rows_covered: bool = False) -> torch.Tensor:
    """Flash attention of q [n, n_q, d] over the paged cache for steps with several tokens per sequence.
    `q_tiles` int32 [n_tiles, 4] cuts the rows into runs of at most 64 consecutive tokens of one
    sequence: {slot, first row, rows, position of the first row}.  Returns [n, n_q * d]."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(k_pool, "k_pool", torch.bfloat16), _dense(v_pool, "v_pool", torch.bfloat16)
    _dense(block_table, "block_table", torch.int32), _dense(q_tiles, "q_tiles", torch.int32)
    n, n_q, d = q.shape
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    if pool_d != d or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not fit head_dim {d}")
    if q_tiles.dim() != 2 or q_tiles.shape[1] != 4 or q_tiles.data_ptr() % 16:
        raise KernelError("q_tiles must be int32 [n_tiles, 4] starting on 16 bytes")
    # rows in no tile (padding) stay zero; when the caller says that every row lies in a tile, nothing is filled
    out = (torch.empty if rows_covered else torch.zeros)((n, n_q * d), dtype=q.dtype, device=q.device)
    check(l.gi_attention_prefill_bf16(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(q_tiles),
                                      q_tiles.shape[0], _ptr(out), n_q, n_kv, d, page_size, block_table.shape[1],
                                      n_pages, int(window or 0), float(scale), _stream()), l)
    return out


def _masked_shapes(q, k_pool, v_pool, maps):
    n, rows, d = q.shape
    n_pages, n_kh, page_size, pool_d = k_pool.shape
    n_kv, dv = v_pool.shape[1], v_pool.shape[3]
    if rows % maps or n_kh != n_kv * maps or pool_d != d or tuple(v_pool.shape) != (n_pages, n_kv, page_size, dv):
        raise KernelError(f"q {tuple(q.shape)}, keys {tuple(k_pool.shape)} and values {tuple(v_pool.shape)} do not fit "
                          f"{maps} maps per head")
    return n, rows, d, dv, n_pages, n_kv, page_size


def attention_prefill_masked_bf16(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                                  q_tiles: torch.Tensor, scale: float, window: int = 0, chunk: int = 0, maps: int = 1,
                                  rows_covered: bool = False, sinks: Optional[torch.Tensor] = None,
                                  dist_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The tensor-core prompt kernel with a chunk mask, optional `sinks` and `dist_bias` (as `attention_masked`), values of a size of their own and `maps` softmax maps per
    head over the same values: q [n, heads * maps, d] (a head's maps side by side), keys [pages, key/value heads *
    maps, page, d], values [pages, key/value heads, page, dv].  Returns [n, heads * maps * dv], a head's maps side
    by side."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(k_pool, "k_pool", torch.bfloat16), _dense(v_pool, "v_pool", torch.bfloat16)
    _dense(block_table, "block_table", torch.int32), _dense(q_tiles, "q_tiles", torch.int32)
    n, rows, d, dv, n_pages, n_kv, page_size = _masked_shapes(q, k_pool, v_pool, maps)
    if q_tiles.dim() != 2 or q_tiles.shape[1] != 4 or q_tiles.data_ptr() % 16:
        raise KernelError("q_tiles must be int32 [n_tiles, 4] starting on 16 bytes")
    n_dist = _check_sinks_bias(sinks, dist_bias, rows)
    out = (torch.empty if rows_covered else torch.zeros)((n, rows * dv), dtype=q.dtype, device=q.device)
    check(l.gi_attention_prefill_masked_bf16(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(q_tiles),
                                             q_tiles.shape[0], _ptr(out), rows // maps, n_kv, d, dv, page_size,
                                             block_table.shape[1], n_pages, int(window or 0), int(chunk or 0), int(maps),
                                             float(scale), _ptr(sinks), _ptr(dist_bias), n_dist, _stream()), l)
    return out


def attention_decode_masked_bf16(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                                 tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float, window: int = 0,
                                 chunk: int = 0, maps: int = 1, n_splits: Optional[int] = None,
                                 sinks: Optional[torch.Tensor] = None, dist_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The split-KV decode kernel with the same options: one token per sequence, q [n_seqs, heads * maps, d].
    Returns [n_seqs, heads * maps * dv]."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(k_pool, "k_pool", torch.bfloat16), _dense(v_pool, "v_pool", torch.bfloat16)
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table")):
        _dense(t, name, torch.int32)
    n, rows, d, dv, n_pages, n_kv, page_size = _masked_shapes(q, k_pool, v_pool, maps)
    heads = rows // maps
    n_splits = n_splits or decode_splits(n, n_kv * maps)
    n_dist = _check_sinks_bias(sinks, dist_bias, rows)
    out = torch.empty((n, rows * dv), dtype=q.dtype, device=q.device)
    part_o = torch.empty((n * rows * n_splits * dv,), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((n * rows * n_splits * 2,), dtype=torch.float32, device=q.device)
    check(l.gi_attention_decode_masked_bf16(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(tok_pos),
                                            _ptr(tok_slot), _ptr(out), _ptr(part_o), _ptr(part_ml), n, heads, n_kv, d, dv,
                                            page_size, block_table.shape[1], n_pages, int(window or 0), int(chunk or 0),
                                            int(maps), float(scale), n_splits, _ptr(sinks), _ptr(dist_bias), n_dist,
                                            _stream()), l)
    counters.launches += 1                                   # the combine kernel
    return out


def tcgen05_attention_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill attention takes this element type, head size and page size."""
    return dtype == torch.bfloat16 and head_dim == 128 and page_size % 64 == 0


def attention_prefill_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                              q_tiles128: torch.Tensor, scale: float, window: int, rows_covered: bool = False,
                              chunk: int = 0, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Flash attention of q [n, n_q, 128] over the paged cache on tcgen05 tensor cores (TMA-fed, S, P and
    P V in tensor memory).  `q_tiles128` int32 [n_tiles, 4] cuts the rows into runs of at most 128
    consecutive tokens of one sequence: {slot, first row, rows, position of the first row}.  `chunk` > 0: a query
    sees only the keys of its own chunk of positions.  `sinks` float32 [n_q]: a score per head that joins the
    softmax's denominator without a value."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(k_pool, "k_pool", torch.bfloat16), _dense(v_pool, "v_pool", torch.bfloat16)
    _dense(block_table, "block_table", torch.int32), _dense(q_tiles128, "q_tiles128", torch.int32)
    n, n_q, d = q.shape
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    if pool_d != d or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not fit head_dim {d}")
    if q_tiles128.dim() != 2 or q_tiles128.shape[1] != 4 or q_tiles128.data_ptr() % 16:
        raise KernelError("q_tiles128 must be int32 [n_tiles, 4] starting on 16 bytes")
    # rows in no tile (padding) stay zero; when the caller says that every row lies in a tile, nothing is filled
    _check_sinks_bias(sinks, None, n_q)
    out = (torch.empty if rows_covered else torch.zeros)((n, n_q * d), dtype=q.dtype, device=q.device)
    check(l.gi_attention_prefill_tcgen05(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(q_tiles128),
                                         q_tiles128.shape[0], _ptr(out), n, n_q, n_kv, d, page_size,
                                         block_table.shape[1], n_pages, int(window or 0), int(chunk or 0), float(scale),
                                         _ptr(tcgen05_error_flag(q.device)), _ptr(sinks), _stream()), l)
    return out


def decode_splits(n_seqs: int, n_kv: int) -> int:
    """Slices of the keys per (sequence, key/value head) in the decode kernel.  Measured on a B200 at
    2,048 and 4,096 cached tokens (8 key/value heads): about 256 CTAs are wanted at small batches (but at
    most 16 slices); three slices are best between 64 and 512 (sequence, head) pairs (batches 16 and 32:
    5 to 12 % better than two), and two slices still pay when the batch alone makes several hundred CTAs,
    because they even out the last wave.  The count is fixed per batch size: a recorded step is replayed
    while the sequences grow."""
    pairs = max(1, n_seqs * n_kv)
    if pairs <= 64:
        return max(1, min(16, -(-256 // pairs)))
    if pairs < 512:
        return 3
    return 2 if pairs < 1776 else 1


def decode_splits_tcgen05(n_seqs: int, n_kv: int) -> int:
    """Slices of the keys per (sequence, key/value head) in the tcgen05 decode kernel.  Measured on a B200 at
    2,048 and 4,096 cached tokens (8 key/value heads): about 256 CTAs at small batches (16 slices at batch 1,
    4 at batch 8, 2 at batch 16) and no slicing from 256 (sequence, head) pairs on (batch 64: 86 us whole
    against 93 us in two slices).  Fixed per batch size: a recorded step is replayed while the sequences grow."""
    return max(1, min(16, -(-256 // max(1, n_seqs * n_kv))))


def tcgen05_decode_takes(dtype: torch.dtype, head_dim: int, page_size: int, group: int) -> bool:
    return dtype == torch.bfloat16 and head_dim == 128 and page_size % 64 == 0 and group <= 16


def attention_decode_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                             tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float, window: int,
                             n_splits: Optional[int] = None) -> torch.Tensor:
    """Split-KV attention for decode steps on TMA and tcgen05: the arguments of `attention_decode_bf16`; heads
    of 128, pages that are a multiple of 64 tokens, at most 16 query heads per key/value head."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(k_pool, "k_pool", torch.bfloat16), _dense(v_pool, "v_pool", torch.bfloat16)
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table")):
        _dense(t, name, torch.int32)
    n, n_q, d = q.shape
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    if pool_d != d or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not fit head_dim {d}")
    if tok_pos.numel() < n or tok_slot.numel() < n:
        raise KernelError("tok_pos / tok_slot are shorter than the token rows")
    n_splits = n_splits or decode_splits_tcgen05(n, n_kv)
    out = torch.empty((n, n_q * d), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((n * n_q * n_splits * d,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * n_q * n_splits * 2,), dtype=torch.float32, device=q.device)
    check(l.gi_attention_decode_tcgen05(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(tok_pos),
                                        _ptr(tok_slot), _ptr(part_o), _ptr(part_ml), _ptr(out), n, n_q, n_kv, d, page_size,
                                        block_table.shape[1], n_pages, int(window or 0), float(scale), n_splits,
                                        _ptr(tcgen05_error_flag(q.device)), _stream()), l)
    if n_splits > 1:                                 # one slice: the kernel wrote the output itself
        check(l.gi_attention_decode_combine(_ptr(part_o), _ptr(part_ml), _ptr(out), n * n_q, d, n_splits, _stream()), l)
    return out


def attention_decode_bf16(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                          tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float, window: int,
                          n_splits: Optional[int] = None) -> torch.Tensor:
    """Split-KV attention for decode steps: q [n_seqs, n_q, d], one token per sequence at position
    tok_pos (the key at that position is already in the cache).  Returns [n_seqs, n_q * d].
    The partial results of the slices go through scratch memory allocated here."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(k_pool, "k_pool", torch.bfloat16), _dense(v_pool, "v_pool", torch.bfloat16)
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table")):
        _dense(t, name, torch.int32)
    n, n_q, d = q.shape
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    if pool_d != d or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not fit head_dim {d}")
    if tok_pos.numel() < n or tok_slot.numel() < n:
        raise KernelError("tok_pos / tok_slot are shorter than the token rows")
    n_splits = n_splits or decode_splits(n, n_kv)
    out = torch.empty((n, n_q * d), dtype=q.dtype, device=q.device)
    part_o = torch.empty((n * n_q * n_splits * d,), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((n * n_q * n_splits * 2,), dtype=torch.float32, device=q.device)
    check(l.gi_attention_decode_bf16(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(tok_pos),
                                     _ptr(tok_slot), _ptr(out), _ptr(part_o), _ptr(part_ml), n, n_q, n_kv, d,
                                     page_size, block_table.shape[1], n_pages, int(window or 0), float(scale),
                                     n_splits, _stream()), l)
    counters.launches += 1                                   # the combine kernel
    return out
