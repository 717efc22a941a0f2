"""Tiny Kenovik configurations for the tests.

They differ from one another in every size: width, vocabulary, query and key/value heads, key and value sizes,
rotated dimensions and their scaling, softmax scale, rows and reach of the distance bias, the query's growth with
the position, channels, blocks and taps of the recurrent block, feed-forwards of both kinds and none, experts in
groups of which all, some or one stay, shared experts with limits of their own, the order of the layers, and which
of them run several times.
"""
from __future__ import annotations

import copy
from pathlib import Path

import torch

from tiny_fivitar import BF16_MEDIAN, judge, row_errors, trace_portions  # noqa: F401  (the same rules of judgement)


def _sink(heads, kv, dim, vdim, dims=None, base=10000.0, factor=None, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5}
    if dims is not None:
        m["rot"] = {"base": base, "dims": dims}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    return {"type": "attention", "mixer": m}


def _bias(heads, kv, dim, vdim, rows, far, temp=None, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5, "bias_max": far,
         "bias_rows": rows}
    if temp is not None:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "attention_2", "mixer": m}


def _rglru(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, limit, experts, top, scale, groups=None, shared=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}
    if shared is not None:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    return mlp


def _with(layer, mlp=None):
    return dict(layer, mlp=mlp)


TINY = {
    # each mechanism alone
    "sink": dict(vocab=300, width=64, eps=1e-5, emb=4.0, seed=41, std=0.1, norm_std=0.1,
                 layers=[_with(_sink(6, 3, 8, 12, dims=6, base=100.0, factor=4.0, scale=0.6))]),
    "bias": dict(vocab=280, width=48, eps=1e-6, emb=2.0, seed=42, std=0.1, norm_std=0.1,
                 layers=[_with(_bias(4, 2, 12, 6, rows=10, far=40, temp=(0.5, 16), scale=0.4))]),
    "rglru": dict(vocab=260, width=40, eps=1e-5, emb=3.0, seed=43, std=0.1, norm_std=0.1,
                  layers=[_with(_rglru(60, 5, 4))]),
    "dense": dict(vocab=270, width=48, eps=1e-5, emb=2.0, seed=44, std=0.1, norm_std=0.1,
                  layers=[_with(_sink(2, 1, 16, 8), _dense(100))]),
    "moe": dict(vocab=280, width=48, eps=1e-5, emb=6.0, seed=45, std=0.1, norm_std=0.1,
                layers=[_with(_rglru(48, 3, 2), _moe(40, 1.2, 12, 3, 1.7, groups=(4, 2), shared=(56, 0.8)))]),
    # everything, in another order than any other configuration's; layers 1 to 3 run three times
    "mix": dict(vocab=411, width=96, eps=2e-6, emb=9.0, seed=46, std=0.06, norm_std=0.15, loop=(1, 4, 3),
                layers=[_with(_rglru(72, 6, 3), _moe(48, 2.0, 8, 2, 2.5, groups=(4, 3))),
                        _with(_bias(6, 3, 8, 12, rows=16, far=100, temp=(0.2, 50)), _dense(128)),
                        _with(_sink(4, 4, 16, 8, dims=16, base=300.0), _moe(32, 0.9, 9, 4, 0.6, groups=(3, 3), shared=(24, 3.0))),
                        _with(_rglru(96, 2, 5)),
                        _with(_sink(3, 1, 24, 16, dims=10, base=5000.0, factor=2.0), _dense(64)),
                        _with(_bias(2, 1, 20, 28, rows=7, far=300), _moe(24, 1.0, 4, 4, 1.0))]),
    # head sizes the tensor-core kernels take (keys twice the values, values twice the keys, equal), a group of
    # more than 16 query heads per key/value head, the first two layers twice
    "tc": dict(vocab=300, width=128, eps=1e-5, emb=3.0, seed=47, std=0.05, norm_std=0.1, loop=(0, 2, 2),
               layers=[_with(_sink(6, 2, 32, 64, dims=16, base=1000.0, factor=3.0), _dense(96)),
                       _with(_bias(4, 1, 64, 64, rows=24, far=150, temp=(0.3, 64)), _moe(32, 2.0, 16, 3, 1.5, groups=(8, 3), shared=(64, 1.0))),
                       _with(_sink(2, 2, 128, 128, dims=128, base=50000.0)),
                       _with(_bias(34, 2, 16, 16, rows=12, far=70), _dense(64)),
                       _with(_bias(3, 3, 32, 16, rows=32, far=500, temp=(1.0, 7)))]),
    # prompts of a thousand tokens on pages of 64: every attention on its tensor-core kernels (flash on tcgen05 for the
    # heads of 128, mma.sync for the others), distances far beyond the bias tables' reach, three layers passed twice
    "long": dict(vocab=384, width=192, eps=1e-5, emb=2.0, seed=50, std=0.06, norm_std=0.1, loop=(1, 4, 2),
                 layers=[_with(_rglru(240, 4, 3), _moe(48, 1.5, 12, 4, 1.8, groups=(3, 2), shared=(80, 2.5))),
                         _with(_sink(6, 3, 32, 64, dims=16, base=250000.0, factor=2.0), _dense(256)),
                         _with(_bias(4, 2, 64, 64, rows=20, far=300, temp=(0.25, 128)), _moe(40, 1.0, 8, 2, 2.2, groups=(4, 3))),
                         _with(_bias(5, 1, 48, 24, rows=32, far=900), _dense(160)),
                         _with(_sink(2, 1, 128, 128, dims=64, base=10000.0), _moe(32, 3.0, 6, 3, 1.0, shared=(64, 1.0)))]),
    # sizes that are multiples of nothing the kernels like
    "odd": dict(vocab=263, width=50, eps=1e-5, emb=2.5, seed=48, std=0.1, norm_std=0.1, loop=(1, 2, 2),
                layers=[_with(_sink(3, 3, 6, 10, dims=2, base=40.0, factor=1.5), _moe(18, 1.5, 6, 2, 1.3, groups=(2, 1))),
                        _with(_rglru(33, 3, 3), _dense(30)),
                        _with(_bias(5, 1, 10, 6, rows=9, far=21, temp=(0.1, 3)))]),
    # ones everywhere: one head, one block, one tap, one expert of one in one group, one bucket row beyond the
    # first, a loop of one pass, no rotation
    "ones": dict(vocab=257, width=48, eps=1e-5, emb=1.0, seed=49, std=0.1, norm_std=0.2, loop=(0, 1, 1),
                 layers=[_with(_rglru(48, 1, 1), _moe(24, 5.0, 1, 1, 1.0, groups=(1, 1))),
                         _with(_sink(1, 1, 8, 8), _dense(48)),
                         _with(_bias(1, 1, 8, 8, rows=2, far=2, temp=(0.3, 1)))]),
}


def config_dict(name: str) -> dict:
    t = TINY[name]
    out = {"architecture": "Kenovik", "vocab": t["vocab"], "width": t["width"], "embedding": {"scale": t["emb"]},
           "norm": {"eps": t["eps"]}, "layers": copy.deepcopy(t["layers"])}
    if "loop" in t:
        out["loop"] = dict(zip(("start", "stop", "times"), t["loop"]))
    return out


def make_config(name: str):
    from garlic_inference_b200.config import KenovikConfig
    return KenovikConfig.from_dict(config_dict(name))


def write_model(name: str, folder) -> Path:
    from garlic_inference_b200 import write_random_model
    t = TINY[name]
    return write_random_model(folder, make_config(name), seed=t["seed"], std=t["std"], norm_std=t["norm_std"])


def plain_logits(model_dir, requests, dtype=torch.float32) -> dict:
    import plain_kenovik as plain
    cfg, weights = plain.read_model_dir(model_dir)
    return {rid: plain.forward(cfg, weights, toks, dtype).to(torch.float64).numpy() for rid, toks in requests.items()}


def plain_pair(model_dir, requests):
    """(float64 logits, float32 logits) of the plain model for every request."""
    return plain_logits(model_dir, requests, torch.float64), plain_logits(model_dir, requests, torch.float32)


# ---- routing that rests on a close call ---------------------------------------------------------------------------
# A router's choice is a step function of its scores: where two groups' scores or the last chosen and the first
# unchosen expert's scores lie closer than bfloat16 arithmetic resolves, the bfloat16 engine may choose otherwise
# than the float64 yardstick, and that row (and, through recurrent state and cached keys, the next few) is then far
# off without any fault.  `close_calls` finds those positions in the plain model; `judge_routed` lets a bfloat16 row
# pass the worst-row bound only if such a position lies at most CLOSE_REACH tokens before it, and only a few rows.
CLOSE_MARGIN, CLOSE_REACH, CLOSE_SHARE = 0.02, 4, 0.02


def close_calls(model_dir, requests) -> dict:
    """{request: positions at which some routed layer's choice of groups or experts has a margin below CLOSE_MARGIN}."""
    import plain_kenovik as plain
    cfg, weights = plain.read_model_dir(model_dir)
    saved, found = plain.route, {}
    current = []

    def spy(h, W, r):
        idx, w = saved(h, W, r)
        s = torch.sigmoid(h @ W["router"].T) + W["correction"]
        T, E = s.shape
        g = r.get("groups") or {"count": 1, "keep": 1}
        per = E // g["count"]
        margin = torch.full((T,), 9.0, dtype=s.dtype)
        allowed = s
        if g["count"] > g["keep"]:
            sums = s.reshape(T, g["count"], per).topk(min(2, per), -1).values.sum(-1)
            ranked = sums.sort(-1, descending=True).values
            margin = torch.minimum(margin, ranked[:, g["keep"] - 1] - ranked[:, g["keep"]])
            kept = torch.zeros(T, g["count"], dtype=torch.bool).scatter_(1, sums.topk(g["keep"], -1).indices, True)
            allowed = torch.where(kept[:, :, None].expand(T, g["count"], per).reshape(T, E), s, torch.full_like(s, -1e9))
        ranked = allowed.sort(-1, descending=True).values
        if r["top"] < E:
            gap = ranked[:, r["top"] - 1] - ranked[:, r["top"]]
            margin = torch.minimum(margin, torch.where(ranked[:, r["top"]] > -1e8, gap, torch.full_like(gap, 9.0)))
        current.extend(int(p) for p in torch.nonzero(margin < CLOSE_MARGIN).flatten())
        return idx, w

    plain.route = spy
    try:
        for rid, toks in requests.items():
            current.clear()
            plain.forward(cfg, weights, toks, torch.float64)
            found[rid] = set(current)
    finally:
        plain.route = saved
    return found


def judge_routed(got, want64, plain32, dtype: str, what: str, model_dir, requests) -> float:
    """`judge`, except that in bfloat16 a few rows right behind a routing close call may miss the worst-row bound."""
    if dtype == "bfloat16":
        from tiny_fivitar import BF16_WORST
        errs = row_errors(got, want64)
        over = [k for k, e in errs.items() if e[1] > BF16_WORST]
        if over:
            close = close_calls(model_dir, requests)
            unexplained = [(rid, p) for rid, p in over if not any(p - k in close[rid] for k in range(CLOSE_REACH + 1))]
            assert not unexplained, f"{what}: rows {unexplained[:5]} are far off and no routing close call is near them"
            assert len(over) <= max(1, CLOSE_SHARE * len(errs)), f"{what}: {len(over)} of {len(errs)} rows are far off"
            got = {rid: {p: row for p, row in rows.items() if (rid, p) not in over} for rid, rows in got.items()}
    return judge(got, want64, plain32, dtype, what)
