"""Tiny Dugopel configurations for the tests.

They differ from one another in every size: width, vocabulary, heads, unrotated and rotated query/key sizes, value
size, the two latents' ranks, rotation over all or a part of the rotated part, softmax scale, feed-forwards of
both kinds and none, limits, experts in groups of which all, some or one stay, weights with and without a factor,
the order of the layers, and layers that read another layer's cached rows.
"""
from __future__ import annotations

import copy
from pathlib import Path

import torch

from tiny_fivitar import BF16_MEDIAN, judge, row_errors, trace_portions  # noqa: F401  (the same rules of judgement)


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, dims=None, base=10000.0, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}, "scale": scale or (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(ff, limit, experts, top, groups, keep, scale):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}


def _with(layer, mlp=None):
    return dict(layer, mlp=mlp)


TINY = {
    # each mechanism alone
    "latent": dict(vocab=300, width=64, eps=1e-5, emb=4.0, cap=30.0, seed=31, std=0.08, norm_std=0.1,
                   layers=[_with(_latent(3, 16, 8, 24, 40, 32, base=100.0, scale=0.5))]),
    "dense": dict(vocab=280, width=48, eps=1e-6, emb=2.0, cap=8.0, seed=32, std=0.1, norm_std=0.1,
                  layers=[_with(_latent(2, 8, 4, 8, 16, 24), _dense(100, 0.7))]),
    "moe": dict(vocab=280, width=48, eps=1e-5, emb=6.0, cap=20.0, seed=33, std=0.1, norm_std=0.1,
                layers=[_with(_latent(2, 8, 8, 16, 24, 16), _moe(40, 1.2, 6, 3, 3, 2, 1.7))]),
    # everything, in another order than any other configuration's; layers on an earlier layer's cached rows, among
    # them a chain of readers of two different sources; a rotation of a part of the rotated part
    "mix": dict(vocab=411, width=96, eps=2e-6, emb=9.0, cap=12.0, seed=34, std=0.06, norm_std=0.15,
                layers=[_with(_latent(4, 16, 8, 24, 48, 40, base=5000.0), _moe(48, 2.0, 8, 3, 4, 2, 2.5)),
                        _with(_latent(6, 24, 16, 16, 32, 56, dims=12, base=300.0), _dense(128, 1.5)),
                        _with(_latent(2, 32, 8, 40, 48, 24, base=5000.0, kv_from=0), _dense(64, 3.0)),
                        _with(_latent(3, 8, 16, 8, 32, 16, dims=12, base=300.0, kv_from=1)),
                        _with(_latent(5, 16, 8, 16, 48, 64, base=5000.0, kv_from=0), _moe(32, 0.9, 9, 4, 3, 3, 0.6)),
                        _with(_latent(4, 16, 4, 24, 24, 32), _moe(24, 1.0, 4, 4, 1, 1, 1.0))]),
    # many heads (more than one group of the decode kernel's heads), a latent wider than a head
    "wide": dict(vocab=300, width=128, eps=1e-5, emb=3.0, cap=15.0, seed=35, std=0.05, norm_std=0.1,
                 layers=[_with(_latent(36, 16, 8, 16, 64, 48, scale=0.3), _dense(96, 2.0)),
                         _with(_latent(36, 16, 8, 16, 64, 48, scale=0.3, kv_from=0), _moe(32, 2.0, 16, 3, 8, 3, 1.5))]),
    # sizes that are multiples of nothing the kernels like: rows of 50, 14, 10 and 6 elements, three heads
    "odd": dict(vocab=263, width=50, eps=1e-5, emb=2.5, cap=25.0, seed=37, std=0.1, norm_std=0.1,
                layers=[_with(_latent(3, 6, 6, 10, 14, 10, base=40.0), _moe(18, 1.5, 6, 2, 2, 1, 1.3)),
                        _with(_latent(3, 10, 6, 6, 14, 22, base=40.0, kv_from=0), _dense(30, 2.5))]),
    # one head, a rotated part of one pair, latents of 8, one expert of one in one group, a second layer on the first's rows
    "ones": dict(vocab=257, width=48, eps=1e-5, emb=1.0, cap=50.0, seed=36, std=0.1, norm_std=0.2,
                 layers=[_with(_latent(1, 8, 2, 8, 8, 8), _moe(24, 5.0, 1, 1, 1, 1, 1.0)),
                         _with(_latent(1, 16, 2, 8, 8, 16, kv_from=0), _dense(48, 0.3)),
                         _with(_latent(2, 8, 6, 24, 16, 8, dims=0))]),
}


def config_dict(name: str) -> dict:
    t = TINY[name]
    return {"architecture": "Dugopel", "vocab": t["vocab"], "width": t["width"], "embedding": {"scale": t["emb"]},
            "norm": {"eps": t["eps"]}, "logit_softcap": t["cap"], "layers": copy.deepcopy(t["layers"])}


def make_config(name: str):
    from garlic_inference_b200.config import DugopelConfig
    return DugopelConfig.from_dict(config_dict(name))


def write_model(name: str, folder) -> Path:
    from garlic_inference_b200 import write_random_model
    t = TINY[name]
    return write_random_model(folder, make_config(name), seed=t["seed"], std=t["std"], norm_std=t["norm_std"])


def plain_logits(model_dir, requests, dtype=torch.float32) -> dict:
    import plain_dugopel as plain
    cfg, weights = plain.read_model_dir(model_dir)
    return {rid: plain.forward(cfg, weights, toks, dtype).to(torch.float64).numpy() for rid, toks in requests.items()}


def plain_pair(model_dir, requests):
    """(float64 logits, float32 logits) of the plain model for every request."""
    return plain_logits(model_dir, requests, torch.float64), plain_logits(model_dir, requests, torch.float32)
