"""Dugopel on the CPU: its configuration, plan and tensors, and the plain implementation against closed forms."""
import json
import math
import warnings

import pytest
import torch

import plain_dugopel as plain
import tiny_dugopel as td


def test_registry_reads_the_architecture_string_and_round_trips(tmp_path):
    from garlic_inference_b200 import load_config
    from garlic_inference_b200.config import DugopelConfig, known_architectures
    assert "Dugopel" in known_architectures()
    (tmp_path / "config.json").write_text(json.dumps(td.config_dict("mix")))
    cfg = load_config(tmp_path)
    assert type(cfg) is DugopelConfig and cfg.width == 96 and cfg.vocab == 411 and cfg.embedding_scale == 9.0
    assert cfg.logit_softcap == 12.0
    assert DugopelConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict() == td.config_dict("mix")
    bare = td.config_dict("latent")
    del bare["logit_softcap"]
    assert "softcap" not in DugopelConfig.from_dict(bare).plan().head.params


def test_plan_tensors_and_borrowed_rows():
    from garlic_inference_b200.engine.model import wanted_tensors
    plan = td.make_config("mix").plan()
    assert [(e.layer, e.cache, e.kv_cache) for e in plan.schedule] == [(0, 0, None), (1, 1, None), (2, 2, 0), (3, 3, 1),
                                                                      (4, 4, 0), (5, 5, None)]
    assert all(layer.block == "parallel_residual" and list(layer.norms) == ["input"] for layer in plan.layers)
    names = wanted_tensors(plan)
    shape = lambda n: tuple(names[n].shape)
    assert shape("l0.mix.dq") == (40, 96) and shape("l0.mix.dq.norm") == (40,) and shape("l0.mix.uq") == (4 * (16 + 8), 40)
    assert shape("l0.mix.dkv") == (48 + 8, 96) and shape("l0.mix.dkv.norm") == (48,)
    assert shape("l0.mix.uk") == (4 * 16, 48) and shape("l0.mix.uv") == (4 * 24, 48)
    assert shape("l0.mix.g") == (4, 96) and shape("l0.mix.o") == (96, 4 * 24) and shape("l0.norm1") == (96,)
    assert "l2.mix.dkv" not in names and "l2.mix.dkv.norm" not in names and shape("l2.mix.uk") == (2 * 32, 48)
    assert shape("l2.mix.uq") == (2 * (32 + 8), 24) and shape("l3.mix.uv") == (3 * 8, 32)
    assert not any(n.startswith("l3.mlp.") for n in names) and "l3.norm2" not in names
    assert shape("l0.mlp.router") == (8, 96) and shape("l0.mlp.e7.gate") == (48, 96) and shape("l0.mlp.e0.down") == (96, 48)
    assert shape("l1.mlp.gate") == (128, 96) and shape("l1.mlp.down") == (96, 128)
    assert shape("final.norm") == (96,) and shape("head") == (411, 96) and shape("embed") == (411, 96)
    assert len(plan.positions) == 3, "three sets of rotary constants, three parts"
    moe = plan.layers[4].feed_forward.params
    assert (moe["groups"], moe["groups_kept"], moe["top"], moe["weight_scale"], moe["gate_max"]) == (3, 3, 4, 0.6, 0.9)
    assert plan.layers[1].feed_forward.params["up_limit"] == 1.5 and plan.layers[1].feed_forward.params["up_shift"] == 1.0
    assert plan.head.params["softcap"] == 12.0 and plan.embedding.params["scale"] == 9.0


def test_refusals_and_warnings():
    from garlic_inference_b200.config import ConfigError, DugopelConfig
    bad = td.config_dict("ones")
    bad["layers"][0] = dict(bad["layers"][0], type="convolution")
    with pytest.raises(ConfigError, match="convolution"):
        DugopelConfig.from_dict(bad)
    bad = td.config_dict("mix")
    bad["layers"][3]["mixer"]["kv_from"] = 2                       # layer 2 borrows its rows itself
    with pytest.raises(ConfigError, match="kv_from"):
        DugopelConfig.from_dict(bad)
    bad = td.config_dict("mix")
    bad["layers"][2]["mixer"]["kv_from"] = 2                       # not an earlier layer
    with pytest.raises(ConfigError, match="kv_from"):
        DugopelConfig.from_dict(bad)
    bad = td.config_dict("mix")
    bad["layers"][2]["mixer"]["kv_rank"] = 40
    with pytest.raises(ConfigError, match="differ"):
        DugopelConfig.from_dict(bad)
    bad = td.config_dict("moe")
    bad["layers"][0]["mlp"]["router"]["top"] = 5                   # two groups of two experts stay
    with pytest.raises(ConfigError, match="top"):
        DugopelConfig.from_dict(bad)
    bad = td.config_dict("moe")
    bad["layers"][0]["mlp"]["router"]["groups"]["count"] = 4      # six experts in four groups
    with pytest.raises(ConfigError, match="groups"):
        DugopelConfig.from_dict(bad)
    bad = td.config_dict("dense")
    bad["layers"][0]["mlp"] = {"kind": "sparse", "ff": 8}
    with pytest.raises(ConfigError, match="sparse"):
        DugopelConfig.from_dict(bad)
    bad = td.config_dict("dense")
    del bad["layers"][0]["mlp"]["limit"]
    with pytest.raises(ConfigError, match="limit"):
        DugopelConfig.from_dict(bad)
    odd = td.config_dict("dense")
    odd["layers"][0]["mixer"]["window"] = 7
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        DugopelConfig.from_dict(odd)
    assert any("window" in str(w.message) for w in seen)


def test_random_folder_loads_and_fits(tmp_path):
    from garlic_inference_b200.engine.model import wanted_tensors
    from garlic_inference_b200.weights import Checkpoint
    d = td.write_model("ones", tmp_path / "ones")
    Checkpoint(d).check(wanted_tensors(td.make_config("ones").plan()))
    cfg, w = plain.read_model_dir(d)
    assert cfg == td.config_dict("ones") and w["l0.mix.dkv"].shape == (10, 48) and "l1.mix.dkv" not in w
    logits = plain.forward(cfg, w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 257) and torch.isfinite(logits).all() and float(logits.abs().max()) < 50.0


# ---- the plain functions against closed forms ----------------------------------------------------
def test_plain_norms_and_the_gated_unit():
    x = torch.tensor([[1.0, 3.0, 5.0, 7.0]])
    got = plain.layer_norm(x, torch.tensor([1.0, 2.0, 1.0, 0.5]), 0.0)
    s = math.sqrt(5.0)                                           # deviations -3 -1 1 3: variance 5
    assert torch.allclose(got, torch.tensor([[-3 / s, -2 / s, 1 / s, 1.5 / s]]), atol=1e-6)
    assert torch.allclose(plain.layer_norm(x + 100.0, torch.ones(4), 0.0), plain.layer_norm(x, torch.ones(4), 0.0), atol=1e-5)
    got = plain.rms_norm(torch.tensor([[3.0, 4.0]]), torch.tensor([2.0, 1.0]), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(got, torch.tensor([[6.0 / r, 4.0 / r]]), atol=1e-6)
    eye = torch.eye(3)
    h = torch.tensor([[5.0, -5.0, 0.5]])
    # gate 5 -> 2, up 5 -> 2 (+1); gate -5 stays, up -5 -> -2 (+1); inside the limits nothing is cut
    want = [2.0 * plain.sigmoid(torch.tensor(1.702 * 2.0)) * 3.0, -5.0 * plain.sigmoid(torch.tensor(1.702 * -5.0)) * -1.0,
            0.5 * plain.sigmoid(torch.tensor(1.702 * 0.5)) * 1.5]
    assert torch.allclose(plain.swish_glu(h, eye, eye, eye, 2.0), torch.tensor([want]), atol=1e-6)


def test_plain_rotation_of_halves():
    x = torch.zeros(3, 1, 6)
    x[:, 0, 0] = 1.0                                             # pair (0, 2) of four turned dimensions
    x[:, 0, 1] = 1.0                                             # pair (1, 3)
    x[:, 0, 5] = 7.0
    y = plain.turn_halves(x, 4, 100.0)
    for p in range(3):
        assert torch.allclose(y[p, 0, [0, 2]], torch.tensor([math.cos(p), math.sin(p)]), atol=1e-6)
        assert torch.allclose(y[p, 0, [1, 3]], torch.tensor([math.cos(p * 0.1), math.sin(p * 0.1)]), atol=1e-6)
        assert y[p, 0, 4] == 0.0 and y[p, 0, 5] == 7.0, "dimensions beyond the turned ones pass"
    later = plain.turn_halves(x[:1], 4, 100.0, first_pos=2)
    assert torch.allclose(later[0], y[2])


def test_plain_router_groups_and_weights():
    # six experts in three groups of two; scores fall as 2 0 4 1 3 5 (expert 2 the best); the best groups are
    # {2,3} and {0,1}: expert 4, third by its score, sits in a group that does not stay
    z = torch.log(torch.tensor([[0.25, 0.05, 0.3, 0.02, 0.2, 0.18]]))
    router = {"experts": 6, "top": 3, "scale": 2.0, "groups": {"count": 3, "keep": 2}}
    idx, w = plain.route(z, router)
    assert idx.tolist() == [[2, 0, 1]] and torch.allclose(w, torch.tensor([[0.6, 0.5, 0.1]]), atol=1e-6)
    idx, w = plain.route(z, dict(router, groups={"count": 3, "keep": 3}))
    assert idx.tolist() == [[2, 0, 4]] and torch.allclose(w.sum(), torch.tensor(1.5), atol=1e-6), "no renormalisation"
    idx, w = plain.route(z, dict(router, top=1, groups={"count": 1, "keep": 1}))
    assert idx.tolist() == [[2]]


def test_plain_attention_reads_the_latent_and_the_shared_part():
    """One head with hand-made weights: equal scores give the mean of the values seen; a large rotated part makes
    the score follow the angle between positions."""
    torch.manual_seed(0)
    T, width = 6, 8
    m = {"heads": 1, "dim": 2, "rot_dim": 2, "vdim": 3, "kv_rank": 4, "q_rank": 4, "scale": 1.0, "rot": {"base": 10.0, "dims": 2}}
    w = {"dq": torch.randn(4, width), "dq.norm": torch.ones(4), "uq": torch.zeros(4, 4), "dkv": torch.randn(6, width),
         "dkv.norm": torch.ones(4), "uk": torch.randn(2, 4), "uv": torch.randn(3, 4), "g": torch.zeros(1, width),
         "o": torch.eye(width)[:, :3].contiguous()}
    h = torch.randn(T, width)
    shared = {}
    y = plain.latent_attention(h, w, m, 1e-6, shared, 0)       # zero queries: every visible key weighs the same
    c, kr = shared[0]
    v = c @ w["uv"].T
    means = torch.stack([v[:t + 1].mean(0) for t in range(T)]) * 0.5      # gate sigmoid(0)
    assert torch.allclose(y[:, :3], means, atol=1e-5) and float(y[:, 3:].abs().max()) == 0.0
    assert torch.allclose((c * c).mean(-1), torch.ones(T), atol=1e-4), "the cached latent is normed"
    assert torch.allclose((kr * kr).sum(-1), ((h @ w["dkv"].T)[:, 4:] ** 2).sum(-1), atol=1e-4), "a turn keeps the length"
    # a second layer on these rows sees the same c and kr whatever its own input is
    m2 = dict(m, kv_from=0)
    w2 = {k: t for k, t in w.items() if not k.startswith("dkv")}
    y2 = plain.latent_attention(torch.randn(T, width), w2, m2, 1e-6, shared, 1)
    assert torch.allclose(y2[:, :3] / 0.5, means / 0.5, atol=1e-5) and shared[1][0] is shared[0][0]


def test_what_the_comparisons_rest_on_shows_in_the_plain_model(tmp_path):
    """Dropping the cached rows before a cut, turning pairs instead of halves, leaving out the gate, the groups or
    the borrowed rows changes the plain logits by far more than any tolerance used against it."""
    d = td.write_model("mix", tmp_path / "mix")
    cfg, w = plain.read_model_dir(d)
    toks = torch.randint(0, 411, (80,), generator=torch.Generator().manual_seed(1)).tolist()
    want = plain.forward(cfg, w, toks)
    scale = float(want.abs().max())
    far = lambda other: float((other - want[-other.shape[0]:]).abs().max()) / scale
    assert far(plain.forward(cfg, w, toks[40:])) > 1e-2
    own = json.loads(json.dumps(cfg))
    own["layers"][4]["mixer"]["kv_from"] = 1                       # another layer's rows (of the wrong width: refuse by shape)
    with pytest.raises(RuntimeError):
        plain.forward(own, w, toks)
    moved = json.loads(json.dumps(cfg))
    moved["layers"][0]["mlp"]["router"]["groups"]["keep"] = 4
    assert far(plain.forward(moved, w, toks)) > 1e-3
    moved = json.loads(json.dumps(cfg))
    moved["layers"][1]["mixer"]["rot"]["dims"] = 16
    assert far(plain.forward(moved, w, toks)) > 1e-3
    no_gate = dict(w, **{"l0.mix.g": torch.zeros_like(w["l0.mix.g"])})
    assert far(plain.forward(cfg, no_gate, toks)) > 1e-3
    no_cap = dict(cfg, logit_softcap=None)
    assert far(plain.forward(no_cap, w, toks)) > 1e-4
