"""Kenovik on the CPU: its configuration, plan and tensors, and the plain implementation against closed forms."""
import json
import math

import pytest
import torch

import plain_kenovik as plain
import tiny_kenovik as tk


def test_registry_reads_the_architecture_string_and_round_trips(tmp_path):
    from garlic_inference_b200 import load_config
    from garlic_inference_b200.config import KenovikConfig, known_architectures
    assert "Kenovik" in known_architectures()
    (tmp_path / "config.json").write_text(json.dumps(tk.config_dict("mix")))
    cfg = load_config(tmp_path)
    assert type(cfg) is KenovikConfig and cfg.width == 96 and cfg.vocab == 411 and cfg.embedding_scale == 9.0
    assert cfg.loop == {"start": 1, "stop": 4, "times": 3}
    assert KenovikConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.to_dict()["layers"][5]["mlp"]["router"]["groups"] == {"count": 1, "keep": 1}, "no groups: one group of all"
    assert tk.make_config("tc").to_dict() == tk.config_dict("tc")
    assert KenovikConfig.from_dict(tk.config_dict("sink")).loop is None


def test_plan_schedule_and_tensors():
    from garlic_inference_b200.engine.model import wanted_tensors
    cfg = tk.make_config("mix")
    plan = cfg.plan()
    # layers 1..3 three times, each run with a cache entry of its own; the first layer of each pass takes a row of
    # `loop.step` along
    assert [(e.layer, e.cache, e.offset) for e in plan.schedule] == \
        [(0, 0, None)] + [(i, 1 + 3 * t + (i - 1), ("loop.step", t) if i == 1 else None) for t in range(3) for i in (1, 2, 3)] + \
        [(4, 10, None), (5, 11, None)]
    assert plan.n_cache_entries() == 12 and list(plan.offsets) == ["loop.step"]
    assert [(i, t) for i, t in cfg.layer_runs()] == plain.layer_order(tk.config_dict("mix"))
    assert all(layer.block == "pre_norm_residual" for layer in plan.layers)
    assert list(plan.layers[3].norms) == ["input"] and plan.layers[3].feed_forward is None
    names = wanted_tensors(plan)
    shape = lambda n: tuple(names[n].shape)
    assert shape("loop.step") == (3, 96) and shape("embed") == (411, 96) and "head" not in names
    assert plan.head.weights == {"weight": "embed"}
    assert shape("l0.mix.y") == (72, 96) and shape("l0.mix.x.b") == (72,) and shape("l0.mix.conv") == (72, 3)
    assert shape("l0.mix.ra") == (6, 12, 12) and shape("l0.mix.ri.b") == (6, 12) and shape("l0.mix.lam") == (72,)
    assert shape("l0.mix.o") == (96, 72)
    assert shape("l1.mix.q") == (48, 96) and shape("l1.mix.k") == (24, 96) and shape("l1.mix.v") == (36, 96)
    assert shape("l1.mix.q.norm") == (48,) and shape("l1.mix.k.norm") == (24,) and shape("l1.mix.rel") == (16, 6)
    assert "l1.mix.q.b" not in names and shape("l1.mix.o") == (96, 72)
    assert shape("l2.mix.q.b") == (64,) and shape("l2.mix.k.b") == (64,) and shape("l2.mix.v.b") == (32,)
    assert "l2.mix.rel" not in names and "l2.mix.q.norm" not in names
    assert not any(n.startswith("l3.mlp.") for n in names) and "l3.norm2" not in names and "l3.norm1" in names
    assert shape("l0.mlp.router") == (8, 96) and shape("l0.mlp.correction") == (8,) and shape("l0.mlp.e7.gate") == (48, 96)
    assert "l0.mlp.shared.gate" not in names and shape("l2.mlp.shared.gate") == (24, 96) and shape("l2.mlp.shared.down") == (96, 24)
    assert shape("l1.mlp.gate") == (128, 96) and shape("final.norm") == (96,)
    assert len(plan.positions) == 2, "two sets of rotary constants, two parts"
    rot = next(p for k, p in plan.positions.items() if "5000" in k).params
    assert rot["layout"] == "interleaved" and rot["rotary_dim"] == 10 and rot["linear_factor"] == 2.0 and rot["tables"] is False
    moe = plan.layers[2].feed_forward.params
    assert (moe["scores"], moe["group_score"], moe["normalize"], moe["correction"]) == ("sigmoid", "top2_sum", True, True)
    assert (moe["groups"], moe["groups_kept"], moe["top"], moe["weight_scale"], moe["gate_max"]) == (3, 3, 4, 0.6, 0.9)
    assert moe["shared"]["size"] == 24 and moe["shared"]["up_limit"] == 3.0 and moe["up_shift"] == 1.0 and moe["swish_alpha"] == 1.702
    free = plan.layers[5].feed_forward.params                      # no groups in the file: one group of all
    assert (free["groups"], free["groups_kept"]) == (1, 1) and "shared" not in free
    att = plan.layers[2].mixer.params
    assert att["sink"] == 0.0 and att["qkv_bias"] is True and "distance_bias" not in att
    att2 = plan.layers[1].mixer.params
    assert att2["distance_bias"] == {"rows": 16, "max_distance": 100} and att2["query_temperature"] == {"coef": 0.2, "every": 50}
    assert att2["projection_norm_eps"] == 2e-6 and "sink" not in att2 and "query_temperature" not in plan.layers[5].mixer.params
    assert plan.layers[0].mixer.params["decay_scale"] == 8.0 and plan.embedding.params["scale"] == 9.0
    # a loop of one pass still has its vector; no loop, no table
    ones = tk.make_config("ones").plan()
    assert [e.offset for e in ones.schedule] == [("loop.step", 0), None, None]
    assert not tk.make_config("sink").plan().offsets


def test_rows_of_the_bias_table_come_from_the_tensor():
    cfg = tk.config_dict("bias")
    del cfg["layers"][0]["mixer"]["bias_rows"]
    from garlic_inference_b200.config import KenovikConfig
    bare = KenovikConfig.from_dict(cfg)
    assert bare.plan().layers[0].mixer.params["distance_bias"]["rows"] == 32          # this library's own default
    sized = bare.with_shapes({"l0.mix.rel": (10, 4), "l0.mix.q": (48, 48)})
    assert sized.plan().layers[0].mixer.params["distance_bias"]["rows"] == 10


def test_refusals_and_warnings():
    from garlic_inference_b200.config import ConfigError, KenovikConfig
    bad = tk.config_dict("ones")
    bad["layers"][0] = dict(bad["layers"][0], type="convolution")
    with pytest.raises(ConfigError, match="convolution"):
        KenovikConfig.from_dict(bad)
    bad = tk.config_dict("mix")
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError, match="loop"):
        KenovikConfig.from_dict(bad)
    bad = tk.config_dict("moe")
    bad["layers"][0]["mlp"]["router"]["top"] = 7                   # 2 groups of 3 stay
    with pytest.raises(ConfigError, match="top 7"):
        KenovikConfig.from_dict(bad)
    bad = tk.config_dict("bias")
    bad["layers"][0]["mixer"]["bias_max"] = 5                      # not beyond half of the 10 rows
    with pytest.raises(ConfigError, match="bias_max"):
        KenovikConfig.from_dict(bad)
    bad = tk.config_dict("rglru")
    bad["layers"][0]["mixer"]["blocks"] = 7
    with pytest.raises(ConfigError, match="blocks"):
        KenovikConfig.from_dict(bad)
    bad = tk.config_dict("dense")
    bad["layers"][0]["mlp"]["kind"] = "conv"
    with pytest.raises(ConfigError, match="conv"):
        KenovikConfig.from_dict(bad)
    odd = tk.config_dict("sink")
    odd["layers"][0]["mixer"]["window"] = 5
    with pytest.warns(UserWarning, match="window"):
        KenovikConfig.from_dict(odd)


def test_distance_buckets_of_the_mixer_and_of_the_plain_model_agree():
    from garlic_inference_b200.parts import MaskedAttention
    for rows, far in ((10, 40), (16, 100), (7, 300), (2, 2), (12, 90), (24, 150), (32, 500), (9, 21), (1, 5), (6, 1000)):
        got = MaskedAttention.distance_buckets(rows, far).tolist()
        assert got == [plain.distance_bucket(n, rows, far) if rows > 1 else 0 for n in range(far + 1)], (rows, far)
        assert got[-1] == rows - 1 and sorted(got) == got, "the last row from `far` on, rows in rising order"
    b = [plain.distance_bucket(n, 8, 64) for n in range(70)]
    assert b[:4] == [0, 1, 2, 3] and b[4] == 4 and b[7] == 4 and b[8] == 5 and b[15] == 5 and b[16] == 6 and b[63] == 7 and b[69] == 7


def test_plain_functions_against_closed_forms():
    torch.manual_seed(0)
    # one key: the sink halves the weight of a key whose score is 0
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 1.0}
    W = {"q": torch.zeros(4, 5), "k": torch.zeros(4, 5), "v": torch.zeros(3, 5), "q.b": torch.zeros(4), "k.b": torch.zeros(4),
         "v.b": torch.tensor([2.0, 4.0, 6.0]), "o": torch.eye(3)}
    out = plain.attention_sink(torch.randn(3, 5), W, m, torch.arange(3))
    torch.testing.assert_close(out[0], torch.tensor([1.0, 2.0, 3.0]))                    # 1 key and the sink
    torch.testing.assert_close(out[2], torch.tensor([1.5, 3.0, 4.5]))                    # 3 keys and the sink
    # rotation: a pair at position p turns by p f / factor, the rest passes
    x = torch.tensor([[[1.0, 0.0, 0.0, 1.0, 5.0, 7.0]]]).repeat(3, 1, 1)
    r = plain.rotate_pairs(x, torch.arange(3), 4, 100.0, 2.0)
    a0, a1 = 2 * 1.0 / 2.0, 2 * 100.0 ** -0.5 / 2.0
    torch.testing.assert_close(r[2, 0], torch.tensor([math.cos(a0), math.sin(a0), -math.sin(a1), math.cos(a1), 5.0, 7.0]))
    # the query's factor
    t = plain.query_temperature(torch.tensor([0, 2, 3, 7, 8]), 0.5, 4, torch.float64)
    torch.testing.assert_close(t, torch.tensor([1.0, 1.0, 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(3), 1 + 0.5 * math.log(3)], dtype=torch.float64))
    # the recurrence: constant gates give a geometric series
    Wd, T = 4, 6
    Wr = {"y": torch.zeros(Wd, 2), "y.b": torch.full((Wd,), 3.0), "x": torch.zeros(Wd, 2), "x.b": torch.ones(Wd),
          "conv": torch.tensor([[0.0, 1.0]]).repeat(Wd, 1), "conv.b": torch.zeros(Wd), "ra": torch.zeros(2, 2, 2),
          "ra.b": torch.zeros(2, 2), "ri": torch.zeros(2, 2, 2), "ri.b": torch.full((2, 2), 50.0), "lam": torch.zeros(Wd),
          "o": torch.eye(Wd)}
    out = plain.rglru(torch.randn(T, 2).double(), {k: v.double() for k, v in Wr.items()}, {"width": Wd, "blocks": 2, "conv": 2})
    a = math.exp(-8 * 0.5 * math.log(2))
    S, want = 0.0, []
    for _ in range(T):
        S = a * S + math.sqrt(1 - a * a)
        want.append(S * float(plain.gelu_tanh(torch.tensor(3.0, dtype=torch.float64))))
    torch.testing.assert_close(out[:, 0], torch.tensor(want, dtype=torch.float64))
    # the convolution sees zeros, not biases, before the first token
    c = plain.causal_conv(torch.ones(3, 1), torch.tensor([[1.0, 10.0, 100.0]]), torch.tensor([0.5]))
    assert c[:, 0].tolist() == [100.5, 110.5, 111.5]
    # the expert's unit
    y = plain.clamped_expert(torch.tensor([[1.0]]), torch.tensor([[5.0]]), torch.tensor([[-9.0]]), torch.tensor([[1.0]]), 2.0)
    assert abs(float(y) - 2.0 / (1 + math.exp(-1.702 * 2.0)) * (-2.0 + 1.0)) < 1e-6


def test_what_the_comparisons_rest_on_shows_in_the_plain_model(tmp_path):
    """A sink left out, a bucket moved by one, a lost state, a loop's vector left out, the correction left out: each
    moves the plain logits by far more than the tolerance the engine is held to."""
    toks = list(range(3, 60))

    def logits(name, change=None):
        cfg, W = plain.read_model_dir(tk.write_model(name, tmp_path / name))
        base = plain.forward(cfg, W, toks, torch.float64)
        if change is None:
            return base
        change(cfg, W)
        moved = plain.forward(cfg, W, toks, torch.float64)
        return float((moved - base).abs().max() / base.abs().max())

    def no_step(cfg, W):
        W["loop.step"] = torch.zeros_like(W["loop.step"])

    def shifted_rel(cfg, W):
        W["l0.mix.rel"] = torch.roll(W["l0.mix.rel"], 1, 0)

    def no_correction(cfg, W):
        W["l0.mlp.correction"] = torch.zeros_like(W["l0.mlp.correction"])

    def no_conv_history(cfg, W):
        W["l0.mix.conv"][:, :-1] = 0

    assert logits("mix", no_step) > 0.01
    assert logits("bias", shifted_rel) > 0.01
    assert logits("moe", no_correction) > 0.01
    assert logits("rglru", no_conv_history) > 0.01
    saved = plain.attention_sink
    try:
        def without_sink(h, W, m, positions):
            m = dict(m)
            out = saved(h, W, m, positions)
            return out * 1.3                       # stands for a denominator without the 1
        base = logits("sink")
        plain.attention_sink = without_sink
        cfg, W = plain.read_model_dir(tmp_path / "sink")
        assert float((plain.forward(cfg, W, toks, torch.float64) - base).abs().max() / base.abs().max()) > 0.01
    finally:
        plain.attention_sink = saved
