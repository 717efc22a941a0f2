"""Typed configuration of the Kenovik decoder.

A Kenovik config.json names its model class as the string `architecture` and
gives `vocab`, `width`, `norm.eps`, `embedding.scale`, a list `layers` and,
optionally, `loop`; every layer entry has a `type` (which mixer), the mixer's
sizes and constants under `mixer` and a feed-forward under `mlp` (or null).  An
unknown mixer or feed-forward kind is refused by name; a key outside the design
is ignored with a warning.

    x0 = E[token] * embedding.scale
    x += mixer(rms(x) w1);   x += ff(rms(x) w2)                   pre-norm, RMS norms with eps inside the root
    logits = E rms(x) w_final                                     the head is the embedding table (without the scale)

`loop` = {start, stop, times}: the layers start .. stop - 1 run `times` times in
a row with the same weights and a cache entry of their own each time; row t of
the tensor `loop.step` [times, width] joins the stream right before pass t.

Mixers.  `attention`: grouped-query attention with biases on q, k, v, a rotation
of pairs (2i, 2i + 1) of the first `rot.dims` dimensions of every head whose
frequencies are divided by `rot.scaling.factor`, and a softmax whose
denominator holds one more 1 (a sink of score 0 without a value).
`attention_2`: no rotation; q and k are RMS-normed over the whole projection
(weights `q.norm`, `k.norm`), q grows with the position by `q_temp`, and a
learned bias per (bucket of the distance, head) joins the scaled scores
(tensor `rel`, whose row count is the number of buckets; distances from
`bias_max` on share the last).  `rglru`: the recurrent block with a real-gated
linear recurrent unit behind a short convolution.
Feed-forwards.  `dense`: down(silu(gate x) * (up x)).  `moe`: `top` of `experts`
gated experts g sigmoid(1.702 g) (u + 1) with g = min(gate x, limit), u =
clamp(up x, -limit, limit); sigmoid router scores, a `correction` per expert on
the scores that choose, groups of neighbours judged by their two best of which
`groups.keep` stay, weights normalised over the chosen and times `router.scale`;
a `shared` expert that every token runs.

The design gives no limit on positions; `MAX_POSITIONS` is this library's
(positions are int32 on the device and are turned into float32 angles).
"""
from __future__ import annotations

import copy
import json
import warnings
from dataclasses import dataclass, field
from typing import Optional

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry, optional, require

ARCHITECTURE = "Kenovik"
MAX_POSITIONS = 1 << 22
SWISH_ALPHA = 1.702        # inside the sigmoid of the experts' activation: fixed by the design
UP_SHIFT = 1.0             # added to the clamped up half: fixed by the design
DECAY_SCALE = 8.0          # log a = -8 r softplus(lam): fixed by the design
SINK_SCORE = 0.0           # the sink's score: exp(0) = 1 joins the denominator
DEFAULT_BIAS_ROWS = 32     # rows of a random model's distance-bias table (a file's tensor gives its own)

_HEADS = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float}


def _typed(d, keys: dict, where: str, optional_keys: tuple = ()) -> dict:
    """The listed keys of `d`, each of its type.  A key this library does not know is left out with a warning."""
    if not isinstance(d, dict):
        raise ConfigError(f"{where}: must be an object, found {d!r}")
    unknown = sorted(set(d) - set(keys) - set(optional_keys))
    if unknown:
        warnings.warn(f"{where}: keys {unknown} are not part of the design and are ignored", stacklevel=3)
    out = {}
    for k, typ in keys.items():
        if typ is dict:
            if not isinstance(d.get(k), dict):
                raise ConfigError(f"{where}: key '{k}' must be an object")
            out[k] = copy.deepcopy(d[k])
        else:
            out[k] = require(d, k, typ, where)
    return out


def _mixer(typ: str, m, w: str) -> dict:
    if typ == "attention":
        out = _typed(m, _HEADS, w, optional_keys=("rot",))
        if m.get("rot") is not None:
            rot = _typed(m["rot"], {"base": float, "dims": int}, w + ".rot", optional_keys=("scaling",))
            if m["rot"].get("scaling") is not None:
                rot["scaling"] = _typed(m["rot"]["scaling"], {"factor": float}, w + ".rot.scaling")
            out["rot"] = rot
        return out
    if typ == "attention_2":
        out = _typed(m, dict(_HEADS, bias_max=int), w, optional_keys=("q_temp", "bias_rows"))
        if m.get("q_temp") is not None:
            out["q_temp"] = _typed(m["q_temp"], {"coef": float, "every": int}, w + ".q_temp")
        if m.get("bias_rows") is not None:       # this library's own key, written with random models (see with_shapes)
            out["bias_rows"] = require(m, "bias_rows", int, w)
        return out
    if typ == "rglru":
        return _typed(m, {"width": int, "blocks": int, "conv": int}, w)
    raise ConfigError(f"{w[:-6]}: mixer type {typ!r} is none of 'attention', 'attention_2', 'rglru'")


def _mlp(mlp, w: str):
    if mlp is None:
        return None
    kind = require(mlp, "kind", str, w)
    if kind == "dense":
        return _typed(mlp, {"kind": str, "ff": int}, w)
    if kind != "moe":
        raise ConfigError(f"{w}: kind {kind!r} is neither 'dense' nor 'moe'")
    out = _typed(mlp, {"kind": str, "expert": dict, "router": dict}, w, optional_keys=("shared",))
    out["expert"] = _typed(out["expert"], {"ff": int, "limit": float}, w + ".expert")
    router = out["router"]
    groups = router.get("groups")
    out["router"] = _typed(router, {"experts": int, "top": int, "scale": float}, w + ".router", optional_keys=("groups",))
    out["router"]["groups"] = _typed(groups, {"count": int, "keep": int}, w + ".router.groups") \
        if groups is not None else {"count": 1, "keep": 1}
    if mlp.get("shared") is not None:
        out["shared"] = _typed(mlp["shared"], {"ff": int, "limit": float}, w + ".shared")
    return out


@dataclass
class KenovikConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float = 1.0
    layers: list = field(default_factory=list)      # the entries of config.json's `layers`, checked
    loop: Optional[dict] = None                     # {start, stop, times} or None
    max_position_embeddings: int = MAX_POSITIONS    # not a key of the design: this library's own limit

    def __post_init__(self):
        self.validate()

    # ---- reading and writing -------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, where: str = "config.json") -> "KenovikConfig":
        norm, emb = cfg.get("norm"), cfg.get("embedding")
        if not isinstance(norm, dict):
            raise ConfigError(f"{where}: key 'norm' must be an object with 'eps'")
        if not isinstance(emb, dict):
            raise ConfigError(f"{where}: key 'embedding' must be an object with 'scale'")
        layers = []
        for i, entry in enumerate(require(cfg, "layers", list, where)):
            w = f"{where}: layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{w}: must be an object")
            unknown = sorted(set(entry) - {"type", "mixer", "mlp"})
            if unknown:
                warnings.warn(f"{w}: keys {unknown} are not part of the design and are ignored", stacklevel=2)
            typ = require(entry, "type", str, w)
            layers.append({"type": typ, "mixer": _mixer(typ, entry.get("mixer"), w + ".mixer"),
                           "mlp": _mlp(entry.get("mlp"), w + ".mlp")})
        loop = None
        if cfg.get("loop") is not None:
            loop = _typed(cfg["loop"], {"start": int, "stop": int, "times": int}, where + ": loop")
        return cls(vocab=require(cfg, "vocab", int, where), width=require(cfg, "width", int, where),
                   norm_eps=require(norm, "eps", float, where + ": norm"),
                   embedding_scale=require(emb, "scale", float, where + ": embedding"), layers=layers, loop=loop)

    def to_dict(self) -> dict:
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "layers": copy.deepcopy(self.layers)}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        return out

    # ---- checks ----------------------------------------------------------------
    def validate(self) -> None:
        bad = []
        if self.vocab <= 0 or self.width <= 0:
            bad.append("vocab and width must be positive")
        if not self.norm_eps > 0:
            bad.append(f"norm.eps must be positive, found {self.norm_eps}")
        if not self.layers:
            bad.append("'layers' is empty")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp["start"] <= lp["stop"] <= len(self.layers)) or lp["times"] < 1:
                bad.append(f"loop {lp} does not fit {len(self.layers)} layers (0 <= start <= stop <= layers, times >= 1)")
        for i, layer in enumerate(self.layers):
            m, at = layer["mixer"], f"layers[{i}].mixer"
            if layer["type"] in ("attention", "attention_2"):
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    if m[k] <= 0:
                        bad.append(f"{at}.{k} must be positive, found {m[k]}")
                if m["kv_heads"] > 0 and m["heads"] % m["kv_heads"]:
                    bad.append(f"{at}: {m['heads']} heads are no multiple of {m['kv_heads']} kv_heads")
            if layer["type"] == "attention" and m.get("rot") is not None:
                rot = m["rot"]
                if rot["dims"] % 2 or not 0 <= rot["dims"] <= m["dim"] or rot["base"] <= 0:
                    bad.append(f"{at}.rot: dims {rot['dims']} must be even and at most dim {m['dim']}, the base positive")
                if rot.get("scaling") is not None and not rot["scaling"]["factor"] > 0:
                    bad.append(f"{at}.rot.scaling.factor must be positive")
            if layer["type"] == "attention_2":
                rows = m.get("bias_rows", DEFAULT_BIAS_ROWS)
                if rows < 1 or m["bias_max"] <= rows // 2:
                    bad.append(f"{at}: bias_max {m['bias_max']} must pass half of the bias table's {rows} rows")
                if m.get("q_temp") is not None and m["q_temp"]["every"] <= 0:
                    bad.append(f"{at}.q_temp.every must be positive")
            if layer["type"] == "rglru":
                if m["width"] <= 0 or m["blocks"] <= 0 or m["width"] % m["blocks"]:
                    bad.append(f"{at}: {m['width']} channels do not fall into {m['blocks']} equal blocks")
                if not 1 <= m["conv"] <= 16:
                    bad.append(f"{at}.conv = {m['conv']} taps is outside this library's 1 to 16")
            mlp = layer["mlp"]
            if mlp is not None and mlp["kind"] == "moe":
                r, g = mlp["router"], mlp["router"]["groups"]
                if mlp["expert"]["ff"] <= 0 or r["experts"] <= 0:
                    bad.append(f"layers[{i}].mlp: {r['experts']} experts of {mlp['expert']['ff']}")
                elif g["count"] <= 0 or r["experts"] % g["count"] or not 0 < g["keep"] <= g["count"]:
                    bad.append(f"layers[{i}].mlp.router: {r['experts']} experts do not fall into {g['count']} equal "
                               f"groups of which {g['keep']} stay")
                elif not 0 < r["top"] <= g["keep"] * (r["experts"] // g["count"]):
                    bad.append(f"layers[{i}].mlp.router: top {r['top']} of the {g['keep']} x "
                               f"{r['experts'] // g['count']} experts that stay")
                if mlp.get("shared") is not None and mlp["shared"]["ff"] <= 0:
                    bad.append(f"layers[{i}].mlp.shared.ff must be positive")
            elif mlp is not None and mlp["ff"] <= 0:
                bad.append(f"layers[{i}].mlp.ff must be positive")
        if bad:
            raise ConfigError("config: " + "; ".join(bad))

    def with_shapes(self, shapes: dict) -> "KenovikConfig":
        """The same configuration with the sizes that only the tensors give (the rows of each distance-bias table,
        from `l<i>.mix.rel`) taken from `shapes` {tensor name: shape}."""
        out = copy.deepcopy(self)
        for i, layer in enumerate(out.layers):
            name = f"l{i}.mix.rel"
            if layer["type"] == "attention_2" and name in shapes:
                layer["mixer"]["bias_rows"] = int(shapes[name][0])
        out.validate()
        return out

    # ---- the plan ----------------------------------------------------------------
    def layer_runs(self) -> list:
        """[(layer, pass or None)] in the order the layers run: the layers before the loop, the looped layers pass
        by pass, the rest."""
        n = len(self.layers)
        lp = self.loop
        if lp is None or lp["stop"] <= lp["start"]:
            return [(i, None) for i in range(n)]
        runs = [(i, None) for i in range(lp["start"])]
        for t in range(lp["times"]):
            runs += [(i, t) for i in range(lp["start"], lp["stop"])]
        return runs + [(i, None) for i in range(lp["stop"], n)]

    def _unit(self, limit: float) -> dict:
        return dict(activation="swish", swish_alpha=SWISH_ALPHA, gate_max=limit, up_limit=limit, up_shift=UP_SHIFT)

    def _mixer_spec(self, i: int, layer: dict):
        m, p, w = layer["mixer"], f"l{i}.mix.", self.width
        if layer["type"] == "rglru":
            names = ("y", "y.b", "x", "x.b", "conv", "conv.b", "ra", "ra.b", "ri", "ri.b", "lam", "o")
            return PartSpec("rglru", dict(hidden_size=w, width=m["width"], blocks=m["blocks"], conv_taps=m["conv"],
                                          decay_scale=DECAY_SCALE), {n: p + n for n in names}), None
        params = dict(hidden_size=w, n_heads=m["heads"], n_kv_heads=m["kv_heads"], key_dim=m["dim"],
                      value_dim=m["vdim"], softmax_scale=m["scale"], mask={"kind": "causal"})
        if layer["type"] == "attention":
            params.update(qkv_bias=True, sink=SINK_SCORE)
            names = ["q", "k", "v", "o", "q.b", "k.b", "v.b"]
            rot, rp = m.get("rot"), None
            if rot is not None and rot["dims"]:
                rp = dict(head_dim=m["dim"], rotary_dim=rot["dims"], theta=rot["base"],
                          max_positions=self.max_position_embeddings, layout="interleaved", tables=False,
                          linear_factor=(rot.get("scaling") or {}).get("factor", 1.0))
            return PartSpec("masked_attention", params, {n: p + n for n in names}), rp
        params.update(projection_norm_eps=self.norm_eps,
                      distance_bias={"rows": m.get("bias_rows", DEFAULT_BIAS_ROWS), "max_distance": m["bias_max"]})
        if m.get("q_temp") is not None:
            params["query_temperature"] = dict(m["q_temp"])
        names = ["q", "k", "v", "o", "q.norm", "k.norm", "rel"]
        return PartSpec("masked_attention", params, {n: p + n for n in names}), None

    def _ff_spec(self, i: int, mlp):
        if mlp is None:
            return None
        p, w = f"l{i}.mlp.", self.width
        if mlp["kind"] == "dense":
            return PartSpec("glu_mlp", dict(hidden_size=w, intermediate_size=mlp["ff"], activation="silu"),
                            {n: p + n for n in ("gate", "up", "down")})
        r = mlp["router"]
        names = ["router", "correction"] + [f"e{e}.{n}" for e in range(r["experts"]) for n in ("gate", "up", "down")]
        params = dict(hidden_size=w, expert_size=mlp["expert"]["ff"], n_experts=r["experts"], top=r["top"],
                      expert="glu", **self._unit(mlp["expert"]["limit"]), scores="sigmoid", correction=True,
                      groups=r["groups"]["count"], groups_kept=r["groups"]["keep"], group_score="top2_sum",
                      normalize=True, weight_scale=r["scale"])
        if mlp.get("shared") is not None:
            params["shared"] = dict(size=mlp["shared"]["ff"], **self._unit(mlp["shared"]["limit"]))
            names += ["shared.gate", "shared.up", "shared.down"]
        return PartSpec("routed_experts", params, {n: p + n for n in names})

    def plan(self) -> ModelPlan:
        w = self.width
        norm = lambda name: PartSpec("rms_norm", dict(size=w, eps=self.norm_eps), dict(weight=name))
        specs, positions = [], {}
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            mixer, rot = self._mixer_spec(i, layer)
            position = None
            if rot is not None:
                position = "rotary:" + json.dumps(rot, sort_keys=True)
                positions.setdefault(position, PartSpec("rotary", rot))
            ff = self._ff_spec(i, layer["mlp"])
            norms = {"input": norm(p + "norm1")}
            if ff is not None:
                norms["post_mixer"] = norm(p + "norm2")
            specs.append(LayerSpec("pre_norm_residual", mixer, ff, norms, position))
        # every run of a layer has a cache entry of its own; the first layer of pass t takes row t of `loop.step` along
        schedule, offsets = [], {}
        looped = self.loop is not None and self.loop["stop"] > self.loop["start"]
        if looped:
            offsets["loop.step"] = PartSpec("stream_offset", dict(rows=self.loop["times"], hidden_size=w),
                                            dict(weight="loop.step"))
        for entry, (i, t) in enumerate(self.layer_runs()):
            first = looped and t is not None and i == self.loop["start"]
            schedule.append(ScheduleEntry(layer=i, cache=entry, offset=("loop.step", t) if first else None))
        return ModelPlan(
            architecture=ARCHITECTURE, hidden_size=w, vocab_size=self.vocab,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=w,
                                                       scale=self.embedding_scale), dict(weight="embed")),
            positions=positions, layers=tuple(specs), schedule=tuple(schedule),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", dict(hidden_size=w, vocab_size=self.vocab), dict(weight="embed")),
            offsets=offsets)
