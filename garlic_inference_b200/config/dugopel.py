"""Typed configuration of the Dugopel decoder.

A Dugopel config.json names its model class as the string `architecture` and
gives `vocab`, `width`, `norm.eps`, `embedding.scale`, `logit_softcap` and a list
`layers`; every entry has a `type` (which mixer), the mixer's sizes and constants
under `mixer` and a feed-forward under `mlp` (or null).  An unknown mixer or
feed-forward kind is refused by name; a key outside the design is ignored with a
warning.

    x0 = E[token] * embedding.scale
    h = ln(x);  x += mixer(h) + ff(h)                    one mean-subtracting norm (weight, no bias) per layer,
                                                         read by both sublayers
    logits = cap * tanh( head ln_final(x) / cap )

Mixer `latent_attention`: queries through a normed latent of `q_rank`, keys and
values expanded from a normed latent of `kv_rank` beside one rotated key part of
`rot_dim` shared by all heads; rotation of halves (dimension i with i + dims/2);
causal softmax with the configuration's `scale`; a sigmoid gate per head made from
the mixer's input.  With `kv_from: j` the layer has no down-projection for keys
and values and reads the latent rows that layer j cached.
Feed-forwards.  `dense`: down( g sigmoid(1.702 g) (u + 1) ) with g = min(gate x,
limit), u = clamp(up x, -limit, limit).  `moe`: `top` of `experts` such
feed-forwards; router scores are a softmax over all experts, experts lie in
`groups.count` groups of neighbours of which the `groups.keep` with the largest
best score stay, the chosen experts' scores times `router.scale` are the weights.

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

ARCHITECTURE = "Dugopel"
MAX_POSITIONS = 1 << 22
SWISH_ALPHA = 1.702        # inside the sigmoid of the feed-forwards' activation: fixed by the design
UP_SHIFT = 1.0             # added to the clamped up half: fixed by the design

_MIXER = {"heads": int, "dim": int, "rot_dim": int, "vdim": int, "kv_rank": int, "q_rank": int, "scale": float,
          "rot": dict}


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


@dataclass
class DugopelConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float = 1.0
    logit_softcap: Optional[float] = None
    layers: list = field(default_factory=list)      # the entries of config.json's `layers`, checked
    max_position_embeddings: int = MAX_POSITIONS    # not a key of the design: this library's own limit

    def __post_init__(self):
        self.validate()

    # ---- reading and writing -------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, where: str = "config.json") -> "DugopelConfig":
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
            if typ != "latent_attention":
                raise ConfigError(f"{w}: mixer type {typ!r} is not 'latent_attention'")
            m = entry.get("mixer")
            mixer = _typed(m, _MIXER, w + ".mixer", optional_keys=("kv_from",))
            mixer["rot"] = _typed(mixer["rot"], {"base": float, "dims": int}, w + ".mixer.rot")
            if m.get("kv_from") is not None:
                mixer["kv_from"] = require(m, "kv_from", int, w + ".mixer")
            mlp = entry.get("mlp")
            if mlp is not None:
                kind = require(mlp, "kind", str, w + ".mlp")
                if kind == "dense":
                    mlp = _typed(mlp, {"kind": str, "ff": int, "limit": float}, w + ".mlp")
                elif kind == "moe":
                    mlp = _typed(mlp, {"kind": str, "expert": dict, "router": dict}, w + ".mlp")
                    mlp["expert"] = _typed(mlp["expert"], {"ff": int, "limit": float}, w + ".mlp.expert")
                    if isinstance(mlp["router"], dict) and mlp["router"].get("groups") is None:
                        mlp["router"] = dict(mlp["router"], groups={"count": 1, "keep": 1})     # no groups: one of all
                    mlp["router"] = _typed(mlp["router"], {"experts": int, "top": int, "scale": float, "groups": dict},
                                           w + ".mlp.router")
                    mlp["router"]["groups"] = _typed(mlp["router"]["groups"], {"count": int, "keep": int},
                                                     w + ".mlp.router.groups")
                else:
                    raise ConfigError(f"{w}.mlp: kind {kind!r} is neither 'dense' nor 'moe'")
            layers.append({"type": typ, "mixer": mixer, "mlp": mlp})
        return cls(vocab=require(cfg, "vocab", int, where), width=require(cfg, "width", int, where),
                   norm_eps=require(norm, "eps", float, where + ": norm"),
                   embedding_scale=require(emb, "scale", float, where + ": embedding"),
                   logit_softcap=optional(cfg, "logit_softcap", float, None, where), layers=layers)

    def to_dict(self) -> dict:
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "layers": copy.deepcopy(self.layers)}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out

    # ---- checks ----------------------------------------------------------------
    def validate(self) -> None:
        bad = []
        if self.vocab <= 0 or self.width <= 0:
            bad.append("vocab and width must be positive")
        if not self.norm_eps > 0:
            bad.append(f"norm.eps must be positive, found {self.norm_eps}")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            bad.append(f"logit_softcap must be positive, found {self.logit_softcap}")
        if not self.layers:
            bad.append("'layers' is empty")
        for i, layer in enumerate(self.layers):
            m, at = layer["mixer"], f"layers[{i}].mixer"
            for k in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
                if m[k] <= 0:
                    bad.append(f"{at}.{k} must be positive, found {m[k]}")
            rot = m["rot"]
            if m["rot_dim"] < 0 or rot["dims"] % 2 or not 0 <= rot["dims"] <= m["rot_dim"] or rot["base"] <= 0:
                bad.append(f"{at}: rot.dims {rot['dims']} must be even and at most rot_dim {m['rot_dim']}, the base "
                           "positive")
            j = m.get("kv_from")
            if j is not None:
                src = self.layers[j] if 0 <= j < i else None
                if src is None or src["mixer"].get("kv_from") is not None:
                    bad.append(f"{at}.kv_from = {j} must name an earlier layer with a latent of its own")
                elif any(src["mixer"][k] != m[k] for k in ("kv_rank", "rot_dim", "rot")):
                    bad.append(f"{at}.kv_from = {j}: that layer's kv_rank, rot_dim or rotation differ from this one's")
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
            elif mlp is not None and mlp["ff"] <= 0:
                bad.append(f"layers[{i}].mlp.ff must be positive")
        if bad:
            raise ConfigError("config: " + "; ".join(bad))

    # ---- the plan ----------------------------------------------------------------
    def _glu(self, limit: float) -> dict:
        return dict(activation="swish", swish_alpha=SWISH_ALPHA, gate_max=limit, up_limit=limit, up_shift=UP_SHIFT)

    def plan(self) -> ModelPlan:
        w = self.width
        norm = lambda name: PartSpec("layer_norm", dict(size=w, eps=self.norm_eps), dict(weight=name))
        specs, positions, schedule = [], {}, []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer["mixer"]
            own = m.get("kv_from") is None
            params = dict(hidden_size=w, n_heads=m["heads"], plain_dim=m["dim"], rot_dim=m["rot_dim"],
                          value_dim=m["vdim"], kv_rank=m["kv_rank"], q_rank=m["q_rank"], softmax_scale=m["scale"],
                          eps=self.norm_eps, head_gate=True, own_kv=own)
            names = ["dq", "dq.norm", "uq", "uk", "uv", "g", "o"] + (["dkv", "dkv.norm"] if own else [])
            mixer = PartSpec("latent_attention", params, {n: p + "mix." + n for n in names})
            position = None
            if m["rot"]["dims"]:
                rp = dict(head_dim=m["rot_dim"], rotary_dim=m["rot"]["dims"], theta=m["rot"]["base"],
                          max_positions=self.max_position_embeddings, layout="half", tables=False)
                position = "rotary:" + json.dumps(rp, sort_keys=True)
                positions.setdefault(position, PartSpec("rotary", rp))
            mlp, ff = layer["mlp"], None
            if mlp is not None and mlp["kind"] == "dense":
                ff = PartSpec("glu_mlp", dict(hidden_size=w, intermediate_size=mlp["ff"], **self._glu(mlp["limit"])),
                              {n: p + "mlp." + n for n in ("gate", "up", "down")})
            elif mlp is not None:
                r = mlp["router"]
                names = ["router"] + [f"e{e}.{n}" for e in range(r["experts"]) for n in ("gate", "up", "down")]
                ff = PartSpec("routed_experts",
                              dict(hidden_size=w, expert_size=mlp["expert"]["ff"], n_experts=r["experts"], top=r["top"],
                                   expert="glu", **self._glu(mlp["expert"]["limit"]), scores="softmax_all",
                                   groups=r["groups"]["count"], groups_kept=r["groups"]["keep"], weight_scale=r["scale"]),
                              {n: p + "mlp." + n for n in names})
            specs.append(LayerSpec("parallel_residual", mixer, ff, {"input": norm(p + "norm1")}, position))
            schedule.append(ScheduleEntry(layer=i, cache=i, kv_cache=m.get("kv_from")))
        head = dict(hidden_size=w, vocab_size=self.vocab)
        if self.logit_softcap is not None:
            head["softcap"] = self.logit_softcap
        return ModelPlan(
            architecture=ARCHITECTURE, hidden_size=w, vocab_size=self.vocab,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=w,
                                                       scale=self.embedding_scale), dict(weight="embed")),
            positions=positions, layers=tuple(specs), schedule=tuple(schedule),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", head, dict(weight="head")))
