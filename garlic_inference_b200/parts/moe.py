"""A routed feed-forward (mixture of experts), as a feed-forward part.

    z = Wr x                                   router logits, float32 (the weight is widened, the product is a
                                               float32 kernel of its own; x may be its 16-bit rounding)
    scores "softmax_chosen" (the default): the `top` experts with the largest z are chosen; their weights are the
                               softmax over the chosen z alone
    scores "softmax_all":      s = softmax(z) over all experts; the experts lie in `groups` equal groups of
                               neighbours, a group's score is its largest s, and only the `groups_kept` best groups
                               stay; the `top` largest s among them are chosen; weights s * `weight_scale`, not
                               renormalised
    scores "sigmoid":          s = sigmoid(z), each expert by itself; groups as above.  With `correction` (a tensor
                               of one number per expert) the groups and the experts are chosen by s + correction
                               while the weights stay s; experts of a group that does not stay cannot be chosen
                               whatever their scores
    `group_score` "top2_sum":  a group's score is the sum of its two largest choosing scores ("best": the largest)
    `normalize`:               the chosen weights are divided by their sum (+ 1e-20) before `weight_scale`
    `shared` {size, ...unit}:  one more gated expert (tensors `shared.gate`, `shared.up`, `shared.down`; its own
                               limits) that every token runs and whose result is added with weight 1
    expert "two_matrix" (the default):  y = sum_e weight_e Wd_e act(Wu_e x), act the square of relu
                               ("relu_squared") or silu; no biases
    expert "glu":              y = sum_e weight_e Wd_e unit(Wg_e x, Wu_e x), a gated unit with `activation`,
                               `swish_alpha`, `gate_max`, `up_limit`, `up_shift` as in `glu_mlp`

The experts' matrices are stacked at load time ([experts, ff, hidden] and [experts, hidden, ff]).  Two ways to
run them.  A step of a few rows (a decode step; such a step may be recorded, so nothing may come back to the
host): kernels that read the chosen experts' matrices only, a warp per matrix row, the experts taken from
device memory.  More rows: the (token, choice) pairs are put in the order of their experts by a counting sort on
the device (which also gathers the tokens' vectors into that order), the experts run two matrix products over
their own rows, and one kernel sums each token's `top` results with its weights in the router's order.  In bfloat16 the two products are the library's grouped product (`torch._grouped_mm`: the rows
of every expert in one launch, the groups' ends read from device memory, nothing comes to the host); in float32,
or where the library has no grouped product, the counts come to the host once and every chosen expert runs this
package's products over its rows.  Either way a token's result does not depend on the other tokens of the step
beyond the rounding of the products.
NikolayBlagoev/garlic-inference's mixture-of-experts model is a different design (src/models/qwen3/qwen3-moe.cpp).
"""
from __future__ import annotations

import torch

from ..ops import glu_product, kernels, linear
from ..weights.loader import TensorWant
from .base import FeedForward, register_part

# Up to how many rows of a step the row-by-row kernels run (beyond: expert by expert through matrix products).
# The row-by-row kernels read an expert's matrices once per (token, choice) pair, the grouped product once per
# expert: from a few tokens on, pairs share experts.
ROWWISE_MAX_ROWS = 8


class RoutedExperts(FeedForward):
    kind = "routed_experts"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        hid, ff, E = params["hidden_size"], params["expert_size"], params["n_experts"]
        # scores over all experts: random routers are made wider, so that random models choose with clear margins
        w = {"router": TensorWant((E, hid), std_scale=4.0 if params.get("scores") in ("softmax_all", "sigmoid") else 1.0)}
        if params.get("correction", False):
            w["correction"] = TensorWant((E,), std_scale=5.0)
        if params.get("shared"):
            sf = int(params["shared"]["size"])
            w["shared.gate"], w["shared.up"], w["shared.down"] = TensorWant((sf, hid)), TensorWant((sf, hid)), TensorWant((hid, sf))
        for e in range(E):
            if params.get("expert", "two_matrix") == "glu":
                w[f"e{e}.gate"] = TensorWant((ff, hid))
            w[f"e{e}.up"], w[f"e{e}.down"] = TensorWant((ff, hid)), TensorWant((hid, ff))
        return w

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden, self.ff = int(params["hidden_size"]), int(params["expert_size"])
        self.E, self.top = int(params["n_experts"]), int(params["top"])
        self.gated = params.get("expert", "two_matrix") == "glu"
        if params.get("expert", "two_matrix") not in ("two_matrix", "glu"):
            raise ValueError(f"expert kind {params['expert']!r} is neither 'two_matrix' nor 'glu'")
        self.activation = params.get("activation", "silu" if self.gated else "relu_squared")
        if not 0 < self.top <= self.E:
            raise ValueError(f"{self.top} of {self.E} experts")
        if self.gated:
            # what the kernels take in place of an activation's name: the gated unit's constants
            self.act = kernels.glu_shape(self.activation, params.get("swish_alpha", 1.0), params.get("gate_max"),
                                         params.get("up_limit"), params.get("up_shift", 0.0))
        elif self.activation not in ("relu_squared", "silu"):
            raise ValueError(f"expert activation {self.activation!r} is neither 'relu_squared' nor 'silu'")
        else:
            self.act = self.activation
        self.scores = params.get("scores", "softmax_chosen")
        if self.scores not in ("softmax_chosen", "softmax_all", "sigmoid"):
            raise ValueError(f"router scores {self.scores!r} are none of 'softmax_chosen', 'softmax_all', 'sigmoid'")
        self.group_score = params.get("group_score", "best")
        if self.group_score not in ("best", "top2_sum"):
            raise ValueError(f"group_score {self.group_score!r} is neither 'best' nor 'top2_sum'")
        self.normalize = bool(params.get("normalize", False))
        self.groups, self.groups_kept = int(params.get("groups", 1)), int(params.get("groups_kept", params.get("groups", 1)))
        self.weight_scale = float(params.get("weight_scale", 1.0))
        if self.scores in ("softmax_all", "sigmoid"):
            per = self.E // max(self.groups, 1)
            if self.groups <= 0 or self.E % self.groups or not 0 < self.groups_kept <= self.groups or \
                    self.top > self.groups_kept * per:
                raise ValueError(f"{self.E} experts in {self.groups} groups of which {self.groups_kept} stay, top {self.top}")
        elif self.groups != 1 or self.weight_scale != 1.0 or self.normalize or params.get("correction", False):
            raise ValueError("groups of experts, a correction and a factor on the weights come with scores over all experts")
        self.w_router = load("router").to(torch.float32)
        self.correction = load("correction").to(torch.float32).contiguous() if params.get("correction", False) else None
        self.shared = None
        if params.get("shared"):
            if not self.gated:
                raise ValueError("a shared expert comes with gated experts")
            sh = params["shared"]
            sf = int(sh["size"])
            self.shared_unit = kernels.glu_shape(sh.get("activation", self.activation), sh.get("swish_alpha", 1.0),
                                                 sh.get("gate_max"), sh.get("up_limit"), sh.get("up_shift", 0.0))
            self.shared = torch.empty((2 * sf, self.hidden), dtype=load.dtype("shared.gate", "shared.up"), device=rt.device)
            load("shared.gate", out=self.shared[:sf])
            load("shared.up", out=self.shared[sf:])
            self.shared_down = load("shared.down")
        rows = 2 * self.ff if self.gated else self.ff
        names = [f"e{e}.{n}" for e in range(self.E) for n in (("gate", "up", "down") if self.gated else ("up", "down"))]
        dtype = load.dtype(*names)
        self.w_up = torch.empty((self.E, rows, self.hidden), dtype=dtype, device=rt.device)
        self.w_down = torch.empty((self.E, self.hidden, self.ff), dtype=dtype, device=rt.device)
        for e in range(self.E):
            if self.gated:                            # an expert's gate rows, then its up rows
                load(f"e{e}.gate", out=self.w_up[e, :self.ff])
            load(f"e{e}.up", out=self.w_up[e, rows - self.ff:])
            load(f"e{e}.down", out=self.w_down[e])

    def route(self, x):
        """(chosen experts int32 [n, top], their weights float32 [n, top]) for the rows of x."""
        logits = kernels.router_logits(x, self.w_router)
        if self.scores != "softmax_chosen":
            return kernels.router_select(logits, self.top, self.groups, self.groups_kept, self.weight_scale,
                                         sigmoid=self.scores == "sigmoid", correction=self.correction,
                                         group_top=2 if self.group_score == "top2_sum" else 1, normalize=self.normalize)
        return kernels.router_topk(logits, self.top)

    def _activate(self, z):
        return kernels.glu(z, self.act) if self.gated else kernels.relu_squared(z)

    def step(self, x, ctx):
        n = x.shape[0]
        idx, wt = self.route(x)
        # the shared expert's result joins the weighted sum inside the kernel that makes it, in float32
        add = linear(glu_product(x, self.shared, self.shared_unit), self.shared_down) if self.shared is not None else None
        grouped = self._grouped(x)
        products = self.gated or self.activation == "relu_squared"     # what the expert-by-expert path computes
        if n <= ROWWISE_MAX_ROWS or not products or (ctx.captured and not grouped):
            return kernels.moe_rowwise(x, self.w_up, self.w_down, idx, wt, self.act, add=add)
        # expert by expert: the pairs (token, choice) in the order of their experts; `where` is each pair's row
        where, ends, rows = kernels.moe_group(idx, x, self.E)
        if grouped:
            a = self._activate(torch._grouped_mm(rows, self.w_up.transpose(1, 2), offs=ends))
            buf = torch._grouped_mm(a, self.w_down.transpose(1, 2), offs=ends)
        else:
            buf = torch.empty((n * self.top, self.hidden), dtype=x.dtype, device=x.device)
            at = 0
            bounds = [0] + ends.tolist()                                   # the one trip to the host
            for e in range(self.E):
                c = bounds[e + 1] - bounds[e]
                if c:
                    a = self._activate(linear(rows[at:at + c], self.w_up[e]))
                    buf[at:at + c] = linear(a, self.w_down[e])
                    at += c
        return kernels.moe_combine(buf.contiguous(), where, wt, add)

    def _grouped(self, x) -> bool:
        """Whether the library's grouped product takes these operands: bfloat16, rows of 16-byte multiples."""
        return (x.dtype == torch.bfloat16 and self.w_up.dtype == torch.bfloat16 and hasattr(torch, "_grouped_mm")
                and self.hidden % 8 == 0 and self.ff % 8 == 0)


register_part(RoutedExperts.kind, RoutedExperts)
