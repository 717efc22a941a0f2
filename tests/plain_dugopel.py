"""Plain, slow restatement of the Dugopel decoder, used only by the tests.

Whole sequences, no cache, one function per mechanism, keys and values expanded
head by head, torch on the CPU in float32 (or float64 when asked).  It shares no
code with the package under test (the file reader is the other plain model's).

The design in this file's notation (x is the float32 residual stream, T tokens at
positions 0 .. T-1):

    x0          = E[token] * embedding.scale
    layer:      h = ln(x);  x += mixer(h) + ff(h)        one norm, both sublayers read it; ff may be absent
    ln:         (x - mean) / sqrt(var + eps) * w          var = mean of squared deviations; no bias
    rms:        z / sqrt(mean(z^2) + eps) * w
    latent:     cq = rms(Wdq h);  q = Wuq cq = per head [ plain (dim) | turned (rot_dim) ]
                [c | kr] = Wdkv h;  c <- rms(c)  (kv_rank);  kr (rot_dim) is one key part for all heads
                key_n = [ Wuk,n c | turn(kr) ],  value_n = Wuv,n c
                turn: of the first rot.dims dimensions, i and i + dims/2 (i < dims/2) turn by
                      position * base^(-2i/dims); the others pass
                p = softmax_j( (q_plain . k_plain + turn(q_rot) . turn(kr)) * scale ),  j <= i
                o_n = sum_j p_j value_n,j * sigmoid(Wg h)_n;   y = Wo concat(o)
                with kv_from = j the layer has no Wdkv: c and turn(kr) are layer j's
    swish-glu:  g = min(Wgate h, limit);  u = clamp(Wup h, -limit, limit);  a = g sigmoid(1.702 g) (u + 1);  Wdown a
    dense ff:   one swish-glu
    moe ff:     s = softmax(Wr h) over all experts;  experts lie in groups.count equal groups of neighbours, a
                group's score is its largest s, only the groups.keep best groups stay;  the `top` largest s among
                them are chosen;  y = sum_e s_e * router.scale * swish-glu_e(h)          (no renormalisation)
    logits      = cap * tanh( head ln_final(x) / cap )
"""
from __future__ import annotations

import torch

from plain_fivitar import read_model_dir, read_safetensors  # noqa: F401  (file readers only)

SWISH_ALPHA = 1.702


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def layer_norm(x, w, eps: float):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_norm(x, w, eps: float):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def turn_halves(x, dims: int, base: float, first_pos: int = 0):
    """x [T, ..., D]: of the first `dims` dimensions, i and i + dims/2 of the token at position p turn by
    p * base^(-2i/dims); dimensions from `dims` on pass."""
    T, half = x.shape[0], dims // 2
    out = x.clone()
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64).to(x.dtype)
    ang = (first_pos + torch.arange(T)).to(x.dtype)[:, None] * f[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def causal_softmax(scores):
    """scores [H, T, T] (query, key): softmax over the keys j <= i."""
    T = scores.shape[-1]
    seen = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    return torch.softmax(scores.masked_fill(~seen[None], float("-inf")), dim=-1)


def latent_attention(h, w, m, eps, shared, index):
    """h [T, width] -> [T, width].  `shared` {layer: (c, turned kr)} holds what the layers run so far cached."""
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    dims, base = m["rot"]["dims"], m["rot"]["base"]
    T = h.shape[0]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], turn_halves(q[..., d:], dims, base)
    if m.get("kv_from") is not None:
        c, kr = shared[m["kv_from"]]
    else:
        ckr = h @ w["dkv"].T
        c = rms_norm(ckr[:, :r], w["dkv.norm"], eps)
        kr = turn_halves(ckr[:, r:], dims, base)
    shared[index] = (c, kr)
    k_plain = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, kr)) * m["scale"]
    o = torch.einsum("hij,jhv->ihv", causal_softmax(scores), v)
    o = o * sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w["o"].T


def swish_glu(h, gate, up, down, limit: float):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * sigmoid(SWISH_ALPHA * g) * (u + 1.0)) @ down.T


def dense_ff(h, w, mlp):
    return swish_glu(h, w["gate"], w["up"], w["down"], mlp["limit"])


def route(z, router: dict):
    """z [T, E] router logits -> (chosen experts [T, top], weights [T, top])."""
    E, top = router["experts"], router["top"]
    count, keep = router["groups"]["count"], router["groups"]["keep"]
    s = torch.softmax(z, dim=-1)
    best = s.view(-1, count, E // count).max(-1).values                       # a group's score
    kept = torch.zeros_like(best, dtype=torch.bool)
    kept.scatter_(1, torch.topk(best, keep, dim=-1).indices, True)
    allowed = kept[:, :, None].expand(-1, -1, E // count).reshape(-1, E)
    val, idx = torch.topk(s.masked_fill(~allowed, -1.0), top, dim=-1)
    return idx, val * router["scale"]


def moe_ff(h, w, mlp):
    router = mlp["router"]
    idx, wt = route(h @ w["router"].T, router)
    out = torch.zeros_like(h)
    for e in range(router["experts"]):
        y = swish_glu(h, w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], mlp["expert"]["limit"])
        out = out + y * (wt * (idx == e)).sum(-1, keepdim=True)
    return out


def under(weights: dict, prefix: str, dtype) -> dict:
    return {n[len(prefix):]: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()
            if n.startswith(prefix)}


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float32, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] for one sequence from position 0; `layers_out` collects the stream after each layer."""
    eps = cfg["norm"]["eps"]
    x = weights["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    shared: dict = {}
    for i, spec in enumerate(cfg["layers"]):
        lw = under(weights, f"l{i}.", dtype)
        h = layer_norm(x, lw["norm1"], eps)
        y = latent_attention(h, under(lw, "mix.", dtype), spec["mixer"], eps, shared, i)
        mlp = spec.get("mlp")
        if mlp is not None:
            mw = under(lw, "mlp.", dtype)
            y = y + (dense_ff(h, mw, mlp) if mlp["kind"] == "dense" else moe_ff(h, mw, mlp))
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    z = layer_norm(x, weights["final.norm"].to(dtype), eps) @ weights["head"].to(dtype).T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
