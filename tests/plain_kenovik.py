"""The Kenovik decoder restated plainly: one function per mechanism, whole sequences, no cache, loops over tokens
where the design has a recurrence.  It shares no code with the package; the tests compare the engine with it.

    x0 = E[token] * embedding.scale
    layers `loop.start` .. `loop.stop` - 1 run `loop.times` times in a row (same weights, a cache of their own each
    time); before pass t the row t of `loop.step` joins the stream; the other layers run once, in order
    x += mixer(rms(x) w1);  x += ff(rms(x) w2)        rms(z) = z / sqrt(mean(z^2) + eps)
    logits = E rms(x) w_final                           the table itself, without the embedding's scale

`weights` maps tensor names to torch tensors; `cfg` is the dict a config.json of the design holds.  Everything runs
in the dtype of `dtype` (float64 for the yardstick, float32 for its own rounding error).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


def read_safetensors(path) -> dict:
    """{name: tensor} of a safetensors file: 8 bytes of length, that many of JSON, then the data."""
    raw = Path(path).read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    meta = json.loads(raw[8:8 + n])
    types = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    out = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        a, b = m["data_offsets"]
        out[name] = torch.frombuffer(bytearray(raw[8 + n + a:8 + n + b]), dtype=types[m["dtype"]]).reshape(m["shape"])
    return out


def read_model_dir(model_dir):
    model_dir = Path(model_dir)
    return json.loads((model_dir / "config.json").read_text()), read_safetensors(model_dir / "model.safetensors")


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ---- rotation of pairs (2i, 2i + 1) of the first `dims` dimensions of every head --------------------------------
def rotate_pairs(x, positions, dims, base, factor):
    """x [T, heads, d]; pair i turns by position * base^(-2i/dims) / factor."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=x.dtype)
    f = base ** (-2.0 * i / dims) / factor
    ang = positions.to(x.dtype)[:, None] * f[None, :]                     # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---- attention with an empty sink -------------------------------------------------------------------------------
def attention_sink(h, W, m, positions):
    """Mixer 'attention': biased projections, rotation, causal softmax whose denominator holds one more 1."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W["q"].T + W["q.b"]).reshape(T, H, d)
    k = (h @ W["k"].T + W["k.b"]).reshape(T, G, d)
    v = (h @ W["v"].T + W["v.b"]).reshape(T, G, dv)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    q = rotate_pairs(q, positions, rot["dims"], rot["base"], factor)
    k = rotate_pairs(k, positions, rot["dims"], rot["base"], factor)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    seen = positions[None, :] <= positions[:, None]
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].T) * m["scale"]
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        top = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)         # the sink's score is 0
        e = torch.exp(s - top)
        p = e / (torch.exp(-top) + e.sum(-1, keepdim=True))
        out[:, n] = p @ v[:, g]
    return out.reshape(T, H * dv) @ W["o"].T


# ---- attention with a learned bias per distance -----------------------------------------------------------------
def distance_bucket(n: int, rows: int, far: int) -> int:
    """Which row of the bias table the distance n >= 0 reads: the first half of the rows one distance each, the
    second half spread evenly over the logarithm up to `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def query_temperature(positions, coef, every, dtype):
    return 1.0 + coef * torch.log(torch.floor((positions.to(dtype) + 1.0) / every) + 1.0)


def attention_bias(h, W, m, positions, eps):
    """Mixer 'attention_2': q and k normed over the whole projection, a factor on q that grows with the position,
    no rotation, a bias per (distance bucket, head) on the scaled scores, plain causal softmax."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ W["q"].T, W["q.norm"], eps)
    k = rms_norm(h @ W["k"].T, W["k.norm"], eps)
    if m.get("q_temp"):
        q = q * query_temperature(positions, m["q_temp"]["coef"], m["q_temp"]["every"], h.dtype)[:, None]
    q, k = q.reshape(T, H, d), k.reshape(T, G, d)
    v = (h @ W["v"].T).reshape(T, G, dv)
    rel = W["rel"]                                                         # [rows, heads]
    rows = rel.shape[0]
    dist = (positions[:, None] - positions[None, :]).clamp(min=0)
    by_distance = torch.tensor([distance_bucket(n, rows, m["bias_max"]) for n in range(int(dist.max()) + 1)])
    buckets = by_distance[dist]
    seen = positions[None, :] <= positions[:, None]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].T) * m["scale"] + rel[:, n][buckets]
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        out[:, n] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * dv) @ W["o"].T


# ---- the recurrent block ------------------------------------------------------------------------------------------
def causal_conv(x, taps, bias):
    """x [T, C]; taps [C, K], the last column on the present token; zeros before the first token."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x])
    out = torch.zeros_like(x) + bias
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j]
    return out


def rglru(h, W, m, state=None):
    """Mixer 'rglru'.  y = gelu(Wy h + by);  u = conv(Wx h + bx);  per block of channels r = sigmoid(Ra u + ra),
    i = sigmoid(Ri u + ri);  a = exp(-8 r softplus(lam));  S <- a S + sqrt(1 - a^2) i u;  out = Wo (S y)."""
    T = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(h @ W["y"].T + W["y.b"])
    u = causal_conv(h @ W["x"].T + W["x.b"], W["conv"], W["conv.b"])
    ub = u.reshape(T, blocks, width // blocks)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W["ra"]) + W["ra.b"]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W["ri"]) + W["ri.b"]).reshape(T, width)
    log_a = -8.0 * r * softplus(W["lam"])
    a = torch.exp(log_a)
    b = torch.sqrt(torch.clamp(1.0 - a * a, min=0.0)) * i * u
    S = torch.zeros(width, dtype=h.dtype) if state is None else state
    out = torch.zeros(T, width, dtype=h.dtype)
    for t in range(T):
        S = a[t] * S + b[t]
        out[t] = S
    return (out * y) @ W["o"].T


# ---- feed-forwards --------------------------------------------------------------------------------------------------
def dense_ff(h, W):
    g = h @ W["gate"].T
    return (g * torch.sigmoid(g) * (h @ W["up"].T)) @ W["down"].T


def clamped_expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, W, r):
    """(chosen experts [T, top], weights [T, top]): sigmoid scores, a correction on the scores that choose, groups
    judged by their two best, weights from the scores without the correction."""
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(h @ W["router"].T)
    choice = s + W["correction"]
    T = h.shape[0]
    per = E // groups["count"]
    if groups["count"] > 1:
        by_group = choice.reshape(T, groups["count"], per)
        best_two = by_group.topk(min(2, per), -1).values.sum(-1)
        kept = best_two.topk(groups["keep"], -1).indices
        open_ = torch.zeros(T, groups["count"], dtype=torch.bool)
        open_.scatter_(1, kept, True)
        choice = torch.where(open_[:, :, None].expand(T, groups["count"], per).reshape(T, E), choice,
                             torch.full_like(choice, -math.inf))
    idx = choice.topk(top, -1).indices
    w = s.gather(1, idx)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    return idx, w


def moe_ff(h, W, mlp):
    idx, w = route(h, W, mlp["router"])
    out = torch.zeros(h.shape[0], W["e0.down"].shape[0], dtype=h.dtype)
    limit = mlp["expert"]["limit"]
    for t in range(h.shape[0]):
        for e, wt in zip(idx[t].tolist(), w[t]):
            out[t] += wt * clamped_expert(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], limit)[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, W["shared.gate"], W["shared.up"], W["shared.down"], mlp["shared"]["limit"])
    return out


# ---- the model ------------------------------------------------------------------------------------------------------
def layer_order(cfg):
    """[(layer, pass or None)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"] if loop["stop"] > loop["start"] else 0):
        order += [(i, t) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"] if loop["stop"] > loop["start"] else loop["start"], n)]


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one whole sequence (positions 0 .. T-1)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = W["embed"][tokens] * cfg["embedding"]["scale"]
    loop = cfg.get("loop") or {}
    after = []
    for i, t in layer_order(cfg):
        if t is not None and i == loop["start"]:
            x = x + W["loop.step"][t]
        layer, p = cfg["layers"][i], f"l{i}."
        h = rms_norm(x, W[p + "norm1"], eps)
        mix = sub(W, p + "mix.")
        if layer["type"] == "attention":
            x = x + attention_sink(h, mix, layer["mixer"], positions)
        elif layer["type"] == "attention_2":
            x = x + attention_bias(h, mix, layer["mixer"], positions, eps)
        elif layer["type"] == "rglru":
            x = x + rglru(h, mix, layer["mixer"])
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, W[p + "norm2"], eps)
            ff = sub(W, p + "mlp.")
            x = x + (dense_ff(h, ff) if mlp["kind"] == "dense" else moe_ff(h, ff, mlp))
        after.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits
