"""A plain, slow implementation of the Tevilix decoder, for tests only.

Whole sequences, no cache, no batching, one function per mechanism, numpy in double precision.
It shares no code with the library.

The design in this file's notation.  x[t] = E[token_t] * s_e.  A layer reads the stream through two layer
norms (weight, no bias) and adds both sublayers at once:
    x <- x + mixer(LN1(x)) + ff(LN2(x))                       (ff absent: the mixer alone)
A range of layers [start, stop) runs `times` times in a row (start .. stop-1, then again), every pass with
memory of its own.  Mixers:

* parallel: a * attention(h) + b * min_gru(h), both on the same h.
  attention: q, k, v with biases; weighted RMS norm on every q and k head; rotation of the first `dims`
  numbers of q and k heads (pairs i, i + dims/2) by angle p * base^(-2i/dims) / factor; scores q.k * scale,
  then mixed across heads, s'_h = sum_g T[h, g] s_g; position i sees j with 0 <= i - j < window; softmax;
  the heads side by side times sigmoid(W_g h); W_o with bias.
  min_gru: z = sigmoid(W_z h + b_z), u = W_x h + b_x, c = u + 1/2 for u >= 0 and sigmoid(u) below;
  S <- (1 - z) S + z c per channel; W_o (S * silu(W_g h)).
* mlstm: matrix memory with exponential gates under a running maximum m (from 0): q = W_q h * dim^-1/2,
  k = W_k h, v = W_v h; i = cap tanh((W_i h + b_i) / cap), f = logsigmoid(cap tanh((W_f h + b_f) / cap));
  m' = max(f + m, i); S <- exp(f + m - m') S + exp(i - m') k v^T; n likewise with k;
  o = S^T q / (max(|n.q|, exp(-m')) + 1e-6); o over its root mean square per head, times a weight over all
  heads, times sigmoid(W_g h); W_o.

Feed-forwards: dense D gelu(U h) with the erf form; or experts D_e relu(U_e h)^2 chosen by a sigmoid router:
choice scores s + correction; experts in equal groups of neighbours, a group's rank the sum of its two best
choice scores, only the best `keep` groups eligible; the `top` best eligible; weights s / (sum + 1e-20) * scale.
Logits = H LN_final(x).
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


def read_safetensors(path: str) -> dict[str, np.ndarray]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, t = e["data_offsets"]
        if e["dtype"] == "BF16":
            arr = np.frombuffer(data[b:t], dtype=np.uint16).reshape(e["shape"])
            out[name] = (arr.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif e["dtype"] == "F32":
            out[name] = np.frombuffer(data[b:t], dtype=np.float32).reshape(e["shape"]).astype(np.float64)
        elif e["dtype"] == "I32":
            out[name] = np.frombuffer(data[b:t], dtype=np.int32).reshape(e["shape"]).copy()
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
    return out


# ---- small functions ---------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu_erf(z):
    return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))


def layer_norm(x, w, eps):
    m = x.mean(-1, keepdims=True)
    d = x - m
    return d / np.sqrt((d * d).mean(-1, keepdims=True) + eps) * w


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sub(w: dict, prefix: str) -> dict:
    """The tensors under `prefix.`, by the rest of their names."""
    p = prefix + "."
    return {k[len(p):]: v for k, v in w.items() if k.startswith(p)}


# ---- mixers -----------------------------------------------------------------------------------------
def rotate(x, pos, dims, base, factor):
    """x [T, heads, dim]: pairs (i, i + dims/2) of the first `dims` numbers turned by pos * f_i."""
    if not dims:
        return x
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims) / factor
    a = pos[:, None].astype(np.float64) * f[None, :]                                  # [T, half]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    y = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    y[..., :half] = u * c - v * s
    y[..., half:dims] = v * c + u * s
    return y


def mixed_heads_attention(h, w, m, eps):
    """Windowed softmax attention whose scores are mixed across heads before the softmax."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, d)
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, d)
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, e)
    q = unit_rms(q, eps) * w["q.norm"]
    k = unit_rms(k, eps) * w["k.norm"]
    pos = np.arange(T)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    q = rotate(q, pos, dims, float(rot.get("base", 10000.0)), factor)
    k = rotate(k, pos, dims, float(rot.get("base", 10000.0)), factor)
    kv_of = np.arange(H) // (H // G)
    s = np.einsum("ihd,jhd->hij", q, k[:, kv_of]) * m["scale"]                       # [H, T, T]
    s = np.einsum("hg,gij->hij", w["talk"], s)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = (i - j >= 0)
    window = int((m.get("mask") or {}).get("size", 0))
    if window:
        seen &= (i - j < window)
    s = np.where(seen[None], s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(-1, keepdims=True)
    o = np.einsum("hij,jhe->ihe", p, v[:, kv_of]).reshape(T, H * e)
    o = o * sigmoid(h @ w["g"].T)
    return o @ w["o"].T + w["o.b"]


def min_gru(h, w):
    z = sigmoid(h @ w["z"].T + w["z.b"])
    u = h @ w["x"].T + w["x.b"]
    c = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(z.shape[1])
    out = np.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        out[t] = S
    return (out * silu(h @ w["g"].T)) @ w["o"].T


def parallel_mixer(h, w, m, eps):
    left = mixed_heads_attention(h, sub(w, "left"), m["left"], eps)
    right = min_gru(h, sub(w, "right"))
    return float(m.get("left_scale", 1.0)) * left + float(m.get("right_scale", 1.0)) * right


def mlstm(h, w, m, eps):
    T = h.shape[0]
    H, d, e, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w["q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).reshape(T, H, d)
    v = (h @ w["v"].T).reshape(T, H, e)
    ig = cap * np.tanh((h @ w["i"].T + w["i.b"]) / cap)                              # [T, H]
    fg = log_sigmoid(cap * np.tanh((h @ w["f"].T + w["f.b"]) / cap))
    S = np.zeros((H, d, e))
    n = np.zeros((H, d))
    mx = np.zeros(H)
    o = np.zeros((T, H, e))
    for t in range(T):
        new = np.maximum(fg[t] + mx, ig[t])
        a = np.exp(fg[t] + mx - new)
        b = np.exp(ig[t] - new)
        mx = new
        for hh in range(H):
            S[hh] = a[hh] * S[hh] + b[hh] * np.outer(k[t, hh], v[t, hh])
            n[hh] = a[hh] * n[hh] + b[hh] * k[t, hh]
            den = max(abs(n[hh] @ q[t, hh]), math.exp(-mx[hh])) + 1e-6
            o[t, hh] = S[hh].T @ q[t, hh] / den
    o = unit_rms(o, eps).reshape(T, H * e) * w["norm"] * sigmoid(h @ w["g"].T)
    return o @ w["o"].T


# ---- feed-forwards ---------------------------------------------------------------------------------
def dense_ff(h, w):
    return gelu_erf(h @ w["up"].T) @ w["down"].T


def route(h, w, r):
    """Chosen experts [T, top], their weights [T, top], and the choice scores with the excluded groups at
    minus infinity [T, E]."""
    E, top = int(r["experts"]), int(r["top"])
    s = sigmoid(h @ w["router"].T)
    c = s + w["correction"]
    groups = r.get("groups") or {}
    count, keep = int(groups.get("count", 1)), int(groups.get("keep", 1))
    per = E // count
    rank = np.sort(c.reshape(-1, count, per), axis=-1)[..., -2:].sum(-1) if per >= 2 else c.reshape(-1, count, per).sum(-1)
    order = np.argsort(-rank, axis=-1, kind="stable")[:, :keep]                       # ties to the lower group
    allowed = np.zeros((h.shape[0], count), dtype=bool)
    np.put_along_axis(allowed, order, True, axis=-1)
    c = np.where(np.repeat(allowed, per, axis=-1), c, -np.inf)
    ids = np.argsort(-c, axis=-1, kind="stable")[:, :top]                             # ties to the lower index
    chosen = np.take_along_axis(s, ids, axis=-1)
    wts = chosen / (chosen.sum(-1, keepdims=True) + 1e-20) * float(r.get("scale", 1.0))
    return ids, wts, c


def experts_ff(h, w, mlp):
    ids, wts, _ = route(h, w, mlp["router"])
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], wts[t]):
            up = np.maximum(h[t] @ w[f"e{e}.up"].T, 0.0)
            out[t] += a * ((up * up) @ w[f"e{e}.down"].T)
    return out


# ---- the model ---------------------------------------------------------------------------------------
def layer_order(cfg: dict) -> list[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def run_layer(x, w, spec, eps):
    h1 = layer_norm(x, w["norm1"], eps)
    mw = sub(w, "mix")
    if spec["type"] == "parallel":
        y = parallel_mixer(h1, mw, spec["mixer"], eps)
    elif spec["type"] == "mlstm":
        y = mlstm(h1, mw, spec["mixer"], eps)
    else:
        raise ValueError(spec["type"])
    mlp = spec.get("mlp")
    if mlp is not None:
        h2 = layer_norm(x, w["norm2"], eps)
        fw = sub(w, "mlp")
        y = y + (dense_ff(h2, fw) if mlp["kind"] == "dense" else experts_ff(h2, fw, mlp))
    return x + y


def forward(cfg: dict, w: dict, tokens, streams: list | None = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence; `streams` collects the stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for li in layer_order(cfg):
        x = run_layer(x, sub(w, f"l{li}"), cfg["layers"][li], eps)
        if streams is not None:
            streams.append(x.copy())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T


def route_gap(h, w, r) -> np.ndarray:
    """Per row, how far the router's decisions are from falling the other way: the gap between the last chosen and
    the first rejected choice score among the eligible experts, and between the last kept and the first dropped group."""
    E, top = int(r["experts"]), int(r["top"])
    _, _, c = route(h, w, r)
    cs = -np.sort(-c, axis=-1)
    gap = np.full(h.shape[0], np.inf)
    if E > top:
        nxt = cs[:, top]
        gap = np.where(np.isfinite(nxt), cs[:, top - 1] - nxt, np.inf)
    groups = r.get("groups") or {}
    count, keep = int(groups.get("count", 1)), int(groups.get("keep", 1))
    if keep < count:
        per = E // count
        c0 = sigmoid(h @ w["router"].T) + w["correction"]
        rank = np.sort(c0.reshape(-1, count, per), axis=-1)[..., -2:].sum(-1) if per >= 2 else c0.reshape(-1, count, per).sum(-1)
        rs = -np.sort(-rank, axis=-1)
        gap = np.minimum(gap, rs[:, keep - 1] - rs[:, keep])
    return gap


def router_gaps(cfg: dict, w: dict, tokens) -> np.ndarray:
    """Per position the smallest routing gap over the model's layer runs (inf without experts)."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    gap = np.full(len(tokens), np.inf)
    for li in layer_order(cfg):
        spec, lw = cfg["layers"][li], sub(w, f"l{li}")
        mlp = spec.get("mlp")
        if mlp is not None and mlp["kind"] == "moe":
            gap = np.minimum(gap, route_gap(layer_norm(x, lw["norm2"], eps), sub(lw, "mlp"), mlp["router"]))
        x = run_layer(x, lw, spec, eps)
    return gap
