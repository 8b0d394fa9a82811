"""A plain, slow implementation of the Kisilix decoder, for tests only.

Whole sequences, no cache, no batching, one function per mechanism, numpy in double precision.
It shares no code with the library.

The design in this file's notation.  x[t] = E[token_t] + P[t] (a learned vector per position).  A layer
runs its sublayers on the stream itself and norms after each sum:
    x <- LN1(alpha x + mixer(x)),   x <- LN2(alpha x + ff(x))      (the second only with a feed-forward)
with LN(x) = (x - mean) / sqrt(var + eps) * w + b.  Mixers:

* channel_delta: a delta rule whose state decays per key channel.  q, k (kv_heads x dim) and v (heads x vdim)
  go through a short causal convolution per channel and silu; q and k become unit vectors per head (q also
  times dim^-1/2); beta = sigmoid(W_b x) per head; decay g = exp(-exp(A_log) softplus(W_a2 W_a1 x + dt_bias))
  per head and key channel; per head S <- diag(g) S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q; o is
  divided by its root mean square per head, times a weight over vdim, times sigmoid(W_g2 W_g1 x); W_o.
* mamba2: W_in x = [z | x | B | C | dt]; x, B, C through a causal convolution with bias and silu;
  dt = softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x; y silu(z) is
  RMS-normed in equal parts, times a weight; W_o.
* attention: q, k, v with biases; RMS norm with a weight on every q and k head; rotation of the first
  rot.dims numbers of q and k heads (pairs i, i + dims/2); the value of position j rotated by j over all of
  vdim (pairs m, m + vdim/2) and the head's result rotated back by the query's position; scores times a
  scale times a number per head; position i sees the last `size` positions and, for every block of `pool`
  positions that ended `size` or more positions ago, the mean of its keys and the mean of its (rotated)
  values; one softmax over both; W_o.

Feed-forwards: dense D (g sigmoid(1.702 g) (u + 1)) with g = min(G x, L), u = clamp(U x, -L, L); or experts
D_e (silu(G_e x) * U_e x) chosen by a softmax router with a correction that only chooses, limited to the best
groups of neighbouring experts, weighted by their softmax scores over the sum of the chosen, plus a shared expert.
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


def softplus(z):
    return np.logaddexp(0.0, z)


def layer_norm(x, w, b, eps):
    m = x.mean(-1, keepdims=True)
    d = x - m
    return d / np.sqrt((d * d).mean(-1, keepdims=True) + eps) * w + b


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def causal_conv(u, taps, bias=None):
    """u [T, C], taps [C, K] with the last column on the current row; zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), u], axis=0)
    y = np.zeros((T, C))
    for j in range(K):
        y += padded[j: j + T] * taps[:, j]
    return y if bias is None else y + bias


# ---- mixers -----------------------------------------------------------------------------------------
def channel_delta(x, w, m, eps):
    """`w`: the mixer's tensors by their short names; `m`: its sizes."""
    T = x.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(x @ w["q"].T, w["q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(x @ w["k"].T, w["k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(x @ w["v"].T, w["v.conv"])).reshape(T, H, e)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(x @ w["b"].T)                                                    # [T, H]
    step = softplus((x @ w["a1"].T) @ w["a2"].T + w["dt_bias"]).reshape(T, H, d)
    g = np.exp(-np.exp(w["A_log"])[None, :, None] * step)                            # [T, H, d]
    S = np.zeros((H, d, e))
    o = np.zeros((T, H, e))
    for t in range(T):
        for h in range(H):
            kh, qh = k[t, h // (H // G)], q[t, h // (H // G)]
            S[h] = g[t, h][:, None] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ kh)
            S[h] = S[h] + np.outer(kh, u)
            o[t, h] = S[h].T @ qh
    gate = sigmoid((x @ w["g1"].T) @ w["g2"].T).reshape(T, H, e)
    o = unit_rms(o, eps) * w["norm"] * gate
    return o.reshape(T, H * e) @ w["o"].T


def mamba2(x, w, m, eps):
    T = x.shape[0]
    H, e, N, G, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * e
    p = x @ w["in"].T
    z, xbc, dt = p[:, :inner], p[:, inner: 2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    xs = xbc[:, :inner].reshape(T, H, e)
    B = xbc[:, inner: inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"])                                                # [T, H]
    decay = np.exp(-np.exp(w["A_log"]) * dt)
    S = np.zeros((H, N, e))
    y = np.zeros((T, H, e))
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = decay[t, h] * S[h] + dt[t, h] * np.outer(B[t, g], xs[t, h])
            y[t, h] = S[h].T @ C[t, g] + w["D"][h] * xs[t, h]
    y = y.reshape(T, inner) * silu(z)
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


def rotate_halves(x, pos, base, dims):
    """The first `dims` numbers of the last axis, pairs (i, i + dims/2), turned by pos * base^(-2i/dims);
    x [T, heads, n], pos [T] (may be negative: turns back).  Angles are formed in 32-bit."""
    half = dims // 2
    f = (np.float32(base) ** (-2.0 * np.arange(half, dtype=np.float64) / dims)).astype(np.float32)
    a = (pos.astype(np.float32)[:, None] * f[None, :]).astype(np.float64)             # [T, half]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def pooled_window_attention(x, w, m, eps):
    T = x.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, P = m["mask"]["size"], m["mask"]["pool"]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    pos = np.arange(T)
    q = (x @ w["q"].T + w["q.b"]).reshape(T, H, d)
    k = (x @ w["k"].T + w["k.b"]).reshape(T, G, d)
    v = (x @ w["v"].T + w["v.b"]).reshape(T, G, e)
    q = unit_rms(q, eps) * w["q.norm"]
    k = unit_rms(k, eps) * w["k.norm"]
    if dims:
        q, k = rotate_halves(q, pos, base, dims), rotate_halves(k, pos, base, dims)
    v = rotate_halves(v, pos, base, e)
    nblocks = T // P
    pk = k[: nblocks * P].reshape(nblocks, P, G, d).mean(1)
    pv = v[: nblocks * P].reshape(nblocks, P, G, e).mean(1)
    o = np.zeros((T, H, e))
    for i in range(T):
        lo = max(0, i - size + 1)
        nb = max(0, (i - size + 1) // P) if i - size + 1 >= 0 else 0
        for h in range(H):
            g = h // (H // G)
            keys = np.concatenate([pk[:nb, g], k[lo: i + 1, g]], axis=0)
            vals = np.concatenate([pv[:nb, g], v[lo: i + 1, g]], axis=0)
            s = keys @ q[i, h] * m["scale"] * w["temp"][h]
            s = np.exp(s - s.max())
            o[i, h] = (s / s.sum()) @ vals
    o = rotate_halves(o, -pos, base, e)
    return o.reshape(T, H * e) @ w["o"].T


MIXERS = {"channel_delta": channel_delta, "mamba2": mamba2, "attention": pooled_window_attention}


# ---- feed-forwards ------------------------------------------------------------------------------------
def clamped_dense(x, w, f):
    L = f["limit"]
    g = np.minimum(x @ w["gate"].T, L)
    u = np.clip(x @ w["up"].T, -L, L)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def silu_expert(x, gate, up, down):
    return (silu(x @ gate.T) * (x @ up.T)) @ down.T


def route(x, w, f):
    """(chosen experts [T, top], their weights [T, top], gap between the last chosen and the first rejected
    choice score [T])."""
    r = f["router"]
    E, top = r["experts"], r["top"]
    count, keep = (r["groups"]["count"], r["groups"]["keep"]) if r.get("groups") else (1, 1)
    z = x @ w["router"].T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    choice = s + w["correction"]
    T = x.shape[0]
    ids = np.zeros((T, top), dtype=np.int64)
    wts = np.zeros((T, top))
    gap = np.zeros(T)
    for t in range(T):
        c = choice[t].copy()
        gs = c.reshape(count, E // count).max(-1)
        kept = np.argsort(-gs, kind="stable")[:keep]
        allowed = np.zeros(count, dtype=bool)
        allowed[kept] = True
        c[~np.repeat(allowed, E // count)] = -np.inf
        order = np.argsort(-c, kind="stable")
        ids[t] = order[:top]
        wts[t] = s[t, ids[t]] / (s[t, ids[t]].sum() + 1e-20)
        gap[t] = c[order[top - 1]] - c[order[top]] if top < E else np.inf
        if keep < count:
            gso = np.sort(gs)[::-1]
            gap[t] = min(gap[t], gso[keep - 1] - gso[keep])
    return ids, wts, gap


def expert_mixture(x, w, f):
    ids, wts, _ = route(x, w, f)
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        for j, e in enumerate(ids[t]):
            y[t] += wts[t, j] * silu_expert(x[t: t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if f.get("shared"):
        y = y + silu_expert(x, w["shared.gate"], w["shared.up"], w["shared.down"])
    return y


def feed_forward(x, w, f):
    return clamped_dense(x, w, f) if f["kind"] == "dense" else expert_mixture(x, w, f)


# ---- the model ----------------------------------------------------------------------------------------
def sub(tensors, prefix):
    return {n[len(prefix):]: t for n, t in tensors.items() if n.startswith(prefix)}


def forward(cfg, tensors, tokens, want_layers=False):
    """Logits [T, vocab] of one sequence; with `want_layers` also the stream after every layer."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    tokens = np.asarray(tokens)
    x = tensors["embed"][tokens] + tensors["pos"][: len(tokens)]
    streams = []
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[lay["type"]](x, sub(tensors, p + "mix."), lay["mixer"], eps)
        x = layer_norm(alpha * x + y, tensors[p + "norm1"], tensors[p + "norm1.b"], eps)
        if lay.get("mlp"):
            y = feed_forward(x, sub(tensors, p + "mlp."), lay["mlp"])
            x = layer_norm(alpha * x + y, tensors[p + "norm2"], tensors[p + "norm2.b"], eps)
        streams.append(x.copy())
    x = layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], eps)
    logits = x @ tensors["head"].T
    return (logits, np.stack(streams)) if want_layers else logits


def router_gaps(cfg, tensors, tokens):
    """Per position, the smallest gap of any routed layer between the last chosen and the first rejected
    choice (positions where rounding may pick another expert)."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    tokens = np.asarray(tokens)
    x = tensors["embed"][tokens] + tensors["pos"][: len(tokens)]
    gaps = np.full(len(tokens), np.inf)
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[lay["type"]](x, sub(tensors, p + "mix."), lay["mixer"], eps)
        x = layer_norm(alpha * x + y, tensors[p + "norm1"], tensors[p + "norm1.b"], eps)
        if lay.get("mlp"):
            if lay["mlp"]["kind"] != "dense":
                gaps = np.minimum(gaps, route(x, sub(tensors, p + "mlp."), lay["mlp"])[2])
            y = feed_forward(x, sub(tensors, p + "mlp."), lay["mlp"])
            x = layer_norm(alpha * x + y, tensors[p + "norm2"], tensors[p + "norm2.b"], eps)
    return gaps
