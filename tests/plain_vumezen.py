"""Plain, slow Vumezen decoder: the oracle the engine is compared with.

Whole sequences, no cache, one function per mechanism, float64 numpy throughout.  Nothing
here imports the product package (the safetensors reader is plain_qwen2's own).

The design, in this file's notation (T tokens, width D):

  embedding   x_t = E[id_t] * c + B[r_t],  r_t = (id_{t-1} a + id_t b) mod n for t > 0, r_0 = n
  layer       x <- x + mixer(rms(x) w1) + ffn(rms(x) w2)       (both branches read the same x)
  mixer       grouped-query attention: rotation of the first R dimensions of every query and key
              head (pairs (i, i + R/2), angle t * base^(-2i/R)); key j is visible from query i when
              j <= i and (i - j < W or j < F); weights e^{s_j} / (1 + sum_j e^{s_j}); a mixer may
              take the rotated keys and the values of an earlier layer instead of projecting its own
  ffn         routed experts: g = sigmoid(Wr h); the `top` largest of g + bias are chosen; the
              output is sum over the chosen of (g_e * router_scale) * expert_e(h), plus a shared
              expert that every token uses; an expert is Wd relu(Wu h)^2
  output      logits = Wh (rms(x) wf)
"""
from __future__ import annotations

import numpy as np


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


def hashed_pair_rows(ids, mul_prev, mul_cur, buckets):
    """Row of the pair table for every token: the hash of (previous id, id); the first token of a
    sequence has no previous one and takes the extra last row."""
    ids = np.asarray(ids, dtype=np.int64)
    rows = np.empty(len(ids), dtype=np.int64)
    rows[0] = buckets
    rows[1:] = (ids[:-1] * mul_prev + ids[1:] * mul_cur) % buckets
    return rows


def embed(ids, table, scale, pair_table=None, pair=None):
    x = table[np.asarray(ids, dtype=np.int64)] * scale
    if pair_table is not None:
        x = x + pair_table[hashed_pair_rows(ids, pair["mul_prev"], pair["mul_cur"], pair["buckets"])]
    return x


def rotate_leading(x, positions, dims, base):
    """x [T, heads, d]: the first `dims` dimensions are rotated in pairs (i, i + dims/2); the rest pass."""
    half = dims // 2
    out = x.copy()
    if half == 0:
        return out
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def visible(n, window, keep_first):
    """[n, n] boolean: query i (row) sees key j (column)."""
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    return (j <= i) & ((i - j < window) | (j < keep_first))


def sink_softmax(scores, mask):
    """Rows of exp(s) / (1 + sum exp(s)) over the visible keys: one more, value-less term of score 0."""
    s = np.where(mask, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), 0.0)
    e = np.where(mask, np.exp(s - m), 0.0)
    return e / (np.exp(-m) + e.sum(axis=-1, keepdims=True))


def attention_keys_values(h, w, p, positions):
    """Rotated keys [T, G, d] and values [T, G, dv] of a mixer that projects its own."""
    T = h.shape[0]
    k = (h @ w["k"].T).reshape(T, p["kv_heads"], p["dim"])
    v = (h @ w["v"].T).reshape(T, p["kv_heads"], p["vdim"])
    return rotate_leading(k, positions, p["rot"]["dims"], p["rot"]["base"]), v


def attention(h, w, p, positions, k, v):
    T = h.shape[0]
    H, G = p["heads"], p["kv_heads"]
    q = rotate_leading((h @ w["q"].T).reshape(T, H, p["dim"]), positions, p["rot"]["dims"], p["rot"]["base"])
    mask = visible(T, p["mask"]["size"], p["mask"]["keep_first"])
    out = np.empty((T, H, p["vdim"]))
    for head in range(H):
        g = head // (H // G)
        prob = sink_softmax((q[:, head] @ k[:, g].T) * p["scale"], mask)
        out[:, head] = prob @ v[:, g]
    return out.reshape(T, -1) @ w["o"].T


def expert(h, up, down):
    a = np.maximum(h @ up.T, 0.0)
    return (a * a) @ down.T


def routed_experts(h, w, p):
    r = p["router"]
    gate = 1.0 / (1.0 + np.exp(-(h @ w["router"].T)))
    choice = gate + w["correction"]
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]))
    for t in range(h.shape[0]):
        chosen = np.argsort(-choice[t], kind="stable")[:r["top"]]
        for e in chosen:
            out[t] += gate[t, e] * r["scale"] * expert(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if p.get("shared"):
        out += expert(h, w["shared.up"], w["shared.down"])
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(tokens, config, weights, want_layers=False):
    """float64 logits [T, vocab] of one whole sequence (and the stream after every layer)."""
    T = len(tokens)
    positions = np.arange(T)
    emb = config["embedding"]
    x = embed(tokens, weights["embed"], emb.get("scale", 1.0), weights.get("bigram"), emb.get("bigram"))
    eps = config["norm"]["eps"]
    kept, streams = {}, []
    for i, layer in enumerate(config["layers"]):
        assert layer["type"] == "attention"
        p = layer["mixer"]
        w = sub(weights, f"l{i}.mix.")
        h = rms_norm(x, weights[f"l{i}.norm1"], eps)
        if p.get("kv_from") is None:
            kept[i] = attention_keys_values(h, w, p, positions)
            k, v = kept[i]
        else:
            k, v = kept[p["kv_from"]]
        delta = attention(h, w, p, positions, k, v)
        if layer.get("mlp"):
            delta = delta + routed_experts(rms_norm(x, weights[f"l{i}.norm2"], eps), sub(weights, f"l{i}.mlp."), layer["mlp"])
        x = x + delta
        streams.append(x.copy())
    logits = rms_norm(x, weights["final.norm"], eps) @ weights["head"].T
    return (logits, np.stack(streams)) if want_layers else logits
