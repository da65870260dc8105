"""A plain, slow implementation of the Nubedra decoder in float64 numpy: one function per mechanism, whole
sequences, no cache, no state carried between calls, and no code shared with the package.

Notation: T tokens, stream width D, x [T, D] the residual stream, h the normed input of a mixer or feed-forward.
Weights come as a dict name -> array with the names of the weights file; matrices are [out, in].
"""
from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def norm_plain(x, w, eps):
    return rms(x, eps) * np.asarray(w, dtype=np.float64)


def norm_offset(x, w, eps):
    """The layers' norm: the stored weight is the distance from one."""
    return rms(x, eps) * (1.0 + np.asarray(w, dtype=np.float64))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


# ---------------------------------------------------------------------------------------------- rotation
def yarn_frequencies(dims, base, scaling):
    """Frequencies f_i (i < dims/2) and the factor both cos and sin are multiplied by."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, dims, base, scaling):
    """Rotates the pairs (2i, 2i+1), i < dims/2, of the last axis of x [T, ..., n >= dims]; the rest passes."""
    f, mag = yarn_frequencies(dims, base, scaling)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    cos, sin = np.cos(ang) * mag, np.sin(ang) * mag
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (dims // 2,)
    cos, sin = cos.reshape(shape), sin.reshape(shape)
    out = np.array(x, dtype=np.float64)
    u, v = out[..., 0:dims:2].copy(), out[..., 1:dims:2].copy()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ---------------------------------------------------------------------------------------------- mixers
def gla_mixer(h, w, p, mix, eps, state=None):
    """Gated linear attention.  Returns (output [T, D], final state [heads, dim, vdim])."""
    H, dk, dv, tau = mix["heads"], mix["dim"], mix["vdim"], float(mix["tau"])
    T = h.shape[0]
    q = (h @ w[p + ".q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + ".k"].T).reshape(T, H, dk)
    v = (h @ w[p + ".v"].T).reshape(T, H, dv)
    z = (h @ w[p + ".a1"].T) @ w[p + ".a2"].T + w[p + ".a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(T, H, dk)
    S = np.zeros((H, dk, dv)) if state is None else np.array(state, dtype=np.float64)
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    o = norm_plain(o, w[p + ".norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ w[p + ".g"].T)) @ w[p + ".o"].T, S


def latent_kv(h, w, p, mix, eps, positions):
    """What a latent-attention layer with its own down projection keeps per token: (latent [T, kv_rank], rotated
    shared key part [T, rot_dim])."""
    r = mix["kv_rank"]
    d = h @ w[p + ".dkv"].T
    c = norm_plain(d[:, :r], w[p + ".dkv.norm"], eps)
    rot = mix["rot"]
    kr = rotate_interleaved(d[:, r:], positions, rot["dims"], rot["base"], rot.get("scaling"))
    return c, kr


def latent_attention_mixer(h, w, p, mix, eps, positions, kv):
    """Latent attention over kv = (latent, rotated key part) of all T positions (the layer's own or another's)."""
    H, dn, dr, dv = mix["heads"], mix["dim"], mix["rot_dim"], mix["vdim"]
    T = h.shape[0]
    c, kr = kv
    cq = norm_plain(h @ w[p + ".dq"].T, w[p + ".dq.norm"], eps)
    q = (cq @ w[p + ".uq"].T).reshape(T, H, dn + dr)
    rot = mix["rot"]
    qr = rotate_interleaved(q[:, :, dn:], positions, rot["dims"], rot["base"], rot.get("scaling"))
    kn = (c @ w[p + ".uk"].T).reshape(T, H, dn)
    val = (c @ w[p + ".uv"].T).reshape(T, H, dv)
    s = (np.einsum("thd,shd->hts", q[:, :, :dn], kn) + np.einsum("thd,sd->hts", qr, kr)) * float(mix["scale"])
    i, j = np.asarray(positions)[:, None], np.asarray(positions)[None, :]
    seen = j <= i
    if mix.get("mask") is not None:
        seen = seen & (i - j < int(mix["mask"]["size"]))
    s = np.where(seen[None], s, -np.inf)
    sink = np.asarray(w[p + ".sink"], dtype=np.float64)
    m = np.maximum(s.max(axis=-1), sink[:, None])
    e = np.exp(s - m[..., None])
    wgt = e / (e.sum(axis=-1) + np.exp(sink[:, None] - m))[..., None]
    o = np.einsum("hts,shv->thv", wgt, val)
    o = o * sigmoid(h @ w[p + ".g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + ".o"].T


def dense_ff(h, w, p):
    return (np.maximum(h @ w[p + ".gate"].T, 0.0) * (h @ w[p + ".up"].T)) @ w[p + ".down"].T


# ---------------------------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, collect=None):
    """Logits [T, vocab] of one whole sequence.  `collect`: a list that receives the stream after every layer."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    T = len(tokens)
    positions = np.arange(T)
    x = w["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, mix = f"l{i}", layer["mixer"]
        h = norm_offset(x, w[p + ".norm1"], eps)
        if layer["type"] == "gla":
            y, _ = gla_mixer(h, w, p + ".mix", mix, eps)
        elif layer["type"] == "latent_attention":
            src = mix.get("kv_from")
            if src is None:
                kept[i] = latent_kv(h, w, p + ".mix", mix, eps, positions)
            y = latent_attention_mixer(h, w, p + ".mix", mix, eps, positions, kept[i if src is None else src])
        else:
            raise ValueError(layer["type"])
        x = x + m * norm_offset(y, w[p + ".norm1b"], eps)
        if layer.get("mlp") is not None:
            y = dense_ff(norm_offset(x, w[p + ".norm2"], eps), w, p + ".mlp")
            x = x + m * norm_offset(y, w[p + ".norm2b"], eps)
        if collect is not None:
            collect.append(x.copy())
    return norm_offset(x, w["final.norm"], eps) @ w["embed"].T
