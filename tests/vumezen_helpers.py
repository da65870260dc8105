"""Shared by the Vumezen tests: small configurations that differ from one another in every size and option, model
folders with seeded weights shaped so that a fault shows, and the plain oracle's logits."""
from __future__ import annotations

import copy
import math
from pathlib import Path

import numpy as np
import torch

import plain_qwen2
import plain_vumezen as plain


def layer(heads, kv_heads, dim, vdim, rot_dims, window, keep_first, kv_from=None, moe=None, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
         "rot": {"dims": rot_dims, "base": base}, "mask": {"size": window, "keep_first": keep_first}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": moe}


def moe(experts, top, ff, shared_ff=None, scale=1.0):
    d = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff}}
    if shared_ff:
        d["shared"] = {"ff": shared_ff}
    return d


def config(vocab, width, layers, scale=1.0, bigram=None, eps=1e-5):
    emb = {"scale": scale}
    if bigram:
        emb["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    return {"architecture": "Vumezen", "vocab": vocab, "width": width, "embedding": emb, "norm": {"eps": eps}, "layers": layers}


# P: keys and values of different widths, a window of 70 keys with 3 kept ones (ring of 3 pages behind a pinned one), a
#    layer that reads an earlier layer's cache through a window of its own, partial rotation, sparse routing.
# Q: every head a key/value head, whole heads rotated, one expert per token, no shared expert, no pair table, a window
#    no request fills, nothing kept, sizes that are no multiples of 8 (the CUDA-core products).
# R: one key/value head, nothing rotated in two layers, 66 kept keys (two pinned pages) with a window of 9 in a layer
#    without a feed-forward, every expert chosen (the routing that 16-bit rounding cannot flip).
CONFIGS = {
    "P": config(211, 64, [
        layer(4, 2, 16, 24, 8, 70, 3, moe=moe(6, 2, 40, 24, scale=1.25)),
        layer(4, 2, 16, 24, 8, 33, 5, kv_from=0, moe=moe(6, 2, 40, 24, scale=1.25)),
        layer(2, 1, 32, 16, 32, 70, 3, moe=moe(5, 3, 24, 48, scale=0.7), base=250000.0),
    ], scale=3.5, bigram=(97, 7, 13)),
    "Q": config(150, 44, [
        layer(3, 3, 18, 18, 18, 1000, 0, moe=moe(4, 1, 20)),
        layer(3, 3, 18, 18, 18, 20, 0, kv_from=0, moe=moe(3, 1, 28, 12)),
    ], scale=1.0, eps=1e-6),
    "R": config(97, 48, [
        layer(6, 1, 16, 16, 0, 130, 1, moe=moe(3, 3, 32, 16, scale=2.0)),
        layer(2, 1, 48, 32, 16, 9, 66),
        layer(6, 1, 16, 16, 0, 64, 64, kv_from=0, moe=moe(2, 2, 16)),
    ], scale=0.37, bigram=(31, 1000003, 999983)),
}
DENSE_ROUTING = {"R"}          # every expert chosen: the choice cannot depend on rounding

GAIN = {torch.float32: 12.0, torch.bfloat16: 5.0}


def make_folder(tmp, cfg: dict, seed: int, attn_gain: float, store="bfloat16") -> Path:
    """Seeded random weights, then: query and key projections scaled by attn_gain (scores spread out, so a lost or
    misplaced key shows); router matrices scaled so that gates leave 1/2 and differ between tokens; choice
    corrections spread over +-0.3 (the chosen experts are not simply those with the largest gates); value, output and
    expert matrices scaled so that the mixer's and the feed-forward's shares of the stream are comparable."""
    from llaisys_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    folder = write_random_model(Path(tmp), cfg, seed, store)
    f = SafetensorsFile(folder / "model.safetensors")
    rng = np.random.default_rng(seed + 1)
    out = {}
    for name in f.entries:
        t = f.get(name).clone()
        if name.endswith(".mix.q") or name.endswith(".mix.k"):
            t = (t.float() * attn_gain).to(t.dtype)
        elif name.endswith(".router"):
            t = (t.float() * 25.0).to(t.dtype)
        elif name.endswith(".correction"):
            t = torch.from_numpy(rng.uniform(-0.3, 0.3, size=tuple(t.shape))).to(t.dtype)
        elif name.endswith(".mix.v") or name.endswith(".mix.o"):
            t = (t.float() * 7.0).to(t.dtype)
        elif name.endswith(".up") or name.endswith(".down"):
            t = (t.float() * 3.5).to(t.dtype)
        out[name] = t
    write_safetensors(folder / "model.safetensors", out)
    return folder


class Oracle:
    """Plain logits of whole requests, computed once per request."""

    def __init__(self, folder):
        import json
        self.config = json.loads((Path(folder) / "config.json").read_text())
        self.weights = plain_qwen2.read_safetensors(Path(folder) / "model.safetensors")
        self._memo = {}

    def logits(self, tokens) -> np.ndarray:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward(list(tokens), self.config, self.weights)
        return self._memo[key]


def like_config(cfg: dict) -> dict:
    """What helpers.tolerance reads."""
    return {"num_hidden_layers": len(cfg["layers"])}


def random_requests(cfg: dict, lengths, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]


def variant(cfg: dict, edit) -> dict:
    c = copy.deepcopy(cfg)
    edit(c)
    return c
