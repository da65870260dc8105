"""Shared by the Nubedra tests: small configurations that differ from one another in every size and option, model folders
with seeded weights shaped so that a fault shows, and the plain oracle's logits."""
from __future__ import annotations

import copy
import json
from pathlib import Path

import numpy as np
import torch

import plain_nubedra as plain
import plain_qwen2


def gla(heads, dim, vdim, tau, ff=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, ff=None, kv_from=None, base=10000.0, scaling=None, scale=None,
           rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "mask": {"size": window},
         "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(vocab, width, layers, embed_scale=1.0, mult=1.0, eps=1e-5):
    return {"architecture": "Nubedra", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale}, "norm": {"eps": eps},
            "residual_mult": mult, "layers": layers}


YARN_A = (4.0, 64, 16.0, 2.0)
YARN_B = (1.5, 512, 40.0, 0.5)

# P: a recurrent layer without feed-forward first, a latent layer whose cache the next one reads through a narrower window
#    (the cache keeps every row), a recurrent layer with feed-forward last; rescaled rotation; all head sizes differ.
# Q: sizes that are no multiples of 8 (the CUDA-core products), latent layers with rings of their own (a window of 20 that
#    every request passes, one of 1000 that none fills), part of the rotated part left unrotated, no rescaling, a
#    recurrent head of 33 value channels (two blocks of columns) with a decay root of 1, constants equal to 1.
# R: cache rows wider than 256 elements, a window of 9, a reader with a window wider than its source's, a recurrent head
#    of 130 key channels, several layers without feed-forward.
CONFIGS = {
    "P": config(211, 64, [
        gla(3, 20, 8, 4.0),
        latent(3, 16, 8, 24, 48, 40, 70, ff=96, scaling=YARN_A, base=5000.0),
        latent(2, 24, 8, 12, 32, 40, 33, ff=80, kv_from=1, scaling=YARN_A, base=5000.0, scale=0.3),
        gla(2, 12, 40, 9.0, ff=56),
    ], embed_scale=3.5, mult=0.6),
    "Q": config(150, 44, [
        latent(2, 6, 10, 14, 22, 18, 20, ff=52, rot_dims=6),
        gla(1, 18, 33, 1.0, ff=36),
        latent(5, 4, 2, 3, 9, 7, 1000, scaling=YARN_B, base=300.0),
    ], embed_scale=1.0, mult=1.0, eps=1e-6),
    "R": config(97, 48, [
        latent(2, 8, 8, 8, 16, 264, 9, scaling=YARN_B),
        gla(1, 130, 4, 30.0),
        latent(6, 16, 8, 16, 24, 264, 130, ff=64, kv_from=0, scaling=YARN_B),
    ], embed_scale=0.37, mult=1.4),
}

GAIN = {torch.float32: 9.0, torch.bfloat16: 3.0}


def make_folder(tmp, cfg: dict, seed: int, gain: float, store="bfloat16") -> Path:
    """Seeded random weights, then: the matrices that make queries and keys scaled by `gain` (scores spread out, so a lost
    or misplaced key shows); sinks spread over +-3; decay biases spread so that channels forget at different speeds and the
    decay's bottleneck scaled so that they differ between tokens; gates scaled away from 1/2; the norms' stored weights
    spread over +-0.5 (an offset left out or applied twice shows)."""
    from llaisys_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    folder = write_random_model(Path(tmp), cfg, seed, store)
    f = SafetensorsFile(folder / "model.safetensors")
    rng = np.random.default_rng(seed + 1)
    out = {}
    for name in f.entries:
        t = f.get(name).clone()
        leaf = name.split(".mix.")[-1] if ".mix." in name else name.rsplit(".", 1)[-1]
        gla_layer = name.startswith("l") and cfg["layers"][int(name[1:name.index(".")])]["type"] == "gla"
        if ".mix." in name and leaf in ("uq", "uk"):
            t = (t.float() * gain).to(t.dtype)
        elif ".mix." in name and leaf == "dkv":
            t = t.float()
            rot = cfg["layers"][int(name[1:name.index(".")])]["mixer"]["rot_dim"]
            t[-rot:] *= gain * 2.0
            t = t.to(f.get(name).dtype)
        elif ".mix." in name and leaf == "sink":
            t = torch.from_numpy(rng.uniform(-3, 3, size=tuple(t.shape))).to(t.dtype)
        elif ".mix." in name and leaf == "a2.b":
            t = torch.from_numpy(rng.uniform(-1, 5, size=tuple(t.shape))).to(t.dtype)
        elif ".mix." in name and leaf in ("a1", "a2"):
            t = (t.float() * 12.0).to(t.dtype)
        elif ".mix." in name and leaf == "g":
            t = (t.float() * (10.0 if not gla_layer else 6.0)).to(t.dtype)
        elif gla_layer and ".mix." in name and leaf in ("q", "k", "v"):
            t = (t.float() * 6.0).to(t.dtype)
        elif ".mlp." in name:
            t = (t.float() * 5.0).to(t.dtype)
        elif leaf.startswith("norm") and ".mix." not in name:
            t = torch.from_numpy(rng.uniform(-0.5, 0.5, size=tuple(t.shape))).to(t.dtype)
        out[name] = t
    write_safetensors(folder / "model.safetensors", out)
    return folder


class Oracle:
    """Plain logits of whole requests, computed once per request."""

    def __init__(self, folder):
        self.config = json.loads((Path(folder) / "config.json").read_text())
        self.weights = plain_qwen2.read_safetensors(Path(folder) / "model.safetensors")
        self._memo = {}

    def logits(self, tokens) -> np.ndarray:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward(self.config, self.weights, list(tokens))
        return self._memo[key]


def like_config(cfg: dict) -> dict:
    """What helpers.tolerance reads.  Its bfloat16 bound counts six roundings to 16 bits a layer; a layer of this design
    has about twice as many (the fused down projections, the query latent, the queries, the queries in the latent space,
    the cached row, the latent result, the gated heads; the normed input, the two halves and their product in the
    feed-forward), so a layer counts twice."""
    return {"num_hidden_layers": 2 * len(cfg["layers"])}


def random_requests(cfg: dict, lengths, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]


def variant(cfg: dict, edit) -> dict:
    c = copy.deepcopy(cfg)
    edit(c)
    return c


def compare(got, oracle, requests, dtype, cfg, what=""):
    """float32: every logits row within the absolute bound of helpers.tolerance.  bfloat16: the recurrent layer's output
    o = S^T q is a sum with cancellation that a norm then scales to unit size, so where o happens to be small the
    rounding of q, k and v to 16 bits is magnified: the error has a heavy tail over positions (more so with few value
    channels) that no fault causes.  A fault (a lost key, a stale state) moves whole ranges of positions by far more
    than the bound.  So: no row beyond eight bounds, and at most one row in ten beyond one."""
    import helpers
    like = like_config(cfg)
    if dtype == torch.float32:
        return helpers.compare(got, oracle, requests, dtype, like, what)
    ratios = []
    for r, toks in enumerate(requests):
        ref = oracle.logits(toks)
        tol = helpers.tolerance(dtype, like, ref)
        for p in range(len(toks)):
            assert (r, p) in got, f"{what}: no logits for request {r} position {p}"
            err = float(np.abs(got[(r, p)].astype(np.float64) - ref[p]).max())
            assert np.isfinite(err), f"{what}: non-finite logits at request {r} position {p}"
            ratios.append((err / tol, r, p))
    worst = max(ratios)
    over = sum(1 for x in ratios if x[0] > 1.0)
    assert worst[0] <= 8.0, f"{what}: request {worst[1]} position {worst[2]} is {worst[0]:.1f} bounds off"
    assert over <= max(1, len(ratios) // 10), f"{what}: {over} of {len(ratios)} rows are beyond the bound (worst {worst[0]:.1f} at {worst[1:]})"
    return worst[0], worst[1:]
