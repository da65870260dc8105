"""Typed configuration of the Nubedra decoder, read from its own config.json keys.

    architecture    "Nubedra"
    vocab, width    vocabulary and stream width
    embedding       {scale}
    norm            {eps}
    residual_mult   what a sub-layer's normed output is multiplied by before it joins the stream
    layers          list of {type: "gla" | "latent_attention", mixer: {...}, mlp: {kind: "dense", ff} or null}
      gla mixer     heads, dim (query/key channels of a head), vdim (value channels), tau (the decay's root)
      latent mixer  heads, dim (unrotated query/key part), rot_dim (rotated part, one key part shared by all heads), vdim,
                    q_rank, kv_rank (latent sizes), scale, rot: {dims, base, scaling: {factor, original, fast, slow}},
                    mask: {size}, kv_from (optional: an earlier latent layer whose cached latent and rotated key part
                    this layer reads instead of projecting its own)

Tensor names: embed, l<i>.norm1, norm1b, norm2, norm2b, l<i>.mix.*, l<i>.mlp.{gate, up, down}, final.norm; the output
head is the embedding table.  The size of the decay's bottleneck of a gla mixer stands in no key: it is the shape of
`mix.a1`.

A layer is `sandwich_residual`: x += m * norm_b(part(norm(x))) for the mixer and then for the feed-forward, every norm
an RMS norm whose stored weight is the distance from one.  The configuration names no longest sequence; MAX_POSITIONS
is this library's own bound.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .registry import register_architecture
from .spec import CallSpec, ConfigError, LayerSpec, ModelSpec, PartSpec, SubLayerSpec
from .vumezen import _dict, _float, _int

MAX_POSITIONS = 1 << 18


@dataclass(frozen=True)
class NubedraGLA:
    heads: int
    dim: int
    vdim: int
    tau: float


@dataclass(frozen=True)
class NubedraLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[Tuple[float, float, float, float]]      # (factor, original, fast, slow)
    window: Optional[int]
    kv_from: Optional[int]


def _latent(m: dict, where: str) -> NubedraLatent:
    rot = _dict(m, "rot", where)
    scaling = None
    if rot.get("scaling") is not None:
        s = _dict(rot, "scaling", f"{where}.rot")
        scaling = tuple(_float(s, k, f"{where}.rot.scaling") for k in ("factor", "original", "fast", "slow"))
    window = None
    if m.get("mask") is not None:
        window = _int(_dict(m, "mask", where), "size", f"{where}.mask")
    kv_from = m.get("kv_from")
    mx = NubedraLatent(
        heads=_int(m, "heads", where), dim=_int(m, "dim", where, 0), rot_dim=_int(m, "rot_dim", where, 0),
        vdim=_int(m, "vdim", where), q_rank=_int(m, "q_rank", where), kv_rank=_int(m, "kv_rank", where),
        scale=_float(m, "scale", where, positive=False), rot_dims=_int(rot, "dims", f"{where}.rot", 0),
        rot_base=_float(rot, "base", f"{where}.rot"), rot_scaling=scaling, window=window,
        kv_from=None if kv_from is None else _int(m, "kv_from", where, 0))
    if mx.rot_dims % 2 or mx.rot_dims > mx.rot_dim:
        raise ConfigError(f"{where}: rot.dims={mx.rot_dims} must be even and at most rot_dim={mx.rot_dim}")
    if mx.dim + mx.rot_dim == 0:
        raise ConfigError(f"{where}: a head needs query/key dimensions (dim + rot_dim > 0)")
    return mx


@register_architecture("Nubedra")
@dataclass(frozen=True)
class NubedraConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    residual_mult: float
    mixers: Tuple[Any, ...]                   # NubedraGLA or NubedraLatent per layer
    ffs: Tuple[Optional[int], ...]            # the dense feed-forward's inner width, or None
    raw: Any = None

    @classmethod
    def from_dict(cls, d: dict) -> "NubedraConfig":
        vocab, width = _int(d, "vocab", "config"), _int(d, "width", "config")
        eps = _float(_dict(d, "norm", "config"), "eps", "norm")
        emb = d.get("embedding") or {}
        embed_scale = _float(emb, "scale", "embedding", positive=False) if "scale" in emb else 1.0
        mult = _float(d, "residual_mult", "config", positive=False) if "residual_mult" in d else 1.0
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config: 'layers' must be a non-empty list")
        mixers, ffs = [], []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"{where} must be an object")
            m = _dict(layer, "mixer", where)
            kind = layer.get("type")
            if kind == "gla":
                mixers.append(NubedraGLA(heads=_int(m, "heads", where), dim=_int(m, "dim", where), vdim=_int(m, "vdim", where),
                                         tau=_float(m, "tau", where)))
            elif kind == "latent_attention":
                mx = _latent(m, where)
                if mx.kv_from is not None:
                    o = mixers[mx.kv_from] if mx.kv_from < i else None
                    if not isinstance(o, NubedraLatent) or o.kv_from is not None:
                        raise ConfigError(f"{where}: kv_from={mx.kv_from} must name an earlier latent_attention layer that "
                                          f"projects its own latent")
                    if (o.kv_rank, o.rot_dim, o.rot_dims, o.rot_base, o.rot_scaling) != (
                            mx.kv_rank, mx.rot_dim, mx.rot_dims, mx.rot_base, mx.rot_scaling):
                        raise ConfigError(f"{where}: its latent size or rotation differs from layer {mx.kv_from}'s, whose cache it reads")
                mixers.append(mx)
            else:
                raise ConfigError(f"{where}: the mixers of this architecture are 'gla' and 'latent_attention', got {kind!r}")
            mlp = layer.get("mlp")
            if mlp is None:
                ffs.append(None)
            elif isinstance(mlp, dict) and mlp.get("kind") == "dense":
                ffs.append(_int(mlp, "ff", f"{where}.mlp"))
            else:
                raise ConfigError(f"{where}.mlp: the only feed-forward of this architecture is kind 'dense'")
        return cls(vocab=vocab, width=width, eps=eps, embed_scale=embed_scale, residual_mult=mult, mixers=tuple(mixers),
                   ffs=tuple(ffs), raw=copy.deepcopy(d))

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)

    def readers(self, layer: int) -> Tuple[int, ...]:
        """Layers that read layer `layer`'s cache."""
        return tuple(i for i, m in enumerate(self.mixers) if isinstance(m, NubedraLatent) and m.kv_from == layer)

    def to_spec(self) -> ModelSpec:
        D = self.width
        norm = {"size": D, "eps": self.eps, "tensor": "", "offset": 1.0}
        layers = []
        for i, (m, ff) in enumerate(zip(self.mixers, self.ffs)):
            p = f"l{i}"
            if isinstance(m, NubedraGLA):
                mixer = PartSpec("gated_linear_attention", {
                    "hidden_size": D, "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "decay_root": m.tau,
                    "query_scale": m.dim ** -0.5, "eps": self.eps}, prefix=f"{p}.mix")
            else:
                # a cache that other layers read keeps every row (their windows may differ); otherwise a ring for the window
                shared = m.kv_from is not None or bool(self.readers(i))
                window = None if m.window is None else min(m.window, MAX_POSITIONS)
                mixer = PartSpec("latent_attention", {
                    "hidden_size": D, "num_heads": m.heads, "nope_dim": m.dim, "rope_dim": m.rot_dim, "value_dim": m.vdim,
                    "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "window": window, "eps": self.eps,
                    "sink": True, "head_gate": True, "own_kv": m.kv_from is None, "cache_window": None if shared else window,
                    "position": PartSpec("rope_interleaved", {
                        "width": m.rot_dim, "dims": m.rot_dims, "base": m.rot_base,
                        "yarn": None if m.rot_scaling is None else dict(zip(("factor", "original", "fast", "slow"), m.rot_scaling))}),
                }, prefix=f"{p}.mix")
            subs = [SubLayerSpec("mixer", mixer, PartSpec("rms_norm", norm, prefix=f"{p}.norm1"),
                                 PartSpec("rms_norm", norm, prefix=f"{p}.norm1b"))]
            if ff is not None:
                ffn = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": ff, "act": "relu",
                                             "names": {"gate": "gate", "up": "up", "down": "down"}}, prefix=f"{p}.mlp")
                subs.append(SubLayerSpec("ffn", ffn, PartSpec("rms_norm", norm, prefix=f"{p}.norm2"),
                                         PartSpec("rms_norm", norm, prefix=f"{p}.norm2b")))
            layers.append(LayerSpec("sandwich_residual", tuple(subs), {"mult": self.residual_mult}))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D, max_positions=MAX_POSITIONS,
            embedding=PartSpec("scaled_pair_embedding", {"vocab_size": self.vocab, "hidden_size": D, "scale": self.embed_scale,
                                                         "tensor": "embed", "pair": None}),
            layers=tuple(layers),
            order=tuple(CallSpec(layer=i, cache_of=getattr(m, "kv_from", None)) for i, m in enumerate(self.mixers)),
            final_norm=PartSpec("rms_norm", norm, prefix="final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": D, "tied_to": "embed", "tensor": ""}, prefix="head"),
            stop_token_ids=())
