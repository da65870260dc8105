"""Typed configuration of the Vumezen decoder, read from its own config.json keys.

    architecture   "Vumezen"
    vocab, width   vocabulary and stream width
    embedding      {scale, bigram: {buckets, mul_prev, mul_cur} (optional)}
    norm           {eps}
    layers         list of {type: "attention", mixer: {...}, mlp: {...} or null}
      mixer        heads, kv_heads, dim (query/key head size), vdim (value head size), scale,
                   rot: {dims, base}, mask: {size, keep_first}, kv_from (optional: an earlier layer whose keys
                   and values this layer reads instead of projecting its own)
      mlp          {kind: "moe", router: {experts, top, scale}, expert: {ff}, shared: {ff} (optional)}

Tensor names: embed, bigram, l<i>.norm1, l<i>.norm2, l<i>.mix.{q,k,v,o}, l<i>.mlp.{router, correction, e<j>.up,
e<j>.down, shared.up, shared.down}, final.norm, head.

A layer is `parallel_residual`: its mixer and its feed-forward read the same stream, each behind a norm of its own.
The configuration names no longest sequence; MAX_POSITIONS below is this library's own bound (it sizes the rotation
tables of a model whose every layer keeps a window only; otherwise the cache's room is the smaller bound).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .registry import register_architecture
from .spec import CallSpec, ConfigError, LayerSpec, ModelSpec, PartSpec, SubLayerSpec

MAX_POSITIONS = 1 << 18


def _int(d: dict, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"{where}: key {key!r} must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"{where}: key {key!r} must be at least {minimum}, got {v}")
    return v


def _float(d: dict, key: str, where: str, positive: bool = True) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"{where}: key {key!r} must be a number, got {v!r}")
    if positive and v <= 0:
        raise ConfigError(f"{where}: key {key!r} must be positive, got {v}")
    return float(v)


def _dict(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: key {key!r} must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class VumezenMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    window: int
    keep_first: int
    kv_from: Optional[int]


@dataclass(frozen=True)
class VumezenMoE:
    experts: int
    top: int
    route_scale: float
    expert_ff: int
    shared_ff: Optional[int]


@register_architecture("Vumezen")
@dataclass(frozen=True)
class VumezenConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    bigram: Optional[Tuple[int, int, int]]            # (buckets, mul_prev, mul_cur)
    mixers: Tuple[VumezenMixer, ...]
    mlps: Tuple[Optional[VumezenMoE], ...]
    raw: Any = None                                    # the dict it was read from (for to_dict)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "VumezenConfig":
        vocab, width = _int(d, "vocab", "config"), _int(d, "width", "config")
        eps = _float(_dict(d, "norm", "config"), "eps", "norm")
        emb = _dict(d, "embedding", "config")
        embed_scale = _float(emb, "scale", "embedding", positive=False) if "scale" in emb else 1.0
        bigram = None
        if emb.get("bigram") is not None:
            b = _dict(emb, "bigram", "embedding")
            bigram = (_int(b, "buckets", "embedding.bigram"), _int(b, "mul_prev", "embedding.bigram", 0),
                      _int(b, "mul_cur", "embedding.bigram", 0))
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config: 'layers' must be a non-empty list")
        mixers, mlps = [], []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") != "attention":
                raise ConfigError(f"{where}: the only mixer of this architecture is 'attention', got {layer.get('type')!r}"
                                  if isinstance(layer, dict) else f"{where} must be an object")
            m = _dict(layer, "mixer", where)
            rot = m.get("rot")
            rot_dims, rot_base = 0, 1.0
            if rot is not None:
                rot = _dict(m, "rot", where)
                rot_dims, rot_base = _int(rot, "dims", f"{where}.rot", 0), _float(rot, "base", f"{where}.rot")
            mask = _dict(m, "mask", where)
            kv_from = m.get("kv_from")
            mx = VumezenMixer(
                heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where), dim=_int(m, "dim", where),
                vdim=_int(m, "vdim", where), scale=_float(m, "scale", where, positive=False), rot_dims=rot_dims, rot_base=rot_base,
                window=_int(mask, "size", f"{where}.mask"), keep_first=_int(mask, "keep_first", f"{where}.mask", 0) if "keep_first" in mask else 0,
                kv_from=None if kv_from is None else _int(m, "kv_from", where, 0))
            if mx.heads % mx.kv_heads:
                raise ConfigError(f"{where}: {mx.heads} heads cannot share {mx.kv_heads} kv_heads")
            if mx.rot_dims % 2 or mx.rot_dims > mx.dim:
                raise ConfigError(f"{where}: rot.dims={mx.rot_dims} must be even and at most dim={mx.dim}")
            if mx.kv_from is not None:
                if mx.kv_from >= i:
                    raise ConfigError(f"{where}: kv_from={mx.kv_from} must name an earlier layer")
                o = mixers[mx.kv_from]
                if o.kv_from is not None:
                    raise ConfigError(f"{where}: kv_from={mx.kv_from} names a layer that has no keys and values of its own")
                if (o.kv_heads, o.dim, o.vdim) != (mx.kv_heads, mx.dim, mx.vdim):
                    raise ConfigError(f"{where}: its key/value heads differ from those of layer {mx.kv_from}, whose cache it reads")
            mixers.append(mx)
            mlp = layer.get("mlp")
            if mlp is None:
                mlps.append(None)
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                raise ConfigError(f"{where}.mlp: the only feed-forward of this architecture is kind 'moe'")
            r = _dict(mlp, "router", f"{where}.mlp")
            shared = mlp.get("shared")
            moe = VumezenMoE(experts=_int(r, "experts", f"{where}.mlp.router"), top=_int(r, "top", f"{where}.mlp.router"),
                             route_scale=_float(r, "scale", f"{where}.mlp.router", positive=False) if "scale" in r else 1.0,
                             expert_ff=_int(_dict(mlp, "expert", f"{where}.mlp"), "ff", f"{where}.mlp.expert"),
                             shared_ff=None if shared is None else _int(_dict(mlp, "shared", f"{where}.mlp"), "ff", f"{where}.mlp.shared"))
            if moe.top > moe.experts:
                raise ConfigError(f"{where}.mlp.router: top={moe.top} exceeds experts={moe.experts}")
            mlps.append(moe)
        return cls(vocab=vocab, width=width, eps=eps, embed_scale=embed_scale, bigram=bigram, mixers=tuple(mixers),
                   mlps=tuple(mlps), raw=copy.deepcopy(d))

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)

    # ------------------------------------------------------------------ derived
    def readers(self, layer: int) -> Tuple[int, ...]:
        """Layers that read layer `layer`'s keys and values."""
        return tuple(i for i, m in enumerate(self.mixers) if m.kv_from == layer)

    def to_spec(self) -> ModelSpec:
        D = self.width
        norm = {"size": D, "eps": self.eps, "tensor": ""}
        layers = []
        for i, (m, moe) in enumerate(zip(self.mixers, self.mlps)):
            p = f"l{i}"
            # a cache other layers read keeps every key (their windows may differ); otherwise a ring for the window
            shared_cache = m.kv_from is not None or bool(self.readers(i))
            mixer = PartSpec("windowed_sink_attention", {
                "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim,
                "scale": m.scale, "window": min(m.window, MAX_POSITIONS), "keep_first": min(m.keep_first, MAX_POSITIONS),
                "sink": True, "own_kv": m.kv_from is None, "cache_window": None if shared_cache else min(m.window, MAX_POSITIONS),
                "position": PartSpec("rope_leading", {"head_dim": m.dim, "dims": m.rot_dims, "base": m.rot_base}),
            }, prefix=f"{p}.mix")
            subs = [SubLayerSpec("mixer", mixer, PartSpec("rms_norm", norm, prefix=f"{p}.norm1"))]
            if moe is not None:
                ffn = PartSpec("routed_experts", {
                    "hidden_size": D, "experts": moe.experts, "top": moe.top, "expert_ff": moe.expert_ff,
                    "route_scale": moe.route_scale, "act": "relu_squared", "shared_ff": moe.shared_ff, "use_bias": True,
                }, prefix=f"{p}.mlp")
                subs.append(SubLayerSpec("ffn", ffn, PartSpec("rms_norm", norm, prefix=f"{p}.norm2")))
            layers.append(LayerSpec("parallel_residual", tuple(subs)))
        pair = None
        if self.bigram is not None:
            pair = {"tensor": "bigram", "buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D, max_positions=MAX_POSITIONS,
            embedding=PartSpec("scaled_pair_embedding", {"vocab_size": self.vocab, "hidden_size": D, "scale": self.embed_scale,
                                                         "tensor": "embed", "pair": pair}),
            layers=tuple(layers),
            order=tuple(CallSpec(layer=i, cache_of=m.kv_from) for i, m in enumerate(self.mixers)),
            final_norm=PartSpec("rms_norm", norm, prefix="final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": D, "tied_to": None, "tensor": ""}, prefix="head"),
            stop_token_ids=())
