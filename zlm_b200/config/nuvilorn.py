"""Typed configuration of the Nuvilorn architecture, read from its own ``config.json`` keys, and
its lowering to a ``ModelSpec``.

A Nuvilorn config.json names the design with a string (``"architecture": "Nuvilorn"``) and lists
its layers one by one, since layers of one model may differ in everything:

    {"architecture": "Nuvilorn", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale",
                           "rot": {"base", "dims"}, "kv_from": j (optional)},
                 "mlp": null
                      | {"kind": "dense", "ff": F}
                      | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k},
                         "shared": {"ff": S} (optional)}}, ...]}

The design: the embedding's rows pass through an RMS norm with a single gain (``embed.norm``); every
layer is pre-norm (``l<i>.norm1``, ``l<i>.norm2``, single gains too) around a latent-attention mixer
(``l<i>.mix.*``) and a feed-forward (``l<i>.mlp.*``): dense gated silu, or routed relu^2 experts with
sigmoid scores that scale the experts' inputs plus a gated shared expert; a last norm (``final.norm``)
and an untied head (``head``).  A mixer with ``kv_from`` = j has no down-projection of its own and reads
layer j's cached latents.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .spec import (ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, coerce, optional, require)

ARCHITECTURE = "Nuvilorn"
# the design sets no longest sequence; the cache an engine is built with does
NO_POSITION_LIMIT = 1 << 24


def _mapping(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "LatentMixerConfig":
        def req(m, key, typ):
            if key not in m or m[key] is None:
                raise ConfigError(f"config.json: {where}missing key '{key}'")
            return coerce(m[key], where + key, typ)
        rot = _mapping(d, "rot", where)
        kv_from = d.get("kv_from")
        c = cls(req(d, "heads", int), req(d, "dim", int), req(d, "rot_dim", int), req(d, "vdim", int),
                req(d, "kv_rank", int), req(d, "scale", float), req(rot, "base", float), req(rot, "dims", int),
                None if kv_from is None else coerce(kv_from, where + "kv_from", int))
        if min(c.heads, c.vdim, c.kv_rank) <= 0 or c.dim < 0 or c.rot_dim < 0 or c.dim + c.rot_dim <= 0:
            raise ConfigError(f"config.json: {where}sizes must be positive")
        if c.rot_dims % 2 or not 0 <= c.rot_dims <= c.rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims={c.rot_dims} must be even and at most rot_dim={c.rot_dim}")
        if c.rot_base <= 0:
            raise ConfigError(f"config.json: {where}rot.base must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                             "kv_rank": self.kv_rank, "scale": self.scale,
                             "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                    # "dense" | "moe"
    ff: int                      # dense: its width; moe: one expert's width
    experts: int = 0
    top: int = 0
    shared_ff: int = 0

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "FeedForwardConfig":
        kind = d.get("kind")
        if kind == "dense":
            c = cls("dense", coerce(d.get("ff"), where + "ff", int))
        elif kind == "moe":
            router, expert = _mapping(d, "router", where), _mapping(d, "expert", where)
            shared = d.get("shared")
            if shared is not None and not isinstance(shared, Mapping):
                raise ConfigError(f"config.json: {where}'shared' must be an object")
            c = cls("moe", coerce(expert.get("ff"), where + "expert.ff", int),
                    coerce(router.get("experts"), where + "router.experts", int),
                    coerce(router.get("top"), where + "router.top", int),
                    coerce(shared.get("ff"), where + "shared.ff", int) if shared is not None else 0)
            if not 0 < c.top <= c.experts:
                raise ConfigError(f"config.json: {where}router.top={c.top} of {c.experts} experts")
            if c.shared_ff < 0:
                raise ConfigError(f"config.json: {where}shared.ff must not be negative")
        else:
            raise ConfigError(f"config.json: {where}kind={kind!r} is not known (dense, moe)")
        if c.ff <= 0:
            raise ConfigError(f"config.json: {where}ff must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff},
                             "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class NuvilornLayer:
    mixer: LatentMixerConfig
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class NuvilornConfig:
    vocab_size: int
    width: int
    norm_eps: float
    layers: Tuple[NuvilornLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    # ---- reading -----------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "NuvilornConfig":
        vocab, width = require(d, "vocab", int), require(d, "width", int)
        eps = require(_mapping(d, "norm", ""), "eps", float)
        if vocab <= 0 or width <= 0 or eps <= 0:
            raise ConfigError("config.json: vocab, width and norm.eps must be positive")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, l in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(l, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            if l.get("type") != "latent_attention":
                raise ConfigError(f"config.json: {where}type={l.get('type')!r} is not known (latent_attention)")
            mixer = LatentMixerConfig.from_dict(_mapping(l, "mixer", where), where + "mixer.")
            mlp = l.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            layers.append(NuvilornLayer(mixer, None if mlp is None else FeedForwardConfig.from_dict(mlp, where + "mlp.")))
        for i, l in enumerate(layers):
            j = l.mixer.kv_from
            if j is None:
                continue
            if not 0 <= j < i:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j} must name an earlier layer")
            src = layers[j].mixer
            if src.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j} names a layer without latents of its own")
            if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (l.mixer.kv_rank, l.mixer.rot_dim,
                                                                          l.mixer.rot_base, l.mixer.rot_dims):
                raise ConfigError(f"config.json: layers[{i}] reads layer {j}'s latents but differs from it in "
                                  "kv_rank, rot_dim or rotation")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab, width, eps, tuple(layers), eos_ids)

    # ---- writing -----------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.width,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": "latent_attention", "mixer": l.mixer.to_dict(),
                        "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers],
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- lowering ----------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        def gain(prefix: str, name: str) -> PartSpec:
            return PartSpec("rms_norm", {"eps": self.norm_eps, "scalar": True}, prefix=prefix, rename={"weight": name})
        layers = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l.mixer
            mixer = PartSpec("latent_attention", {
                "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim, "kv_rank": m.kv_rank,
                "scale": m.scale, "norm_eps": self.norm_eps, "kv_proj": m.kv_from is None,
                "position": {"kind": "rope_interleaved", "base": m.rot_base, "dims": m.rot_dims},
            }, prefix=p + "mix.")
            if l.mlp is None:
                ffn, norm_f = PartSpec("none", {}), PartSpec("none", {})
            elif l.mlp.kind == "dense":
                ffn = PartSpec("swiglu", {"intermediate_size": l.mlp.ff}, prefix=p + "mlp.",
                               rename={"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"})
                norm_f = gain(p, "norm2")
            else:
                ffn = PartSpec("routed_experts", {
                    "num_experts": l.mlp.experts, "top_k": l.mlp.top, "expert_ff": l.mlp.ff,
                    "shared_ff": l.mlp.shared_ff, "shared_gate": True, "score": "sigmoid", "renormalize": False,
                    "weight_on": "input"}, prefix=p + "mlp.")
                norm_f = gain(p, "norm2")
            layers.append(LayerSpec("pre_norm", mixer, ffn, gain(p, "norm1"), norm_f))
        # a layer with kv_from reads the cache of the schedule entry of the layer it names (entries and
        # layers coincide: every layer runs once)
        schedule = tuple(ScheduleEntry(i, l.mixer.kv_from) for i, l in enumerate(self.layers))
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=self.width, vocab_size=self.vocab_size,
            max_position=NO_POSITION_LIMIT, layers=tuple(layers), schedule=schedule,
            embedding=PartSpec("token_embedding", {"norm": {"kind": "rms_norm", "eps": self.norm_eps, "scalar": True}},
                               rename={"weight": "embed", "norm.weight": "embed.norm"}),
            final_norm=gain("final.", "norm"),
            head=PartSpec("lm_head", {"tied": False}, rename={"weight": "head"}),
        )
        spec.validate()
        return spec
