"""Typed configuration of the Zekazen architecture, read from its own ``config.json`` keys, and its lowering
to a ``ModelSpec``.

A Zekazen config.json names the design with a string and lists its layers one by one; layers of one model may
differ in kind and in every size:

    {"architecture": "Zekazen", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "retention",
                 "mixer": {"heads", "dim", "vdim", "decay": [one per head], "rot": {"base", "dims"}},
                 "mlp": null | {"kind": "moe", "expert": {"ff": F},
                                "router": {"experts": E, "identity": I, "top": k, "scale": s,
                                           "groups": {"count": n, "keep": m}}}},
                {"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv": taps, "scale", "mask": {"size": window}},
                 "mlp": ...}, ...]}

The design: every layer is pre-norm (``l<i>.norm1``, ``l<i>.norm2``, RMS norms with a weight per coordinate) around
a mixer (``l<i>.mix.*``) and a feed-forward (``l<i>.mlp.*``).  A ``retention`` mixer is linear attention with a
fixed decay per head, rotary positions on q and k, a per-head unit norm of its output and a silu gate.  An
``attention`` mixer is grouped-query attention over a sliding window whose q, k and v pass through a short causal
convolution (``<tensor>.conv``), with unit-normed q and k, no positions, a sink term in the softmax and a sigmoid
gate.  The feed-forward is a mixture of gated silu experts chosen by softmax scores plus a correction vector,
inside the best groups of neighbouring experts, with identity experts that return their input; the weights are
the scores times ``scale``.  A last norm (``final.norm``) and an untied head (``head``) give the logits.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, coerce, require

ARCHITECTURE = "Zekazen"
# the design sets no longest sequence; the cache an engine is built with does
NO_POSITION_LIMIT = 1 << 24


def _mapping(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


def _req(m: Mapping[str, Any], key: str, typ, where: str):
    if key not in m or m[key] is None:
        raise ConfigError(f"config.json: {where}missing key '{key}'")
    return coerce(m[key], where + key, typ)


def _opt(m: Mapping[str, Any], key: str, typ, where: str, default):
    return default if m.get(key) is None else coerce(m[key], where + key, typ)


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_base: float
    rot_dims: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "RetentionConfig":
        decay = d.get("decay")
        if not isinstance(decay, (list, tuple)):
            raise ConfigError(f"config.json: {where}'decay' must be a list with one number per head")
        rot = d.get("rot")
        if rot is None:
            base, dims = 10000.0, 0
        else:
            rot = _mapping(d, "rot", where)
            base, dims = _req(rot, "base", float, where + "rot."), _req(rot, "dims", int, where + "rot.")
        c = cls(_req(d, "heads", int, where), _req(d, "dim", int, where), _req(d, "vdim", int, where),
                tuple(coerce(x, where + "decay", float) for x in decay), base, dims)
        if min(c.heads, c.dim, c.vdim) <= 0:
            raise ConfigError(f"config.json: {where}sizes must be positive")
        if len(c.decay) != c.heads:
            raise ConfigError(f"config.json: {where}decay lists {len(c.decay)} numbers for {c.heads} heads")
        if c.rot_dims % 2 or not 0 <= c.rot_dims <= c.dim:
            raise ConfigError(f"config.json: {where}rot.dims={c.rot_dims} must be even and at most dim={c.dim}")
        if c.rot_base <= 0:
            raise ConfigError(f"config.json: {where}rot.base must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay),
                "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclass(frozen=True)
class ConvAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    window: int              # 0: every earlier token

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "ConvAttentionConfig":
        heads = _req(d, "heads", int, where)
        mask = d.get("mask")
        window = 0 if mask is None else _req(_mapping(d, "mask", where), "size", int, where + "mask.")
        c = cls(heads, _opt(d, "kv_heads", int, where, heads), _req(d, "dim", int, where), _req(d, "vdim", int, where),
                _opt(d, "conv", int, where, 1), _req(d, "scale", float, where), window)
        if min(c.heads, c.kv_heads, c.dim, c.vdim, c.conv) <= 0 or c.window < 0:
            raise ConfigError(f"config.json: {where}sizes must be positive")
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}heads={c.heads} is not a multiple of kv_heads={c.kv_heads}")
        if c.conv > 8:
            raise ConfigError(f"config.json: {where}conv={c.conv}: at most 8 taps are built")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "conv": self.conv, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    experts: int
    identity: int
    top: int
    scale: float
    groups: int
    keep: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "ExpertsConfig":
        if d.get("kind") != "moe":
            raise ConfigError(f"config.json: {where}kind={d.get('kind')!r} is not known (moe)")
        router, expert = _mapping(d, "router", where), _mapping(d, "expert", where)
        groups = router.get("groups")
        if groups is None:
            count, keep = 1, 1
        else:
            groups = _mapping(router, "groups", where + "router.")
            count, keep = _req(groups, "count", int, where + "router.groups."), _req(groups, "keep", int, where + "router.groups.")
        c = cls(_req(expert, "ff", int, where + "expert."), _req(router, "experts", int, where + "router."),
                _opt(router, "identity", int, where + "router.", 0), _req(router, "top", int, where + "router."),
                _opt(router, "scale", float, where + "router.", 1.0), count, keep)
        n = c.experts + c.identity
        if c.ff <= 0 or c.experts <= 0 or c.identity < 0:
            raise ConfigError(f"config.json: {where}sizes must be positive")
        if not 0 < c.top <= n:
            raise ConfigError(f"config.json: {where}router.top={c.top} of {n} router outputs")
        if not 1 <= c.keep <= c.groups or n % c.groups:
            raise ConfigError(f"config.json: {where}router.groups: {c.groups} groups (keep {c.keep}) over {n} router outputs")
        if c.keep * (n // c.groups) < c.top:
            raise ConfigError(f"config.json: {where}router.groups: {c.keep} groups of {n // c.groups} cannot give {c.top} choices")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "identity": self.identity, "top": self.top, "scale": self.scale,
                           "groups": {"count": self.groups, "keep": self.keep}}}


@dataclass(frozen=True)
class ZekazenLayer:
    mixer: Union[RetentionConfig, ConvAttentionConfig]
    mlp: Optional[ExpertsConfig]

    @property
    def type(self) -> str:
        return "retention" if isinstance(self.mixer, RetentionConfig) else "attention"


@dataclass(frozen=True)
class ZekazenConfig:
    vocab_size: int
    width: int
    norm_eps: float
    layers: Tuple[ZekazenLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    # ---- reading -----------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ZekazenConfig":
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
            kind = l.get("type")
            m = _mapping(l, "mixer", where)
            if kind == "retention":
                mixer = RetentionConfig.from_dict(m, where + "mixer.")
            elif kind == "attention":
                mixer = ConvAttentionConfig.from_dict(m, where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type={kind!r} is not known (retention, attention)")
            mlp = l.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            layers.append(ZekazenLayer(mixer, None if mlp is None else ExpertsConfig.from_dict(mlp, where + "mlp.")))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab, width, eps, tuple(layers), eos_ids)

    # ---- writing -----------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.width,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                       for l in self.layers],
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- lowering ----------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        def norm(prefix: str, name: str) -> PartSpec:
            return PartSpec("rms_norm", {"eps": self.norm_eps}, prefix=prefix, rename={"weight": name})
        proj = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g", "o_proj.weight": "o"}
        layers = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l.mixer
            if isinstance(m, RetentionConfig):
                position = ({"kind": "rope_half_split", "theta": m.rot_base, "head_dim": m.rot_dims, "n_rot": m.rot_dims}
                            if m.rot_dims else {"kind": "none"})
                mixer = PartSpec("retention", {
                    "num_heads": m.heads, "head_dim": m.dim, "v_dim": m.vdim, "decay": tuple(m.decay),
                    "norm_eps": self.norm_eps, "position": position, "gate": "silu"}, prefix=p + "mix.", rename=proj)
            else:
                mixer = PartSpec("conv_attention", {
                    "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
                    "conv_taps": m.conv, "scale": m.scale, "norm_eps": self.norm_eps, "window": m.window,
                    "qk_norm": True, "sink": True, "gate": "sigmoid"}, prefix=p + "mix.",
                    rename={**proj, "q_conv.weight": "q.conv", "k_conv.weight": "k.conv", "v_conv.weight": "v.conv"})
            if l.mlp is None:
                ffn, norm_f = PartSpec("none", {}), PartSpec("none", {})
            else:
                f = l.mlp
                ffn = PartSpec("routed_experts", {
                    "num_experts": f.experts, "top_k": f.top, "expert_ff": f.ff, "shared_ff": 0, "score": "softmax",
                    "renormalize": False, "weight_on": "output", "activation": "swiglu", "correction": True,
                    "groups": f.groups, "keep": f.keep, "route_scale": f.scale, "identity": f.identity},
                    prefix=p + "mlp.")
                norm_f = norm(p, "norm2")
            layers.append(LayerSpec("pre_norm", mixer, ffn, norm(p, "norm1"), norm_f))
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=self.width, vocab_size=self.vocab_size,
            max_position=NO_POSITION_LIMIT, layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            embedding=PartSpec("token_embedding", {}, rename={"weight": "embed"}),
            final_norm=norm("final.", "norm"),
            head=PartSpec("lm_head", {"tied": False}, rename={"weight": "head"}),
        )
        spec.validate()
        return spec
