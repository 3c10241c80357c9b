"""Typed configuration of the Kedesun design, read from config.json (``"architecture": "Kedesun"``).

Keys: ``vocab``, ``width``, ``norm.eps``, ``layers`` (a list; each entry has ``type`` = latent_attention | retention,
the mixer's sizes and constants under ``mixer``, and ``mlp`` = {kind: dense, ff} | {kind: moe, router: {experts, top},
expert: {ff}, shared: {ff} or absent} | null). Latent attention: ``heads``, ``dim`` (unrotated query/key size a head),
``rot_dim`` (rotated size), ``vdim``, ``kv_rank``, ``scale`` (absent: 1 / sqrt(dim + rot_dim)), ``rot`` = {base, dims,
scaling: {factor, original, fast, slow} or absent}. Retention: ``heads``, ``dim``, ``vdim``, ``decay`` (one number a
head). Every size and every constant that can differ between two models of the design comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .ramosun import DEFAULT_MAX_CONTEXT, _need, _positive_int

LATENT_ATTENTION, RETENTION = "latent_attention", "retention"
DENSE, MOE = "dense", "moe"


@dataclass(frozen=True)
class YarnRotaryConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, original, fast, slow

    @staticmethod
    def from_dict(raw: Mapping[str, Any], rotated: int, where: str) -> "YarnRotaryConfig":
        dims = _positive_int(raw, "dims", where)
        if dims % 2 or dims > rotated:
            raise ConfigError(f"{where}: 'dims' {dims} must be even and at most the rotated size {rotated}")
        base = float(_need(raw, "base", where))
        if base <= 1.0:
            raise ConfigError(f"{where}: 'base' must exceed 1")
        scaling = raw.get("scaling")
        if scaling is not None:
            scaling = tuple(float(_need(scaling, key, where + ".scaling")) for key in ("factor", "original", "fast", "slow"))
            if scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0:
                raise ConfigError(f"{where}.scaling: factor, original, fast and slow must be positive")
        return YarnRotaryConfig(base=base, dims=dims, scaling=scaling)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return out


@dataclass(frozen=True)
class KedesunFeedForward:
    kind: str
    ff: int                                  # dense: the inner size; moe: an expert's inner size
    experts: int = 0
    top: int = 0
    shared_ff: Optional[int] = None          # moe: the shared expert's inner size (None: no shared expert)

    @staticmethod
    def from_dict(raw: Mapping[str, Any], where: str) -> "KedesunFeedForward":
        kind = _need(raw, "kind", where)
        if kind == DENSE:
            return KedesunFeedForward(kind=DENSE, ff=_positive_int(raw, "ff", where))
        if kind == MOE:
            router = _need(raw, "router", where)
            experts = _positive_int(router, "experts", where + ".router")
            top = _positive_int(router, "top", where + ".router")
            if top > experts:
                raise ConfigError(f"{where}.router: top {top} exceeds the {experts} experts")
            shared = raw.get("shared")
            return KedesunFeedForward(kind=MOE, ff=_positive_int(_need(raw, "expert", where), "ff", where + ".expert"),
                                      experts=experts, top=top,
                                      shared_ff=None if shared is None else _positive_int(shared, "ff", where + ".shared"))
        raise ConfigError(f"{where}: unknown kind {kind!r}; known: {DENSE}, {MOE}")

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == DENSE:
            return {"kind": DENSE, "ff": self.ff}
        out: Dict[str, Any] = {"kind": MOE, "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class KedesunLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    mlp: Optional[KedesunFeedForward] = None
    rot_dim: int = 0                               # latent attention
    kv_rank: int = 0
    scale: Optional[float] = None
    rotary: Optional[YarnRotaryConfig] = None
    decay: Tuple[float, ...] = ()                  # retention: one decay a head

    @staticmethod
    def from_dict(raw: Mapping[str, Any], index: int) -> "KedesunLayer":
        where = f"layers[{index}]"
        kind = _need(raw, "type", where)
        if kind not in (LATENT_ATTENTION, RETENTION):
            raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {LATENT_ATTENTION}, {RETENTION}")
        mixer = _need(raw, "mixer", where)
        where_mixer = where + ".mixer"
        heads = _positive_int(mixer, "heads", where_mixer)
        dim = _positive_int(mixer, "dim", where_mixer)
        vdim = _positive_int(mixer, "vdim", where_mixer)
        mlp = raw.get("mlp")
        fields: Dict[str, Any] = {"mlp": None if mlp is None else KedesunFeedForward.from_dict(mlp, where + ".mlp")}
        if kind == LATENT_ATTENTION:
            rot_dim = _positive_int(mixer, "rot_dim", where_mixer)
            fields["rot_dim"] = rot_dim
            fields["kv_rank"] = _positive_int(mixer, "kv_rank", where_mixer)
            fields["scale"] = float(mixer["scale"]) if mixer.get("scale") is not None else (dim + rot_dim) ** -0.5
            fields["rotary"] = YarnRotaryConfig.from_dict(_need(mixer, "rot", where_mixer), rot_dim, where_mixer + ".rot")
        else:
            decay = _need(mixer, "decay", where_mixer)
            if not isinstance(decay, (list, tuple)) or len(decay) != heads:
                raise ConfigError(f"{where_mixer}: 'decay' must list one number for each of the {heads} heads")
            fields["decay"] = tuple(float(d) for d in decay)
        return KedesunLayer(type=kind, heads=heads, dim=dim, vdim=vdim, **fields)

    def to_dict(self) -> Dict[str, Any]:
        mixer: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.type == LATENT_ATTENTION:
            mixer.update(rot_dim=self.rot_dim, kv_rank=self.kv_rank, scale=self.scale, rot=self.rotary.to_dict())
        else:
            mixer["decay"] = list(self.decay)
        return {"type": self.type, "mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class KedesunConfig:
    vocab: int
    width: int
    layers: Tuple[KedesunLayer, ...]
    norm_eps: float
    max_context: int = DEFAULT_MAX_CONTEXT
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    model_type: str = "Kedesun"

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "KedesunConfig":
        layers_raw = _need(raw, "layers", "config.json")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        eos = raw.get("eos_token_id")
        eos_ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (() if eos is None else (int(eos),))
        context = raw.get("max_context")
        eps = float(_need(_need(raw, "norm", "config.json"), "eps", "norm"))
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        return KedesunConfig(
            vocab=_positive_int(raw, "vocab", "config.json"), width=_positive_int(raw, "width", "config.json"),
            layers=tuple(KedesunLayer.from_dict(layer, index) for index, layer in enumerate(layers_raw)),
            norm_eps=eps, max_context=DEFAULT_MAX_CONTEXT if context is None else int(context), eos_token_ids=eos_ids,
            bos_token_id=None if raw.get("bos_token_id") is None else int(raw["bos_token_id"]))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.model_type, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers],
                "max_context": self.max_context}
