"""Typed configuration of the Ramosun design, read from config.json (``"architecture": "Ramosun"``).

Keys: ``vocab``, ``width``, ``norm.eps``, ``logit_softcap`` (absent or null: none), ``layers`` (a list; each entry
has ``type`` = attention | mlstm | delta, the mixer's sizes under ``mixer`` (``kv_heads`` absent: as many as heads;
the attention's ``scale`` absent: 1 / sqrt(dim); ``mask``, ``rot``, ``rot.scaling`` absent: none) and ``mlp`` =
{kind: dense, ff} or null), ``loop`` = {start, stop, times} (absent: every layer runs once). Every size and every constant that can
differ between two models of the design comes from here; nothing is taken from a particular checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError

ATTENTION, MLSTM, DELTA = "attention", "mlstm", "delta"
DEFAULT_MAX_CONTEXT = 131072     # the design states no longest sequence; this bounds a request's block table


def _need(mapping: Mapping[str, Any], key: str, where: str):
    if not isinstance(mapping, Mapping) or key not in mapping or mapping[key] is None:
        raise ConfigError(f"{where} lacks '{key}'")
    return mapping[key]


def _positive_int(mapping: Mapping[str, Any], key: str, where: str) -> int:
    value = _need(mapping, key, where)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"{where}: '{key}' must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, low, high, original

    @staticmethod
    def from_dict(raw: Mapping[str, Any], dim: int, where: str) -> "RotaryConfig":
        dims = _positive_int(raw, "dims", where)
        if dims % 2 or dims > dim:
            raise ConfigError(f"{where}: 'dims' {dims} must be even and at most the head size {dim}")
        scaling = raw.get("scaling")
        if scaling is not None:
            scaling = tuple(float(_need(scaling, key, where + ".scaling")) for key in ("factor", "low", "high", "original"))
        return RotaryConfig(base=float(_need(raw, "base", where)), dims=dims, scaling=scaling)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = dict(zip(("factor", "low", "high", "original"), self.scaling))
        return out


@dataclass(frozen=True)
class RamosunLayer:
    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    ff: Optional[int] = None                 # None: the layer has no feed-forward
    window: Optional[int] = None             # attention: how many most recent positions a query sees
    scale: Optional[float] = None            # attention: factor of the scores
    rotary: Optional[RotaryConfig] = None    # attention
    gate_cap: Optional[float] = None         # mlstm
    taps: Optional[int] = None               # delta: taps of the short convolutions

    @staticmethod
    def from_dict(raw: Mapping[str, Any], index: int) -> "RamosunLayer":
        where = f"layers[{index}]"
        kind = _need(raw, "type", where)
        if kind not in (ATTENTION, MLSTM, DELTA):
            raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {ATTENTION}, {MLSTM}, {DELTA}")
        mixer = _need(raw, "mixer", where)
        where_mixer = where + ".mixer"
        heads = _positive_int(mixer, "heads", where_mixer)
        dim = _positive_int(mixer, "dim", where_mixer)
        vdim = _positive_int(mixer, "vdim", where_mixer)
        kv_heads = heads if kind == MLSTM or mixer.get("kv_heads") is None else _positive_int(mixer, "kv_heads", where_mixer)
        if heads % kv_heads:
            raise ConfigError(f"{where_mixer}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        ff = None
        mlp = raw.get("mlp")
        if mlp is not None:
            if _need(mlp, "kind", where + ".mlp") != "dense":
                raise ConfigError(f"{where}.mlp: unknown kind {mlp['kind']!r}; known: dense")
            ff = _positive_int(mlp, "ff", where + ".mlp")
        fields: Dict[str, Any] = {}
        if kind == ATTENTION:
            if vdim != dim:
                raise ConfigError(f"{where_mixer}: the values are the keys, so vdim {vdim} must equal dim {dim}")
            mask = mixer.get("mask")
            fields["window"] = _positive_int(mask, "size", where_mixer + ".mask") if mask is not None else None
            fields["scale"] = float(mixer["scale"]) if mixer.get("scale") is not None else dim ** -0.5
            rot = mixer.get("rot")
            fields["rotary"] = RotaryConfig.from_dict(rot, dim, where_mixer + ".rot") if rot is not None else None
        elif kind == MLSTM:
            fields["gate_cap"] = float(_need(mixer, "gate_cap", where_mixer))
            if fields["gate_cap"] <= 0:
                raise ConfigError(f"{where_mixer}: gate_cap must be positive")
        else:
            fields["taps"] = _positive_int(mixer, "conv", where_mixer)
        return RamosunLayer(type=kind, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, ff=ff, **fields)

    def to_dict(self) -> Dict[str, Any]:
        mixer: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.type != MLSTM:
            mixer["kv_heads"] = self.kv_heads
        if self.type == ATTENTION:
            mixer["scale"] = self.scale
            if self.window is not None:
                mixer["mask"] = {"size": self.window}
            if self.rotary is not None:
                mixer["rot"] = self.rotary.to_dict()
        elif self.type == MLSTM:
            mixer["gate_cap"] = self.gate_cap
        else:
            mixer["conv"] = self.taps
        return {"type": self.type, "mixer": mixer,
                "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class RamosunConfig:
    vocab: int
    width: int
    layers: Tuple[RamosunLayer, ...]
    norm_eps: float
    logit_softcap: Optional[float] = None
    loop: Optional[Tuple[int, int, int]] = None       # start, stop, times
    max_context: int = DEFAULT_MAX_CONTEXT
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    model_type: str = "Ramosun"

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "RamosunConfig":
        layers_raw = _need(raw, "layers", "config.json")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = tuple(RamosunLayer.from_dict(layer, index) for index, layer in enumerate(layers_raw))
        loop = raw.get("loop")
        if loop is not None:
            start, stop, times = (int(_need(loop, key, "loop")) for key in ("start", "stop", "times"))
            if not (0 <= start < stop <= len(layers)) or times < 1:
                raise ConfigError(f"loop: start {start}, stop {stop}, times {times} do not name a run of the "
                                  f"{len(layers)} layers that runs at least once")
            loop = (start, stop, times)
        cap = raw.get("logit_softcap")
        if cap is not None and float(cap) <= 0:
            raise ConfigError("logit_softcap must be positive (or absent)")
        eos = raw.get("eos_token_id")
        eos_ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (() if eos is None else (int(eos),))
        context = raw.get("max_context")
        return RamosunConfig(
            vocab=_positive_int(raw, "vocab", "config.json"), width=_positive_int(raw, "width", "config.json"),
            layers=layers, norm_eps=float(_need(_need(raw, "norm", "config.json"), "eps", "norm")),
            logit_softcap=None if cap is None else float(cap), loop=loop,
            max_context=DEFAULT_MAX_CONTEXT if context is None else int(context), eos_token_ids=eos_ids,
            bos_token_id=None if raw.get("bos_token_id") is None else int(raw["bos_token_id"]))

    def run_order(self) -> Tuple[Tuple[int, bool], ...]:
        """(layer, whether a pass of the repeated run begins there) for every position of the run order."""
        count = len(self.layers)
        if self.loop is None:
            return tuple((index, False) for index in range(count))
        start, stop, times = self.loop
        order = [(index, False) for index in range(start)]
        for _ in range(times):
            order.extend((index, index == start) for index in range(start, stop))
        order.extend((index, False) for index in range(stop, count))
        return tuple(order)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.model_type, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers],
                               "max_context": self.max_context}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return out
