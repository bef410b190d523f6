"""The typed configuration of a Gagotar model, read from its own ``config.json`` keys.

Gagotar is a pre-norm decoder whose mixer runs a softmax attention (``left``) beside a gated
linear attention (``right``) and whose feed-forward is a mixture of experts.
``config.json``::

    {"architecture": "Gagotar", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv,
                                    "scale": s, "mask": {"size": c},
                                    "rot": {"base": b, "dims": r,
                                            "scaling": {"factor": f, "low": l, "high": h,
                                                        "original": o} or null}},
                           "right": {"heads": H', "dim": d', "vdim": dv', "tau": t
                                     (, "rank": r)}},
                 "mlp": {"kind": "moe", "expert": {"ff": F, "limit": L},
                         "router": {"experts": E, "top": k}} or null}, ...]}

Every size and constant of a layer is in its own entry, so layers may differ; nothing here
has a default that a model could silently rely on (``rot.scaling`` may be null or absent: the
frequencies are then unscaled; ``right.rank``, the rank of the decay's two projections, may
be absent: it is then read from the shape of the stored tensor).
"""

from __future__ import annotations

import math
from collections.abc import Mapping
from dataclasses import dataclass

from ayaka_b200.errors import ConfigError, ModelLoadError

__all__ = ["GagotarConfig", "GagotarLayer", "GagotarLeft", "GagotarMoE", "GagotarRight",
           "RotScaling"]

LAYER_TYPE = "parallel"


def _number(value: object, path: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or \
            not math.isfinite(value):
        raise ConfigError(path, "WRONG_TYPE", f"must be a finite number, got {value!r}")
    return float(value)


def _count(value: object, path: str, minimum: int = 1) -> int:
    if type(value) is not int:
        raise ConfigError(path, "WRONG_TYPE", f"must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(path, "INVALID_RANGE", f"must be at least {minimum}, got {value}")
    return value


def _object(parent: Mapping[str, object], key: str, where: str) -> Mapping[str, object]:
    value = parent.get(key)
    if not isinstance(value, Mapping):
        raise ModelLoadError(f"{where} lacks the object {key!r}", context={"missing": (key,)})
    return value


def _require(mapping: Mapping[str, object], keys: tuple[str, ...], where: str) -> None:
    lacking = [key for key in keys if mapping.get(key) is None]
    if lacking:
        raise ModelLoadError(f"{where} lacks " + ", ".join(lacking),
                             context={"missing": tuple(lacking)})


@dataclass(frozen=True, slots=True)
class RotScaling:
    """Rescaling of rotary frequencies by wavelength: above ``original / low`` a frequency is
    divided by ``factor``, below ``original / high`` it is kept, between them blended."""

    factor: float
    low: float
    high: float
    original: float

    def as_tuple(self) -> tuple[float, float, float, float]:
        return (self.factor, self.low, self.high, self.original)


@dataclass(frozen=True, slots=True)
class GagotarLeft:
    """The softmax-attention side of a layer's mixer."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int  # ``mask.size``: a query sees keys of its own block of this many positions
    rot_dims: int
    rot_base: float
    rot_scaling: RotScaling | None


@dataclass(frozen=True, slots=True)
class GagotarRight:
    """The gated-linear-attention side of a layer's mixer."""

    heads: int
    dim: int
    vdim: int
    tau: float
    #: rows of the first of the decay's two projections; ``None`` until a stored tensor's
    #: shape has given it (the key ``rank`` is optional in ``config.json``)
    rank: int | None = None


@dataclass(frozen=True, slots=True)
class GagotarMoE:
    """A layer's mixture of experts."""

    experts: int
    top: int
    ff: int
    limit: float


@dataclass(frozen=True, slots=True)
class GagotarLayer:
    left: GagotarLeft
    right: GagotarRight
    mlp: GagotarMoE | None


def _left(entry: Mapping[str, object], where: str) -> GagotarLeft:
    _require(entry, ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"), where)
    mask, rot = _object(entry, "mask", where), _object(entry, "rot", where)
    _require(mask, ("size",), f"{where}.mask")
    _require(rot, ("base", "dims"), f"{where}.rot")
    heads = _count(entry["heads"], f"{where}.heads")
    kv_heads = _count(entry["kv_heads"], f"{where}.kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"{where}.kv_heads", "INVALID_RANGE",
                          f"{kv_heads} key/value heads do not divide {heads} heads")
    dim = _count(entry["dim"], f"{where}.dim")
    rot_dims = _count(rot["dims"], f"{where}.rot.dims", minimum=0)
    if rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"{where}.rot.dims", "INVALID_RANGE",
                          f"must be even and at most dim ({dim}), got {rot_dims}")
    base = _number(rot["base"], f"{where}.rot.base")
    if base <= 0:
        raise ConfigError(f"{where}.rot.base", "INVALID_RANGE", "must be positive")
    scaling = None
    raw = rot.get("scaling")
    if raw is not None:
        if not isinstance(raw, Mapping):
            raise ConfigError(f"{where}.rot.scaling", "WRONG_TYPE", "must be an object or null")
        _require(raw, ("factor", "low", "high", "original"), f"{where}.rot.scaling")
        scaling = RotScaling(_number(raw["factor"], f"{where}.rot.scaling.factor"),
                             _number(raw["low"], f"{where}.rot.scaling.low"),
                             _number(raw["high"], f"{where}.rot.scaling.high"),
                             _number(raw["original"], f"{where}.rot.scaling.original"))
        if scaling.factor <= 0 or scaling.low <= 0 or scaling.high <= scaling.low or \
                scaling.original <= 0:
            raise ConfigError(f"{where}.rot.scaling", "INVALID_RANGE",
                              "needs factor > 0, original > 0 and 0 < low < high")
    return GagotarLeft(heads, kv_heads, dim, _count(entry["vdim"], f"{where}.vdim"),
                       _number(entry["scale"], f"{where}.scale"),
                       _count(mask["size"], f"{where}.mask.size"), rot_dims, base, scaling)


def _right(entry: Mapping[str, object], where: str) -> GagotarRight:
    _require(entry, ("heads", "dim", "vdim", "tau"), where)
    tau = _number(entry["tau"], f"{where}.tau")
    if tau <= 0:
        raise ConfigError(f"{where}.tau", "INVALID_RANGE", "must be positive")
    rank = entry.get("rank")
    return GagotarRight(_count(entry["heads"], f"{where}.heads"),
                        _count(entry["dim"], f"{where}.dim"),
                        _count(entry["vdim"], f"{where}.vdim"), tau,
                        None if rank is None else _count(rank, f"{where}.rank"))


def _moe(entry: Mapping[str, object], where: str) -> GagotarMoE:
    if entry.get("kind") != "moe":
        raise ModelLoadError(f"{where} must be null or of kind 'moe'")
    expert, router = _object(entry, "expert", where), _object(entry, "router", where)
    _require(expert, ("ff", "limit"), f"{where}.expert")
    _require(router, ("experts", "top"), f"{where}.router")
    experts = _count(router["experts"], f"{where}.router.experts")
    top = _count(router["top"], f"{where}.router.top")
    if top > experts:
        raise ConfigError(f"{where}.router.top", "INVALID_RANGE",
                          f"{top} chosen experts of {experts}")
    limit = _number(expert["limit"], f"{where}.expert.limit")
    if limit <= 0:
        raise ConfigError(f"{where}.expert.limit", "INVALID_RANGE", "must be positive")
    return GagotarMoE(experts, top, _count(expert["ff"], f"{where}.expert.ff"), limit)


@dataclass(frozen=True, slots=True)
class GagotarConfig:
    """Everything ``config.json`` says.

    Attributes:
        architecture: the registry key.
        vocab: rows of the embedding and of the head.
        width: width of the residual stream.
        eps: eps of every norm by the root mean square.
        layers: the layers in the order they run.
    """

    architecture: str
    vocab: int
    width: int
    eps: float
    layers: tuple[GagotarLayer, ...]

    @classmethod
    def from_json_dict(cls, config: Mapping[str, object]) -> GagotarConfig:
        missing = [key for key in ("architecture", "vocab", "width", "norm", "layers")
                   if config.get(key) is None]
        norm = config.get("norm")
        if not missing and (not isinstance(norm, Mapping) or norm.get("eps") is None):
            missing = ["norm.eps"]
        if missing:
            raise ModelLoadError("config.json lacks required keys for " + ", ".join(missing),
                                 context={"missing": tuple(missing)})
        entries = config["layers"]
        if not isinstance(entries, (list, tuple)):
            raise ConfigError("model.layers", "WRONG_TYPE", "must be a list")
        eps = _number(norm["eps"], "model.norm.eps")  # type: ignore[index]
        if eps <= 0:
            raise ConfigError("model.norm.eps", "INVALID_RANGE", "must be positive")
        layers = []
        for index, entry in enumerate(entries):
            where = f"model.layers[{index}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(where, "WRONG_TYPE", "must be an object")
            if entry.get("type") != LAYER_TYPE:
                raise ModelLoadError(f"{where}.type {entry.get('type')!r} is not a layer of "
                                     f"this design; known: [{LAYER_TYPE!r}]")
            mixer = _object(entry, "mixer", where)
            left = _left(_object(mixer, "left", f"{where}.mixer"), f"{where}.mixer.left")
            right = _right(_object(mixer, "right", f"{where}.mixer"), f"{where}.mixer.right")
            mlp = entry.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise ConfigError(f"{where}.mlp", "WRONG_TYPE", "must be an object or null")
            layers.append(GagotarLayer(left, right,
                                       None if mlp is None else _moe(mlp, f"{where}.mlp")))
        architecture = config["architecture"]
        if not isinstance(architecture, str) or not architecture:
            raise ConfigError("model.architecture", "WRONG_TYPE", "must be a non-empty string")
        return cls(architecture=architecture, vocab=_count(config["vocab"], "model.vocab"),
                   width=_count(config["width"], "model.width"), eps=eps, layers=tuple(layers))

    def to_json_dict(self) -> dict[str, object]:
        """The ``config.json`` content that reads back as this configuration."""
        entries = []
        for layer in self.layers:
            left, right, mlp = layer.left, layer.right, layer.mlp
            scaling = left.rot_scaling
            entries.append({
                "type": LAYER_TYPE,
                "mixer": {
                    "left": {"heads": left.heads, "kv_heads": left.kv_heads, "dim": left.dim,
                             "vdim": left.vdim, "scale": left.scale,
                             "mask": {"size": left.chunk},
                             "rot": {"base": left.rot_base, "dims": left.rot_dims,
                                     "scaling": None if scaling is None else {
                                         "factor": scaling.factor, "low": scaling.low,
                                         "high": scaling.high, "original": scaling.original}}},
                    "right": {"heads": right.heads, "dim": right.dim, "vdim": right.vdim,
                              "tau": right.tau,
                              **({} if right.rank is None else {"rank": right.rank})}},
                "mlp": None if mlp is None else {
                    "kind": "moe", "expert": {"ff": mlp.ff, "limit": mlp.limit},
                    "router": {"experts": mlp.experts, "top": mlp.top}}})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "layers": entries}
