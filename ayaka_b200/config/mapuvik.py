"""The typed configuration of a Mapuvik model, read from its own ``config.json`` keys.

Mapuvik is a decoder whose layers each run one mixer (``latent_attention``, ``mamba2`` or
``mlstm``) beside an optional dense feed-forward, from one shared norm. ``config.json``::

    {"architecture": "Mapuvik", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "<mixer kind>", "mixer": {...}, "mlp": {"kind": "dense", "ff": F}
                 or null, "weights_of": j (optional)}, ...]}

A layer with ``weights_of: j`` owns no tensors: it runs with layer ``j``'s weights and a
cache or state of its own. Every size and constant of a mixer is in its ``mixer`` object;
nothing here has a default that a model could silently rely on.
"""

from __future__ import annotations

import math
from collections.abc import Mapping
from dataclasses import dataclass

from ayaka_b200.errors import ConfigError, ModelLoadError

__all__ = ["MIXER_KEYS", "MapuvikConfig", "MapuvikLayer"]

#: mixer kind -> the keys its ``mixer`` object must hold (nested ones dotted)
MIXER_KEYS: dict[str, tuple[str, ...]] = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "mask.size",
                         "rot.base", "rot.dims"),
    "mamba2": ("heads", "vdim", "state", "groups", "conv", "norm_groups"),
    "mlstm": ("heads", "dim", "vdim", "gate_cap"),
}
_FLOAT_KEYS = {"scale", "rot.base", "gate_cap"}


def _lookup(mapping: Mapping[str, object], dotted: str) -> object:
    value: object = mapping
    for piece in dotted.split("."):
        if not isinstance(value, Mapping) or piece not in value:
            return None
        value = value[piece]
    return value


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


@dataclass(frozen=True, slots=True)
class MapuvikLayer:
    """One entry of ``layers``.

    Attributes:
        kind: the mixer's kind (``type`` in the file).
        mixer: the mixer's sizes and constants, flat (``mask.size`` and the like dotted).
        ff: width of the dense feed-forward's hidden layer, or ``None`` for no feed-forward.
        weights_of: index of the layer whose tensors this layer uses (itself when it owns
            them).
    """

    kind: str
    mixer: tuple[tuple[str, float | int], ...]
    ff: int | None
    weights_of: int

    def get(self, key: str) -> float | int:
        return dict(self.mixer)[key]


@dataclass(frozen=True, slots=True)
class MapuvikConfig:
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
    layers: tuple[MapuvikLayer, ...]

    @classmethod
    def from_json_dict(cls, config: Mapping[str, object]) -> MapuvikConfig:
        missing = [key for key in ("architecture", "vocab", "width", "norm", "layers")
                   if config.get(key) is None]
        if missing or _lookup(config, "norm.eps") is None:
            missing = missing or ["norm.eps"]
            raise ModelLoadError("config.json lacks required keys for " + ", ".join(missing),
                                 context={"missing": tuple(missing)})
        entries = config["layers"]
        if not isinstance(entries, (list, tuple)):
            raise ConfigError("model.layers", "WRONG_TYPE", "must be a list")
        eps = _number(_lookup(config, "norm.eps"), "model.norm.eps")
        if eps <= 0:
            raise ConfigError("model.norm.eps", "INVALID_RANGE", "must be positive")
        layers: list[MapuvikLayer] = []
        for index, entry in enumerate(entries):
            where = f"model.layers[{index}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(where, "WRONG_TYPE", "must be an object")
            kind = entry.get("type")
            if kind not in MIXER_KEYS:
                raise ModelLoadError(
                    f"{where}.type {kind!r} is not a mixer of this design; known: "
                    f"{sorted(MIXER_KEYS)}")
            mixer = entry.get("mixer")
            if not isinstance(mixer, Mapping):
                raise ConfigError(f"{where}.mixer", "WRONG_TYPE", "must be an object")
            lacking = [key for key in MIXER_KEYS[kind] if _lookup(mixer, key) is None]
            if lacking:
                raise ModelLoadError(f"{where}.mixer lacks " + ", ".join(lacking),
                                     context={"missing": tuple(lacking)})
            values = []
            for key in MIXER_KEYS[kind]:
                raw = _lookup(mixer, key)
                path = f"{where}.mixer.{key}"
                values.append((key, _number(raw, path) if key in _FLOAT_KEYS
                               else _count(raw, path)))
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ModelLoadError(f"{where}.mlp must be null or of kind 'dense'")
                ff = _count(mlp.get("ff"), f"{where}.mlp.ff")
            owner = entry.get("weights_of", index)
            owner = _count(owner, f"{where}.weights_of", minimum=0)
            if owner > index:
                raise ModelLoadError(f"{where}.weights_of must name an earlier layer")
            if owner < index:
                owner = layers[owner].weights_of  # (a layer that borrows in turn: its owner)
            layer = MapuvikLayer(str(kind), tuple(values), ff, owner)
            if owner != index and (layers[owner].kind, layers[owner].mixer, layers[owner].ff) \
                    != (layer.kind, layer.mixer, layer.ff):
                raise ModelLoadError(
                    f"{where} uses the tensors of layer {owner} but describes another layer")
            layers.append(layer)
        architecture = config["architecture"]
        if not isinstance(architecture, str) or not architecture:
            raise ConfigError("model.architecture", "WRONG_TYPE", "must be a non-empty string")
        return cls(architecture=architecture, vocab=_count(config["vocab"], "model.vocab"),
                   width=_count(config["width"], "model.width"), eps=eps, layers=tuple(layers))

    def to_json_dict(self) -> dict[str, object]:
        """The ``config.json`` content that reads back as this configuration."""
        entries = []
        for index, layer in enumerate(self.layers):
            mixer: dict[str, object] = {}
            for key, value in layer.mixer:
                at = mixer
                *outer, last = key.split(".")
                for piece in outer:
                    at = at.setdefault(piece, {})  # type: ignore[assignment]
                at[last] = value
            entry: dict[str, object] = {
                "type": layer.kind, "mixer": mixer,
                "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}}
            if layer.weights_of != index:
                entry["weights_of"] = layer.weights_of
            entries.append(entry)
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "layers": entries}
