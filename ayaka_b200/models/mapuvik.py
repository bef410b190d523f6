"""Mapuvik as data: its parts, its checkpoint names, its random weights.

A layer is ``h = norm1(x); x += mixer(h) + mlp(h)`` (block ``parallel``) with the norm
``rms(x) * (1 + w)``; the mixer is latent attention, a Mamba-2 layer or an mLSTM (``parts/
latent.py``, ``parts/recurrent.py``), the feed-forward dense with the erf GELU and no bias, or
absent. ``logits = head(final norm(x))``, head and embedding untied. A layer may run with an
earlier layer's tensors (``weights_of``): the execution order then names that layer again,
and the run gets a cache or state of its own.

Checkpoint names: ``embed``, ``head``, ``final.norm``, and per owning layer ``l<i>.norm1``,
``l<i>.mix.*``, ``l<i>.mlp.up`` / ``.down``; linear weights ``[out, in]``. Several stored
matrices that multiply the same input are stacked into one parameter (queries, latent and
gate of the attention; the six projections of the mLSTM).
"""

from __future__ import annotations

import hashlib
import math
from collections.abc import Iterator, Mapping

import torch

from ayaka_b200.config.mapuvik import MapuvikConfig, MapuvikLayer
from ayaka_b200.models.registry import Architecture, register_architecture
from ayaka_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, Run
from ayaka_b200.weights.rules import RandomInit, WeightRule, WeightRules

__all__ = ["MAPUVIK", "UNBOUNDED_POSITIONS", "mapuvik_model_spec", "mapuvik_weight_rules"]

#: The design has no table of positions and no longest sequence; the engine bounds a
#: sequence by its cache instead (positions are int32 on the device).
UNBOUNDED_POSITIONS = 1 << 30


def _mixer_spec(layer: MapuvikLayer, width: int, eps: float) -> PartSpec:
    get = layer.get
    if layer.kind == "latent_attention":
        return PartSpec("latent_attention", width=width, num_heads=get("heads"), dim=get("dim"),
                        rot=get("rot_dim"), value_dim=get("vdim"), rank=get("kv_rank"),
                        scale=get("scale"), window=get("mask.size"), rot_dims=get("rot.dims"),
                        rot_base=get("rot.base"), rot_layout="neighbours", eps=eps)
    if layer.kind == "mamba2":
        return PartSpec("mamba2", width=width, num_heads=get("heads"), columns=get("vdim"),
                        state=get("state"), groups=get("groups"), taps=get("conv"),
                        norm_groups=get("norm_groups"), eps=eps)
    return PartSpec("mlstm", width=width, num_heads=get("heads"), dim=get("dim"),
                    columns=get("vdim"), gate_cap=get("gate_cap"), eps=eps)


def _owners(config: MapuvikConfig) -> dict[int, int]:
    """Index in ``config.layers`` of every layer that owns tensors -> its index among the
    model's layers."""
    return {index: place for place, index in enumerate(
        i for i, layer in enumerate(config.layers) if layer.weights_of == i)}


def mapuvik_model_spec(config: MapuvikConfig) -> ModelSpec:
    """The model as parts. Every size comes from ``config``."""
    width = config.width
    norm = PartSpec("rms_norm", width=width, eps=config.eps, offset=1.0)
    owners = _owners(config)
    layers = []
    for index in owners:
        layer = config.layers[index]
        feed_forward = PartSpec("none") if layer.ff is None else PartSpec(
            "dense", width=width, inner=layer.ff, activation="gelu_erf", bias=False)
        layers.append(LayerSpec(block="parallel", mixer=_mixer_spec(layer, width, config.eps),
                                feed_forward=feed_forward, mixer_norm=norm,
                                feed_forward_norm=norm))
    return ModelSpec(
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=UNBOUNDED_POSITIONS,
        embedding=PartSpec("token", vocab_size=config.vocab, width=width),
        position=PartSpec("none"),
        layers=tuple(layers),
        order=tuple(Run(layer=owners[layer.weights_of]) for layer in config.layers),
        final_norm=norm,
        head=PartSpec("linear", vocab_size=config.vocab, width=width, tied=False),
        eos_token_id=None,
    )


def _stacked(dst: str, pieces: list[tuple[str, int]]) -> dict[str, WeightRule]:
    """Rules that put stored tensors one under the other into parameter ``dst``."""
    rules, at = {}, 0
    for name, rows in pieces:
        rules[name] = WeightRule(dst, dim=0, offset=at)
        at += rows
    return rules


def mapuvik_weight_rules(config: MapuvikConfig) -> WeightRules:
    rules: dict[str, WeightRule | tuple[WeightRule, ...]] = {
        "embed": WeightRule("embedding.weight"),
        "head": WeightRule("head.weight"),
        "final.norm": WeightRule("final_norm.weight"),
    }
    for index, place in _owners(config).items():
        layer, get = config.layers[index], config.layers[index].get
        src, dst = f"l{index}.", f"layers.{place}."
        mix, mixer = f"{src}mix.", f"{dst}mixer."
        rules[f"{src}norm1"] = WeightRule(f"{dst}mixer_norm.weight")
        if layer.ff is not None:
            rules[f"{src}mlp.up"] = WeightRule(f"{dst}feed_forward.up.weight")
            rules[f"{src}mlp.down"] = WeightRule(f"{dst}feed_forward.down.weight")
        heads = int(get("heads"))
        if layer.kind == "latent_attention":
            rot = int(get("rot_dim"))
            rules.update(_stacked(f"{mixer}proj.weight", [
                (f"{mix}q", heads * (int(get("dim")) + rot)),
                (f"{mix}dkv", int(get("kv_rank")) + rot),
                (f"{mix}g", heads * int(get("vdim")))]))
            rules[f"{mix}dkv.norm"] = WeightRule(f"{mixer}latent_norm.weight")
            rules[f"{mix}uk"] = WeightRule(f"{mixer}up_key.weight")
            rules[f"{mix}uv"] = WeightRule(f"{mixer}up_value.weight")
            rules[f"{mix}o"] = WeightRule(f"{mixer}out.weight")
        elif layer.kind == "mamba2":
            for stored, param in (("in", "in.weight"), ("conv", "conv.weight"),
                                  ("conv.b", "conv.bias"), ("dt_bias", "dt_bias"),
                                  ("A_log", "a_log"), ("D", "skip"), ("norm", "norm.weight"),
                                  ("o", "out.weight")):
                rules[f"{mix}{stored}"] = WeightRule(f"{mixer}{param}")
        else:
            qk, inner = heads * int(get("dim")), heads * int(get("vdim"))
            rules.update(_stacked(f"{mixer}proj.weight", [
                (f"{mix}q", qk), (f"{mix}k", qk), (f"{mix}v", inner), (f"{mix}g", inner),
                (f"{mix}i", heads), (f"{mix}f", heads)]))
            rules.update(_stacked(f"{mixer}gate_bias", [(f"{mix}i.b", heads),
                                                        (f"{mix}f.b", heads)]))
            rules[f"{mix}norm"] = WeightRule(f"{mixer}norm.weight")
            rules[f"{mix}o"] = WeightRule(f"{mixer}out.weight")
    return WeightRules(rules=rules)


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    return torch.Generator().manual_seed(int.from_bytes(digest, "big") & ((1 << 63) - 1))


def _random_tensors(config: MapuvikConfig, seed: int,
                    init: RandomInit) -> Iterator[tuple[str, torch.Tensor]]:
    """Random float32 tensors under checkpoint names. A matrix is drawn with deviation
    ``weight_std * sqrt(width / fan_in)``, so that a product keeps the size of its input
    whatever its inner width; norm weights (stored as deviations from one, or plain ones around
    one) with ``norm_std``; gate and step-size parameters in ranges in which the recurrences
    neither freeze nor forget at once. Each tensor has its own generator, seeded from
    ``seed`` and its name."""
    width = config.width
    loud = init.weight_std * math.sqrt(width)

    def normal(name: str, shape: tuple[int, ...], std: float, mean: float = 0.0) -> torch.Tensor:
        if std == 0.0:
            return torch.full(shape, mean, dtype=torch.float32)
        values = torch.randn(shape, generator=_generator(seed, name), dtype=torch.float32)
        return values.mul_(std).add_(mean)

    def matrix(name: str, rows: int, cols: int, gain: float = 1.0) -> torch.Tensor:
        return normal(name, (rows, cols), gain * loud / math.sqrt(cols))

    def uniform(name: str, shape: tuple[int, ...], low: float, high: float) -> torch.Tensor:
        values = torch.rand(shape, generator=_generator(seed, name), dtype=torch.float32)
        return values.mul_(high - low).add_(low)

    down = 1.0 / math.sqrt(2 * max(len(config.layers), 1)) \
        if init.scale_residual_projections else 1.0
    yield "embed", normal("embed", (config.vocab, width), max(init.weight_std, 1e-3) * 10)
    for index in _owners(config):
        layer, get = config.layers[index], config.layers[index].get
        p, mix = f"l{index}.", f"l{index}.mix."
        yield f"{p}norm1", normal(f"{p}norm1", (width,), init.norm_std)
        heads = int(get("heads"))
        if layer.kind == "latent_attention":
            dim, rot, vdim, rank = (int(get(k)) for k in ("dim", "rot_dim", "vdim", "kv_rank"))
            yield f"{mix}q", matrix(f"{mix}q", heads * (dim + rot), width)
            yield f"{mix}dkv", matrix(f"{mix}dkv", rank + rot, width)
            yield f"{mix}dkv.norm", normal(f"{mix}dkv.norm", (rank,), init.norm_std, 1.0)
            yield f"{mix}uk", matrix(f"{mix}uk", heads * dim, rank)
            yield f"{mix}uv", matrix(f"{mix}uv", heads * vdim, rank)
            yield f"{mix}g", matrix(f"{mix}g", heads * vdim, width)
            yield f"{mix}o", matrix(f"{mix}o", width, heads * vdim, down)
        elif layer.kind == "mamba2":
            P, N, G, taps = (int(get(k)) for k in ("vdim", "state", "groups", "conv"))
            inner, channels = heads * P, heads * P + 2 * G * N
            yield f"{mix}in", matrix(f"{mix}in", 2 * inner + 2 * G * N + heads, width)
            yield f"{mix}conv", normal(f"{mix}conv", (channels, taps), 1.0 / math.sqrt(taps))
            yield f"{mix}conv.b", normal(f"{mix}conv.b", (channels,), init.bias_std)
            yield f"{mix}dt_bias", uniform(f"{mix}dt_bias", (heads,), -3.0, 0.0)
            yield f"{mix}A_log", uniform(f"{mix}A_log", (heads,), -1.0, 1.5)
            yield f"{mix}D", normal(f"{mix}D", (heads,), 0.5, 1.0)
            yield f"{mix}norm", normal(f"{mix}norm", (inner,), init.norm_std, 1.0)
            yield f"{mix}o", matrix(f"{mix}o", width, inner, down)
        else:
            dim, vdim = int(get("dim")), int(get("vdim"))
            for name, rows in (("q", heads * dim), ("k", heads * dim), ("v", heads * vdim),
                               ("g", heads * vdim), ("i", heads), ("f", heads)):
                yield f"{mix}{name}", matrix(f"{mix}{name}", rows, width)
            yield f"{mix}i.b", normal(f"{mix}i.b", (heads,), 0.5)
            yield f"{mix}f.b", uniform(f"{mix}f.b", (heads,), 1.0, 4.0)
            yield f"{mix}norm", normal(f"{mix}norm", (heads * vdim,), init.norm_std, 1.0)
            yield f"{mix}o", matrix(f"{mix}o", width, heads * vdim, down)
        if layer.ff is not None:
            yield f"{p}mlp.up", matrix(f"{p}mlp.up", layer.ff, width)
            yield f"{p}mlp.down", matrix(f"{p}mlp.down", width, layer.ff, down)
    yield "final.norm", normal("final.norm", (width,), init.norm_std)
    yield "head", matrix("head", config.vocab, width)


def _parse(config_json: Mapping[str, object]) -> MapuvikConfig:
    return MapuvikConfig.from_json_dict(config_json)


MAPUVIK = register_architecture(Architecture(
    name="Mapuvik",
    parse_config=_parse,
    model_spec=mapuvik_model_spec,  # type: ignore[arg-type]
    weight_rules=mapuvik_weight_rules,  # type: ignore[arg-type]
    random_tensors=_random_tensors,  # type: ignore[arg-type]
    config_json=lambda config: config.to_json_dict(),  # type: ignore[attr-defined]
))
