"""Gagotar as data: its parts, its checkpoint names, its random weights.

A layer is ``x += ls1 * mixer(norm1(x)); x += ls2 * mlp(norm2(x))`` (block ``pre_norm`` with
layer scale, norm ``rms(x) * w``). The mixer runs a softmax attention (``left``: grouped keys,
biases, norms over the whole query and key projections, rotated positions with rescaled
frequencies, a factor per head and a mixing of the heads' scores before the softmax, keys
visible inside the query's block of positions, a gate per head) beside a gated linear
attention (``right``), each normed over the width, and returns their mean (``parts/
side_by_side.py``, ``parts/recurrent.py``). The feed-forward is a mixture of experts
(``parts/experts.py``) or absent. ``logits = head(final norm(x))``, head and embedding untied.

Checkpoint names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.mix.left.*``, ``l<i>.mix.right.*``,
``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate`` / ``.up`` / ``.down``; linear weights ``[out, in]``.
Stored matrices that multiply the same input are stacked into one parameter, and all experts'
matrices of a kind lie one under the other.

One size is in no key of ``config.json``: the rank of the decay's two projections. It is the
row count of ``l<i>.mix.right.a1`` (``complete_config``); a configuration written by this
package carries it as ``right.rank``.
"""

from __future__ import annotations

import hashlib
import math
from collections.abc import Callable, Iterator, Mapping
from dataclasses import replace

import torch

from ayaka_b200.config.gagotar import GagotarConfig
from ayaka_b200.errors import ModelLoadError
from ayaka_b200.models.registry import Architecture, register_architecture
from ayaka_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, Run
from ayaka_b200.weights.rules import RandomInit, WeightRule, WeightRules

__all__ = ["GAGOTAR", "EXPERT_ALPHA", "gagotar_model_spec", "gagotar_weight_rules"]

#: The design has no table of positions and no longest sequence; the engine bounds a
#: sequence by its cache instead (positions are int32 on the device).
UNBOUNDED_POSITIONS = 1 << 30
#: the factor inside an expert's sigmoid, fixed by the design
EXPERT_ALPHA = 1.702


def gagotar_model_spec(config: GagotarConfig) -> ModelSpec:
    """The model as parts. Every size comes from ``config``."""
    width, eps = config.width, config.eps
    norm = PartSpec("rms_norm", width=width, eps=eps, offset=0.0)
    layers = []
    for index, layer in enumerate(config.layers):
        left, right, mlp = layer.left, layer.right, layer.mlp
        if right.rank is None:
            raise ModelLoadError(
                f"layer {index}: the rank of the decay's projections is neither in "
                "config.json nor known from a stored tensor")
        scaling = left.rot_scaling
        attention = PartSpec(
            "talking_attention", width=width, num_heads=left.heads, num_kv_heads=left.kv_heads,
            head_dim=left.dim, value_dim=left.vdim, scale=left.scale, chunk=left.chunk,
            window=0, bias=True, qk_norm=True, eps=eps, head_temperature=True, talking=True,
            head_gate=True, rot_dims=left.rot_dims, rot_base=left.rot_base,
            rot_scaling=None if scaling is None else scaling.as_tuple(), rot_layout="halves")
        linear = PartSpec("gated_linear_attention", width=width, num_heads=right.heads,
                          dim=right.dim, columns=right.vdim, tau=right.tau,
                          decay_rank=right.rank, eps=eps)
        mixer = PartSpec("side_by_side", width=width, eps=eps, sides=(attention, linear),
                         names=("left", "right"))
        feed_forward = PartSpec("none") if mlp is None else PartSpec(
            "experts", width=width, experts=mlp.experts, top=mlp.top, inner=mlp.ff,
            limit=mlp.limit, alpha=EXPERT_ALPHA)
        layers.append(LayerSpec(block="pre_norm", mixer=mixer, feed_forward=feed_forward,
                                mixer_norm=norm, feed_forward_norm=norm, layer_scale=True))
    return ModelSpec(
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=UNBOUNDED_POSITIONS,
        embedding=PartSpec("token", vocab_size=config.vocab, width=width),
        position=PartSpec("none"),
        layers=tuple(layers),
        order=tuple(Run(layer=index) for index in range(len(layers))),
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


def gagotar_weight_rules(config: GagotarConfig) -> WeightRules:
    rules: dict[str, WeightRule | tuple[WeightRule, ...]] = {
        "embed": WeightRule("embedding.weight"),
        "head": WeightRule("head.weight"),
        "final.norm": WeightRule("final_norm.weight"),
    }
    ignore: list[str] = []
    width = config.width
    for index, layer in enumerate(config.layers):
        left, right, mlp = layer.left, layer.right, layer.mlp
        src, dst = f"l{index}.", f"layers.{index}."
        rules[f"{src}norm1"] = WeightRule(f"{dst}mixer_norm.weight")
        rules[f"{src}ls1"] = WeightRule(f"{dst}mixer_scale")
        lsrc, ldst = f"{src}mix.left.", f"{dst}mixer.left."
        q, k, v = left.heads * left.dim, left.kv_heads * left.dim, left.kv_heads * left.vdim
        rules.update(_stacked(f"{ldst}proj.weight", [
            (f"{lsrc}q", q), (f"{lsrc}k", k), (f"{lsrc}v", v), (f"{lsrc}g", left.heads)]))
        rules.update(_stacked(f"{ldst}proj.bias", [
            (f"{lsrc}q.b", q), (f"{lsrc}k.b", k), (f"{lsrc}v.b", v)]))
        for stored, param in (("q.norm", "q_norm.weight"), ("k.norm", "k_norm.weight"),
                              ("talk", "talk"), ("temp", "temperature"), ("o", "out.weight")):
            rules[f"{lsrc}{stored}"] = WeightRule(f"{ldst}{param}")
        rsrc, rdst = f"{src}mix.right.", f"{dst}mixer.right."
        qk, inner = right.heads * right.dim, right.heads * right.vdim
        rules.update(_stacked(f"{rdst}proj.weight", [
            (f"{rsrc}q", qk), (f"{rsrc}k", qk), (f"{rsrc}v", inner), (f"{rsrc}g", inner)]))
        for stored, param in (("a1", "decay_down.weight"), ("a2", "decay_up.weight"),
                              ("a2.b", "decay_up.bias"), ("norm", "norm.weight"),
                              ("o", "out.weight")):
            rules[f"{rsrc}{stored}"] = WeightRule(f"{rdst}{param}")
        rules[f"{src}mix.left.out"] = WeightRule(f"{dst}mixer.left_out.weight")
        rules[f"{src}mix.right.out"] = WeightRule(f"{dst}mixer.right_out.weight")
        if mlp is None:
            # a layer without a feed-forward may still store the vectors that would go with it
            ignore.extend((rf"l{index}\.norm2", rf"l{index}\.ls2"))
            continue
        rules[f"{src}norm2"] = WeightRule(f"{dst}feed_forward_norm.weight")
        rules[f"{src}ls2"] = WeightRule(f"{dst}feed_forward_scale")
        ff = f"{dst}feed_forward."
        rules[f"{src}mlp.router"] = WeightRule(f"{ff}router.weight")
        for e in range(mlp.experts):
            rules[f"{src}mlp.e{e}.gate"] = WeightRule(f"{ff}in.weight", dim=0,
                                                      offset=e * 2 * mlp.ff)
            rules[f"{src}mlp.e{e}.up"] = WeightRule(f"{ff}in.weight", dim=0,
                                                    offset=e * 2 * mlp.ff + mlp.ff)
            rules[f"{src}mlp.e{e}.down"] = WeightRule(f"{ff}out.weight", dim=0,
                                                      offset=e * width)
    return WeightRules(rules=rules, ignore=tuple(ignore))


def _complete(config: GagotarConfig,
              shape_of: Callable[[str], tuple[int, ...] | None]) -> GagotarConfig:
    """Fill the sizes that only stored tensors give: a layer's decay rank."""
    layers = []
    for index, layer in enumerate(config.layers):
        if layer.right.rank is None:
            shape = shape_of(f"l{index}.mix.right.a1")
            if shape is not None and len(shape) == 2:
                layer = replace(layer, right=replace(layer.right, rank=int(shape[0])))
        layers.append(layer)
    return replace(config, layers=tuple(layers))


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    return torch.Generator().manual_seed(int.from_bytes(digest, "big") & ((1 << 63) - 1))


def _random_tensors(config: GagotarConfig, seed: int,
                    init: RandomInit) -> Iterator[tuple[str, torch.Tensor]]:
    """Random float32 tensors under checkpoint names. A matrix is drawn with deviation
    ``weight_std * sqrt(width / fan_in)``, so that a product keeps the size of its input
    whatever its inner width; norm weights and layer scales around one with ``norm_std``;
    biases with ``bias_std``; the decay's bias in a range in which the state neither freezes
    nor forgets at once. Each tensor has its own generator, seeded from ``seed`` and its
    name."""
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
    for index, layer in enumerate(config.layers):
        left, right, mlp = layer.left, layer.right, layer.mlp
        p = f"l{index}."
        yield f"{p}norm1", normal(f"{p}norm1", (width,), init.norm_std, 1.0)
        yield f"{p}ls1", normal(f"{p}ls1", (width,), init.norm_std, 1.0)
        m = f"{p}mix.left."
        q, k, v = left.heads * left.dim, left.kv_heads * left.dim, left.kv_heads * left.vdim
        for name, rows in (("q", q), ("k", k), ("v", v)):
            yield f"{m}{name}", matrix(f"{m}{name}", rows, width)
            yield f"{m}{name}.b", normal(f"{m}{name}.b", (rows,), init.bias_std)
        yield f"{m}q.norm", normal(f"{m}q.norm", (q,), init.norm_std, 1.0)
        yield f"{m}k.norm", normal(f"{m}k.norm", (k,), init.norm_std, 1.0)
        talk = normal(f"{m}talk", (left.heads, left.heads), 0.3 / math.sqrt(left.heads))
        yield f"{m}talk", talk + torch.eye(left.heads)
        yield f"{m}temp", uniform(f"{m}temp", (left.heads,), 0.5, 2.0)
        yield f"{m}g", matrix(f"{m}g", left.heads, width)
        yield f"{m}o", matrix(f"{m}o", width, left.heads * left.vdim, down)
        m = f"{p}mix.right."
        qk, inner = right.heads * right.dim, right.heads * right.vdim
        rank = right.rank if right.rank is not None else max(1, min(16, width // 4))
        for name, rows in (("q", qk), ("k", qk), ("v", inner), ("g", inner)):
            yield f"{m}{name}", matrix(f"{m}{name}", rows, width)
        yield f"{m}o", matrix(f"{m}o", width, inner, down)
        yield f"{m}norm", normal(f"{m}norm", (right.vdim,), init.norm_std, 1.0)
        yield f"{m}a1", matrix(f"{m}a1", rank, width)
        yield f"{m}a2", normal(f"{m}a2", (qk, rank), 1.0 / math.sqrt(rank))
        yield f"{m}a2.b", uniform(f"{m}a2.b", (qk,), 1.0, 5.0)
        yield f"{p}mix.left.out", normal(f"{p}mix.left.out", (width,), init.norm_std, 1.0)
        yield f"{p}mix.right.out", normal(f"{p}mix.right.out", (width,), init.norm_std, 1.0)
        if mlp is None:
            continue
        yield f"{p}norm2", normal(f"{p}norm2", (width,), init.norm_std, 1.0)
        yield f"{p}ls2", normal(f"{p}ls2", (width,), init.norm_std, 1.0)
        m = f"{p}mlp."
        yield f"{m}router", matrix(f"{m}router", mlp.experts, width, 2.0)
        for e in range(mlp.experts):
            yield f"{m}e{e}.gate", matrix(f"{m}e{e}.gate", mlp.ff, width)
            yield f"{m}e{e}.up", matrix(f"{m}e{e}.up", mlp.ff, width)
            yield f"{m}e{e}.down", matrix(f"{m}e{e}.down", width, mlp.ff, down)
    yield "final.norm", normal("final.norm", (width,), init.norm_std, 1.0)
    yield "head", matrix("head", config.vocab, width)


def _parse(config_json: Mapping[str, object]) -> GagotarConfig:
    return GagotarConfig.from_json_dict(config_json)


GAGOTAR = register_architecture(Architecture(
    name="Gagotar",
    parse_config=_parse,
    model_spec=gagotar_model_spec,  # type: ignore[arg-type]
    weight_rules=gagotar_weight_rules,  # type: ignore[arg-type]
    random_tensors=_random_tensors,  # type: ignore[arg-type]
    config_json=lambda config: config.to_json_dict(),  # type: ignore[attr-defined]
    complete_config=_complete,  # type: ignore[arg-type]
))
