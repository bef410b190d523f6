"""Mixers that run side by side on one input, and the attention with mixed heads that is one
of them in Gagotar."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import (BuildContext, CacheNeed, Part, StateNeed, build_part,
                                   register_part)
from ayaka_b200.parts.context import LayerCache, StepContext
from ayaka_b200.parts.mixer import Mixer
from ayaka_b200.parts.spec import PartSpec

__all__ = ["SideBySide", "TalkingAttention"]


@register_part("mixer", "side_by_side")
class SideBySide(Mixer):
    """Several mixers read the same normed input; each result is normalised over the model's
    width by its root mean square with a weight of its own, and the mixer returns their mean:
    ``(1 / n) * sum_b rms(side_b(h)) * w_b``. The join, an optional scale of the layer and the
    sum into the residual stream are one kernel (``ops.norm_sum``).

    At most one side may keep pages and at most one a per-request state (a layer has one
    cache and one state). A side that has ``forward_into(hidden, out, step, cache)`` writes
    its result into its scratch rows; any other mixer adds into zeroed rows.

    Spec parameters: ``width``, ``eps``, ``sides`` (a tuple of mixer ``PartSpec``), ``names``
    (the sides' names: children ``<name>`` and parameters ``<name>_out.weight``).
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext, position: Part | None = None) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.eps = float(spec.eps)  # type: ignore[arg-type]
        sides = tuple(spec.sides)  # type: ignore[arg-type]
        names = tuple(spec.names)  # type: ignore[arg-type]
        if not 1 <= len(sides) <= 4 or len(names) != len(sides) or len(set(names)) != len(names):
            raise ValueError("side_by_side takes one to four sides with a name each")
        self.sides: list[Mixer] = []
        self.weights: list[torch.Tensor] = []
        for name, side in zip(names, sides):
            part = build_part("mixer", side.kind, side, ctx, position)
            self.sides.append(self.add_child(str(name), part))  # type: ignore[arg-type]
            self.weights.append(self.add_param(f"{name}_out.weight", (self.width,), "vector"))
        if sum(side.cache_need() is not None for side in self.sides) > 1 or \
                sum(side.state_need() is not None for side in self.sides) > 1:
            raise ValueError("at most one side may keep pages and at most one a state")

    def cache_need(self) -> CacheNeed | None:
        return next((need for need in (side.cache_need() for side in self.sides)
                     if need is not None), None)

    def state_need(self) -> StateNeed | None:
        return next((need for need in (side.state_need() for side in self.sides)
                     if need is not None), None)

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache) -> None:
        self.forward_scaled(hidden, residual, step, cache, None)

    def forward_scaled(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                       cache: LayerCache, scale: torch.Tensor | None) -> None:
        n = step.num_rows
        branches = []
        for index, side in enumerate(self.sides):
            branch = step.workspace.buffer(f"side_by_side.{index}", self.width, torch.float32)
            if hasattr(side, "forward_into"):
                side.forward_into(hidden, branch, step, cache)
            else:
                branch[:n].zero_()
                side.forward(hidden, branch, step, cache)
            branches.append(branch)
        ops.norm_sum(branches, self.weights, self.eps, residual, factor=1.0 / len(branches),
                     scale=scale, accumulate=True, rows=n)


@register_part("mixer", "talking_attention")
class TalkingAttention(Mixer):
    """Softmax attention whose heads talk before the softmax, over paged keys and values.

    One fused projection gives queries (``num_heads x head_dim``), keys (``num_kv_heads x
    head_dim``), values (``num_kv_heads x value_dim``) and, with ``head_gate``, one raw gate
    per head. Optional pieces, each a spec parameter: a ``bias`` on queries, keys and values;
    ``qk_norm``: queries and keys each normalised by the root mean square over their *whole*
    projection (all heads at once) with a weight per entry; rotation of the first ``rot_dims``
    entries of every head by the position (``rot_layout``, frequencies from ``rot_base`` and
    ``rot_scaling``); ``head_temperature``: a learned factor per head on its scores;
    ``talking``: a learned ``[heads, heads]`` matrix that mixes the heads' scores for every
    (query, key) pair before the softmax; ``chunk``: a query sees only keys of its own block of
    that many positions (0: all earlier keys), ``window`` as elsewhere; ``head_gate``: head
    ``h``'s output times ``sigmoid(gate_h)``. Then the output projection.

    The mixing, the factors and ``scale`` are applied to the queries (``ops.talking_prepare``):
    the mix is linear in them, so nothing is mixed per pair and scores are plain fp32 sums.

    Spec parameters: ``width``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``value_dim``,
    ``scale``, ``chunk``, ``window``, ``bias``, ``qk_norm``, ``eps``, ``head_temperature``,
    ``talking``, ``head_gate``, ``rot_dims``, ``rot_base``, ``rot_scaling`` (``(factor, low,
    high, original)`` or ``None``), ``rot_layout``.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext, position: Part | None = None) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.num_heads = heads = int(spec.num_heads)  # type: ignore[arg-type]
        self.num_kv_heads = kv_heads = int(spec.num_kv_heads)  # type: ignore[arg-type]
        self.head_dim = dim = int(spec.head_dim)  # type: ignore[arg-type]
        self.value_dim = vdim = int(spec.get("value_dim", dim))  # type: ignore[arg-type]
        self.scale = float(spec.scale)  # type: ignore[arg-type]
        self.chunk = int(spec.get("chunk", 0))  # type: ignore[arg-type]
        self.window = int(spec.get("window", 0))  # type: ignore[arg-type]
        self.eps = float(spec.get("eps", 1e-6))  # type: ignore[arg-type]
        self.rot_dims = int(spec.get("rot_dims", 0))  # type: ignore[arg-type]
        self.rot_base = float(spec.get("rot_base", 10000.0))  # type: ignore[arg-type]
        self.rot_scaling = spec.get("rot_scaling")
        self.rot_layout = str(spec.get("rot_layout", "halves"))
        if heads < 1 or kv_heads < 1 or heads % kv_heads:
            raise ValueError(f"num_kv_heads ({kv_heads}) must divide num_heads ({heads})")
        if dim < 1 or vdim < 1 or self.chunk < 0 or self.window < 0:
            raise ValueError("talking attention needs head_dim, value_dim >= 1 and chunk, "
                             "window >= 0")
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= dim:
            raise ValueError(f"rot_dims must be even and at most head_dim ({dim}), got "
                             f"{self.rot_dims}")
        self.q_width, self.k_width, self.v_width = heads * dim, kv_heads * dim, kv_heads * vdim
        self.qkv_width = self.q_width + self.k_width + self.v_width
        self.head_gate = bool(spec.get("head_gate", False))
        out_features = self.qkv_width + (heads if self.head_gate else 0)
        self.proj_weight = self.add_param("proj.weight", (out_features, self.width), "matrix")
        self.proj_bias = self.add_param("proj.bias", (self.qkv_width,), "vector") \
            if spec.get("bias", False) else None
        self.q_norm = self.k_norm = self.temperature = self.talk = None
        if spec.get("qk_norm", False):
            self.q_norm = self.add_param("q_norm.weight", (self.q_width,), "vector")
            self.k_norm = self.add_param("k_norm.weight", (self.k_width,), "vector")
        if spec.get("head_temperature", False):
            self.temperature = self.add_param("temperature", (heads,), "vector")
        if spec.get("talking", False):
            # (role "vector": kept in float32 whatever the compute dtype)
            self.talk = self.add_param("talk", (heads, heads), "vector")
        self.out_weight = self.add_param("out.weight", (self.width, heads * vdim), "matrix")
        self._freq: torch.Tensor | None = None

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window, chunk=self.chunk,
                         value_dim=0 if self.value_dim == self.head_dim else self.value_dim)

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache) -> None:
        self._run(hidden, residual, step, cache, accumulate=True)

    def forward_into(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
                     cache: LayerCache) -> None:
        """The same, written into ``out`` (fp32 ``[N, width]``) instead of added to it."""
        self._run(hidden, out, step, cache, accumulate=False)

    def _run(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
             cache: LayerCache, accumulate: bool) -> None:
        n, dtype, work, heads = step.num_rows, self.ctx.dtype, step.workspace, self.num_heads
        if self._freq is None:
            self._freq = ops.rope_frequencies(
                self.rot_dims, self.rot_base, hidden.device,
                None if self.rot_scaling is None else tuple(self.rot_scaling))  # type: ignore
        group = step.groups[cache.group]  # type: ignore[index]
        proj = work.buffer("talking.proj", self.proj_weight.shape[0], torch.float32)
        qmix = work.buffer("talking.qmix", heads * self.k_width, dtype)
        attended = work.buffer("talking.out", heads * self.value_dim, dtype)
        ops.linear(hidden, self.proj_weight, None, proj, rows=n)
        ops.talking_prepare(
            proj, k_offset=self.q_width, v_offset=self.q_width + self.k_width,
            bias=self.proj_bias, q_weight=self.q_norm, k_weight=self.k_norm, eps=self.eps,
            positions=step.positions, freq=self._freq, layout=self.rot_layout, talk=self.talk,
            temp=self.temperature, scale=self.scale, slot_mapping=group.slot_mapping,
            k_pages=cache.k_pages if cache.writes else None,
            v_pages=cache.v_pages if cache.writes else None, qmix=qmix, heads=heads,
            kv_heads=self.num_kv_heads, dim=self.head_dim, vdim=self.value_dim, rows=n)
        reach = step.max_kv_len
        if self.chunk:
            reach = min(reach, self.chunk)
        if self.window:
            reach = min(reach, self.window)
        ops.talking_attention(
            qmix, cache.k_pages, cache.v_pages, group.block_table, step.request_of_row,
            step.positions, attended, heads=heads, chunk=self.chunk, window=self.window,
            reach=reach, gate=proj[:, self.qkv_width:] if self.head_gate else None, rows=n,
            single_rows=step.decode_only)
        ops.linear(attended, self.out_weight, None, out, residual=accumulate, rows=n)
