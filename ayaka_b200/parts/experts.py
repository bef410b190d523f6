"""Feed-forward as a mixture of experts: a router picks a few small gated feed-forwards per
row; their products run grouped by expert (``csrc/moe.cu``)."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, register_part
from ayaka_b200.parts.context import StepContext
from ayaka_b200.parts.feed_forward import FeedForward
from ayaka_b200.parts.spec import PartSpec

__all__ = ["MixtureOfExperts"]


@register_part("feed_forward", "experts")
class MixtureOfExperts(FeedForward):
    """``experts`` feed-forwards without biases, of which every row uses ``top``.

    Router logits ``z = W_router h`` in fp32; the ``top`` largest are chosen and weighted by
    the softmax over just those. Expert ``e``: ``g = min(W_gate,e h, limit)``,
    ``u = clamp(W_up,e h, -limit, limit)``, ``y = g * sigmoid(alpha * g) * (u + 1)``, output
    ``W_down,e y``. The row's result is the weighted sum of its experts' outputs, added in fp32
    in the order of the choice (with the layer's scale, if any, in the same kernel).

    Parameters: ``router.weight`` ``[experts, width]``, ``in.weight`` ``[experts * 2 * inner,
    width]`` (every expert's gate rows, then its up rows), ``out.weight`` ``[experts * width,
    inner]``.

    Spec parameters: ``width``, ``experts``, ``top``, ``inner``, ``limit``, ``alpha``.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.experts = int(spec.experts)  # type: ignore[arg-type]
        self.top = int(spec.top)  # type: ignore[arg-type]
        self.inner = int(spec.inner)  # type: ignore[arg-type]
        self.limit = float(spec.limit)  # type: ignore[arg-type]
        self.alpha = float(spec.alpha)  # type: ignore[arg-type]
        if not 1 <= self.top <= self.experts <= 1024 or self.inner < 1 or not self.limit > 0:
            raise ValueError("experts takes 1 <= top <= experts <= 1024, inner >= 1 and a "
                             "positive limit")
        self.router = self.add_param("router.weight", (self.experts, self.width), "matrix")
        self.in_weight = self.add_param("in.weight", (self.experts * 2 * self.inner, self.width),
                                        "matrix")
        self.out_weight = self.add_param("out.weight", (self.experts * self.width, self.inner),
                                         "matrix")

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext) -> None:
        self.forward_scaled(hidden, residual, step, None)

    def forward_scaled(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                       scale: torch.Tensor | None) -> None:
        n, work, top = step.num_rows, step.workspace, self.top
        # scratch for the largest step, so that its addresses never change
        most = work.max_rows
        places, tiles = ops.moe_scratch(most, self.experts, top)
        logits = work.buffer("experts.logits", self.experts, torch.float32)
        chosen = work.buffer("experts.chosen", top, torch.int32).view(-1)
        share = work.buffer("experts.share", top, torch.float32).view(-1)
        sorted_pairs = work.buffer("experts.sorted", 1, torch.int32, rows=places).view(-1)
        tile_expert = work.buffer("experts.tile_expert", 1, torch.int32, rows=tiles).view(-1)
        inner = work.buffer("experts.inner", self.inner, self.ctx.dtype, rows=places)
        pair_out = work.buffer("experts.pair_out", self.width, torch.float32, rows=most * top)
        ops.linear(hidden, self.router, None, logits, rows=n)
        ops.moe_route(logits, chosen, share, top=top, rows=n)
        ops.moe_experts(hidden, self.in_weight, self.out_weight, chosen, pair_out,
                        experts=self.experts, top=top, limit=self.limit, alpha=self.alpha,
                        sorted_pairs=sorted_pairs, tile_expert=tile_expert, inner=inner, rows=n)
        ops.moe_join(pair_out, share, residual, top=top, scale=scale, accumulate=True, rows=n)
