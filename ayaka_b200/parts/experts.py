"""Feed-forward as a mixture of experts: a router picks a few small gated feed-forwards per
row; their products run grouped by expert (``csrc/moe.cu``)."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, build_part, register_part
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

    With ``scoring="sigmoid"`` the router instead scores ``s = sigmoid(z)``: the experts form
    ``groups`` equal groups of neighbours, a group's score is the sum of its two largest
    ``s``, only experts of the ``keep_groups`` best groups can be chosen, the ``top`` largest
    of those are, and their weights are ``route_scale * s`` (divided by their sum with
    ``renormalise``). With ``unit="silu"`` an expert is ``W_down (silu(W_gate h) * (W_up h))``.
    With ``shared_inner`` a gated feed-forward of that inner width (child ``shared``, the same
    unit) runs for every row and is added.

    With ``scoring="softmax_all"`` the scores are the softmax over *all* experts, the ``top``
    largest are chosen and weighted by their scores as they are (no renormalising). With
    ``unit="relu_squared"`` an expert has no gate: ``W_down relu(W_up h)^2``, and ``in.weight``
    is ``[experts * inner, width]``.

    Spec parameters: ``width``, ``experts``, ``top``, ``inner``; ``unit`` (``clamped`` when
    absent, with ``limit`` and ``alpha``; or ``silu``; or ``relu_squared``); ``scoring``
    (``softmax`` when absent; ``softmax_all``; or ``sigmoid`` with ``groups``, ``keep_groups``,
    ``route_scale``, ``renormalise``); ``shared_inner`` (0 when absent).
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.experts = int(spec.experts)  # type: ignore[arg-type]
        self.top = int(spec.top)  # type: ignore[arg-type]
        self.inner = int(spec.inner)  # type: ignore[arg-type]
        self.unit = str(spec.get("unit", "clamped"))
        self.single = self.unit == "relu_squared"
        if self.unit in ("silu", "relu_squared"):
            self.limit, self.alpha, self.shift = float("inf"), 1.0, 0.0
        elif self.unit == "clamped":
            self.limit = float(spec.limit)  # type: ignore[arg-type]
            self.alpha = float(spec.alpha)  # type: ignore[arg-type]
            self.shift = 1.0
        else:
            raise ValueError(f"unknown expert unit {self.unit!r}")
        if not 1 <= self.top <= self.experts <= 1024 or self.inner < 1 or not self.limit > 0:
            raise ValueError("experts takes 1 <= top <= experts <= 1024, inner >= 1 and a "
                             "positive limit")
        self.scoring = str(spec.get("scoring", "softmax"))
        self.groups = int(spec.get("groups", 1))  # type: ignore[arg-type]
        self.keep_groups = int(spec.get("keep_groups", self.groups))  # type: ignore[arg-type]
        self.route_scale = float(spec.get("route_scale", 1.0))  # type: ignore[arg-type]
        self.renormalise = bool(spec.get("renormalise", False))
        if self.scoring not in ("softmax", "softmax_all", "sigmoid"):
            raise ValueError(f"unknown router scoring {self.scoring!r}")
        if self.scoring == "sigmoid" and (
                self.groups < 1 or self.experts % self.groups
                or not 1 <= self.keep_groups <= self.groups
                or self.top > self.keep_groups * (self.experts // self.groups)):
            raise ValueError("groups must divide experts, 1 <= keep_groups <= groups, and the "
                             "kept groups must hold at least top experts")
        self.router = self.add_param("router.weight", (self.experts, self.width), "matrix")
        self.in_weight = self.add_param(
            "in.weight", (self.experts * (1 if self.single else 2) * self.inner, self.width),
            "matrix")
        self.out_weight = self.add_param("out.weight", (self.experts * self.width, self.inner),
                                         "matrix")
        shared_inner = int(spec.get("shared_inner", 0))  # type: ignore[arg-type]
        self.shared = None
        if shared_inner:
            if self.unit != "silu":
                raise ValueError("a shared expert comes with the silu unit")
            self.shared = self.add_child("shared", build_part(
                "feed_forward", "gated_dense",
                PartSpec("gated_dense", width=self.width, inner=shared_inner,
                         activation="silu"), ctx))

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext) -> None:
        self.forward_scaled(hidden, residual, step, None)

    def forward_into(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        """The same, written into ``out`` (fp32 ``[N, width]``) instead of added to it."""
        self.forward_scaled(hidden, out, step, None, accumulate=False)

    def forward_scaled(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                       scale: torch.Tensor | None, accumulate: bool = True) -> None:
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
        if self.scoring == "sigmoid":
            ops.moe_route_scored(logits, chosen, share, top=top, groups=self.groups,
                                 keep=self.keep_groups, factor=self.route_scale,
                                 renormalise=self.renormalise, rows=n)
        else:
            ops.moe_route(logits, chosen, share, top=top, rows=n,
                          over_all=self.scoring == "softmax_all")
        ops.moe_experts(hidden, self.in_weight, self.out_weight, chosen, pair_out,
                        experts=self.experts, top=top, limit=self.limit, alpha=self.alpha,
                        shift=self.shift, sorted_pairs=sorted_pairs, tile_expert=tile_expert,
                        inner=inner, rows=n, single=self.single)
        ops.moe_join(pair_out, share, residual, top=top, scale=scale, accumulate=accumulate,
                     rows=n)
        if self.shared is not None:
            self.shared.forward(hidden, residual, step)  # type: ignore[attr-defined]
