"""Feed-forward parts. Here: the dense two-matrix MLP."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, Part, register_part
from ayaka_b200.parts.context import StepContext, Workspace
from ayaka_b200.parts.spec import PartSpec

__all__ = ["DenseMLP", "FeedForward", "GatedMLP", "NoFeedForward"]


class FeedForward(Part):
    """Interface of a feed-forward: read ``hidden`` (``[N, width]``, compute dtype) and **add**
    the result to ``residual`` (fp32 ``[N, width]``) in place. Optional:
    ``forward_normed(norm, residual, step)`` applies the norm itself (see ``Mixer``)."""

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext) -> None:
        raise NotImplementedError


@register_part("feed_forward", "none")
class NoFeedForward(FeedForward):
    """A layer without a feed-forward: no parameter, no launch."""

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext) -> None:
        return None


@register_part("feed_forward", "dense")
class DenseMLP(FeedForward):
    """``residual += act(h @ Wup.T + b_up) @ Wdown.T + b_down`` with the activation evaluated
    in fp32 inside the first product's epilogue (``python/ayaka/layers/ffn/dense.py:22-57``).

    With ``activation="xielu"`` the unit is ``softplus(p) z^2 + z / 2`` for ``z > 0`` and
    ``(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2`` otherwise, with two learned numbers
    (parameter ``act.numbers`` = ``(p, q)``): the first product writes fp32, one element-wise
    launch adds the bias and applies the unit.

    Spec parameters: ``width``, ``inner``, ``activation`` (``gelu_tanh``, ``gelu_erf`` or
    ``xielu``), ``bias`` (bool).
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.inner = int(spec.inner)  # type: ignore[arg-type]
        self.activation = str(spec.activation)
        self.learned_unit = self.activation == "xielu"
        if not self.learned_unit and (self.activation not in ops.ACTIVATIONS
                                      or self.activation == "none"):
            raise ValueError(f"unknown activation {self.activation!r}")
        bias = bool(spec.get("bias", True))
        self.up_weight = self.add_param("up.weight", (self.inner, self.width), "matrix")
        self.up_bias = self.add_param("up.bias", (self.inner,), "vector") if bias else None
        self.down_weight = self.add_param("down.weight", (self.width, self.inner), "matrix")
        self.down_bias = self.add_param("down.bias", (self.width,), "vector") if bias else None
        self.numbers = self.add_param("act.numbers", (2,), "vector") if self.learned_unit \
            else None
        self._native: dict[tuple[int, int], object] = {}

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext) -> None:
        self._run(hidden, residual, step, accumulate=True)

    def forward_into(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        """The same, written into ``out`` (fp32 ``[N, width]``) instead of added to it."""
        self._run(hidden, out, step, accumulate=False)

    def _run(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
             accumulate: bool) -> None:
        n = step.num_rows
        inner = step.workspace.buffer("feed_forward.inner", self.inner, self.ctx.dtype)
        if self.learned_unit:
            raw = step.workspace.buffer("feed_forward.raw", self.inner, torch.float32)
            ops.linear(hidden, self.up_weight, None, raw, rows=n)
            ops.unary_rows(raw, inner, activation="xielu", rows=n, bias=self.up_bias,
                           numbers=self.numbers)
        else:
            ops.linear(hidden, self.up_weight, self.up_bias, inner, activation=self.activation,
                       rows=n)
        ops.linear(inner, self.down_weight, self.down_bias, out, residual=accumulate, rows=n)

    def native_part(self, norm: Part, workspace: Workspace):  # noqa: ANN201
        """This feed-forward with ``norm`` in front of it as the C++ host code takes it
        (packed once per workspace)."""
        if self.learned_unit:  # (the C++ host path knows the built-in units only)
            return None
        key = (id(norm), id(workspace))
        found = self._native.get(key)
        if found is None:
            from ayaka_b200.kernels import native

            dtype = self.ctx.dtype
            found = native.mlp_part(
                dtype=dtype, width=self.width, inner=self.inner, activation=self.activation,
                eps=norm.eps, norm_weight=norm.weight, norm_bias=norm.bias,  # type: ignore
                up_weight=self.up_weight, up_bias=self.up_bias, down_weight=self.down_weight,
                down_bias=self.down_bias,
                normed=workspace.buffer("block.normed", self.width, dtype),
                inner_buf=workspace.buffer("feed_forward.inner", self.inner, dtype))
            self._native[key] = found
        return found

    def forward_normed(self, norm: Part, residual: torch.Tensor, step: StepContext) -> None:
        if self.learned_unit:
            scratch = step.workspace.buffer("block.normed", self.width, self.ctx.dtype)
            norm.forward(residual, scratch, count=step.num_rows)  # type: ignore[attr-defined]
            self.forward(scratch, residual, step)
            return
        if ops.NATIVE_STEP:
            from ayaka_b200.kernels import native

            native.run_mlp(self.native_part(norm, step.workspace),
                           native.step_args(step, residual.device), residual)
            return
        n = step.num_rows
        inner = step.workspace.buffer("feed_forward.inner", self.inner, self.ctx.dtype)
        scratch = step.workspace.buffer("block.normed", self.width, self.ctx.dtype)
        ops.linear_normed(residual, norm.weight, norm.bias, norm.eps,  # type: ignore
                          self.up_weight, self.up_bias, inner, scratch=scratch, count=n,
                          activation=self.activation)
        ops.linear(inner, self.down_weight, self.down_bias, residual, residual=True, rows=n)


@register_part("feed_forward", "gated_dense")
class GatedMLP(FeedForward):
    """``W_down (act(W_gate h) * (W_up h))`` without biases; the unit is evaluated in fp32.

    Parameters: ``in.weight`` ``[2 * inner, width]`` (the gate rows, then the up rows: one
    product), ``out.weight`` ``[width, inner]``.

    Spec parameters: ``width``, ``inner``, ``activation`` (``silu`` or ``gelu_tanh``).
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.inner = int(spec.inner)  # type: ignore[arg-type]
        self.activation = str(spec.get("activation", "silu"))
        if self.inner < 1 or self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError("a gated feed-forward needs inner >= 1 and a known activation")
        self.in_weight = self.add_param("in.weight", (2 * self.inner, self.width), "matrix")
        self.out_weight = self.add_param("out.weight", (self.width, self.inner), "matrix")

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext) -> None:
        self._run(hidden, residual, step, accumulate=True)

    def forward_into(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        """The same, written into ``out`` (fp32 ``[N, width]``) instead of added to it."""
        self._run(hidden, out, step, accumulate=False)

    def _run(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
             accumulate: bool) -> None:
        n, work = step.num_rows, step.workspace
        both = work.buffer("gated_dense.both", 2 * self.inner, torch.float32)
        unit = work.buffer("gated_dense.unit", self.inner, self.ctx.dtype)
        ops.linear(hidden, self.in_weight, None, both, rows=n)
        ops.gated_unit(both[:, :self.inner], unit, activation=self.activation, rows=n,
                       other=both[:, self.inner:])
        ops.linear(unit, self.out_weight, None, out, residual=accumulate, rows=n)
