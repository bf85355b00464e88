"""Side inputs of a layer: what a layer adds to the residual stream besides its two halves."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, Part, register_part
from ayaka_b200.parts.context import StepContext
from ayaka_b200.parts.spec import PartSpec

__all__ = ["TokenGatedInput"]


@register_part("side", "token_gated")
class TokenGatedInput(Part):
    """A small embedding of the row's own token, gated by the stream, back into the stream:
    ``e = table[token]`` (``dim`` entries), ``g = act(W_gate x) * e``, ``y = W_proj g``,
    ``x += factor * y / sqrt(mean(y^2) + eps) * weight`` (a plain norm weight).

    Parameters: ``table`` ``[vocab_size, dim]``, ``gate.weight`` ``[dim, width]``,
    ``proj.weight`` ``[width, dim]``, ``norm.weight`` ``[width]``.

    Spec parameters: ``width``, ``dim``, ``vocab_size``, ``activation`` (``gelu_tanh`` or
    ``silu``), ``eps``.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.dim = int(spec.dim)  # type: ignore[arg-type]
        self.vocab_size = int(spec.vocab_size)  # type: ignore[arg-type]
        self.activation = str(spec.get("activation", "gelu_tanh"))
        self.eps = float(spec.eps)  # type: ignore[arg-type]
        if self.dim < 1 or self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError("a token-gated input needs dim >= 1 and a known activation")
        self.table = self.add_param("table", (self.vocab_size, self.dim), "table")
        self.gate_weight = self.add_param("gate.weight", (self.dim, self.width), "matrix")
        self.proj_weight = self.add_param("proj.weight", (self.width, self.dim), "matrix")
        self.norm_weight = self.add_param("norm.weight", (self.width,), "vector")

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext, *,
                factor: float = 1.0, copy: torch.Tensor | None = None,
                then: Part | None = None, then_out: torch.Tensor | None = None) -> None:
        """``hidden``: the stream in the compute type; ``residual``: the fp32 stream, updated
        in place (and ``copy`` with it); ``then`` (an ``rms_norm`` part) with ``then_out``:
        the norm in front of the next sublayer, applied to the new stream in the same launch."""
        n, work = step.num_rows, step.workspace
        raw = work.buffer("token_input.gate", self.dim, torch.float32)
        gated = work.buffer("token_input.gated", self.dim, self.ctx.dtype)
        branch = work.buffer("token_input.branch", self.width, torch.float32)
        ops.linear(hidden, self.gate_weight, None, raw, rows=n)
        ops.gated_unit(raw, gated, activation=self.activation, rows=n, table=self.table,
                       index=step.tokens)
        ops.linear(gated, self.proj_weight, None, branch, rows=n)
        if then is None or then_out is None:
            ops.norm_add(branch, self.norm_weight, self.eps, residual, factor=factor, copy=copy,
                         rows=n)
        else:
            ops.norm_add(branch, self.norm_weight, self.eps, residual, factor=factor, copy=copy,
                         rows=n, next_weight=then.weight, next_eps=then.eps,  # type: ignore
                         next_offset=then.offset, next_out=then_out)  # type: ignore
