"""Mixers that carry a fixed-size state per request instead of cached keys: a Mamba-2
state-space layer, an mLSTM matrix memory, a gated linear attention and a generalised delta
rule. The state lives in float32 in the request's
slot of the cache storage's state tensor, starts at zero, and is carried through whatever
rows a step brings: ``csrc/recurrent.cu``."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, Part, StateNeed, register_part
from ayaka_b200.parts.context import LayerCache, StepContext
from ayaka_b200.parts.mixer import Mixer
from ayaka_b200.parts.spec import PartSpec

__all__ = ["MLSTM", "DeltaRule", "GatedLinearAttention", "Mamba2"]


@register_part("mixer", "mamba2")
class Mamba2(Mixer):
    """Selective state-space layer (state-space duality form, scalar decay per head).

    ``in`` projects the normed input to ``[z | x | B | C | dt]`` (``inner = heads * columns``
    for z and x, ``groups * state`` each for B and C, ``heads`` for dt). x, B and C pass a
    causal convolution per channel over ``taps`` rows (with bias) and silu. Per head (its
    group is ``head // (heads / groups)``): ``dt = softplus(dt + dt_bias)``,
    ``S <- exp(-exp(A_log) dt) S + dt B x^T``, ``y = S^T C + D x``. Then ``y * silu(z)`` is
    normalised by its root mean square in ``norm_groups`` equal parts, weighted, and projected
    back into the residual stream.

    State of a request: the last ``taps - 1`` inputs of the convolution, then S per head.

    Spec parameters: ``width``, ``num_heads``, ``columns`` (a head's width), ``state``,
    ``groups``, ``taps``, ``norm_groups``, ``eps``.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext, position: Part | None = None) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.num_heads = int(spec.num_heads)  # type: ignore[arg-type]
        self.columns = int(spec.columns)  # type: ignore[arg-type]
        self.state = int(spec.state)  # type: ignore[arg-type]
        self.groups = int(spec.groups)  # type: ignore[arg-type]
        self.taps = int(spec.taps)  # type: ignore[arg-type]
        self.norm_groups = int(spec.get("norm_groups", 1))  # type: ignore[arg-type]
        self.eps = float(spec.eps)  # type: ignore[arg-type]
        self.inner = self.num_heads * self.columns
        if self.groups < 1 or self.num_heads % self.groups:
            raise ValueError(f"groups ({self.groups}) must divide heads ({self.num_heads})")
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ValueError(f"norm_groups ({self.norm_groups}) must divide heads * columns "
                             f"({self.inner})")
        if not 1 <= self.taps <= 16 or not 1 <= self.state <= 512:
            raise ValueError("the convolution takes 1 to 16 taps, the state 1 to 512 entries")
        self.channels = self.inner + 2 * self.groups * self.state
        self.in_weight = self.add_param(
            "in.weight", (2 * self.inner + 2 * self.groups * self.state + self.num_heads,
                          self.width), "matrix")
        # (role "vector": kept in float32 whatever the compute dtype)
        self.conv_weight = self.add_param("conv.weight", (self.channels, self.taps), "vector")
        self.conv_bias = self.add_param("conv.bias", (self.channels,), "vector")
        self.dt_bias = self.add_param("dt_bias", (self.num_heads,), "vector")
        self.a_log = self.add_param("a_log", (self.num_heads,), "vector")
        self.skip = self.add_param("skip", (self.num_heads,), "vector")
        self.norm_weight = self.add_param("norm.weight", (self.inner,), "vector")
        self.out_weight = self.add_param("out.weight", (self.width, self.inner), "matrix")
        self.kept = (self.taps - 1) * self.channels

    def state_need(self) -> StateNeed:
        return StateNeed((ops.scan_state_floats(
            "mamba2", heads=self.num_heads, inner=self.state, columns=self.columns,
            taps=self.taps, channels=self.channels),))

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache) -> None:
        n, work, inner = step.num_rows, step.workspace, self.inner
        state = cache.state
        assert state is not None
        proj = work.buffer("mamba2.proj", self.in_weight.shape[0], torch.float32)
        xbc = work.buffer("mamba2.xbc", self.channels, torch.float32)
        y = work.buffer("mamba2.y", inner, torch.float32)
        gated = work.buffer("mamba2.gated", inner, self.ctx.dtype)
        ops.linear(hidden, self.in_weight, None, proj, rows=n)
        ops.causal_conv_silu(proj[:, inner:inner + self.channels], self.conv_weight,
                             self.conv_bias, state, xbc, request_of_row=step.request_of_row,
                             row_start=step.row_start, state_slot=step.state_slot, rows=n,
                             requests=step.num_requests)
        ops.mamba2_scan(xbc, proj[:, inner + self.channels:], self.dt_bias, self.a_log,
                        self.skip, state[:, self.kept:], y, row_start=step.row_start,
                        state_slot=step.state_slot, requests=step.num_requests,
                        heads=self.num_heads, groups=self.groups, state_size=self.state,
                        columns=self.columns)
        ops.rms_norm(y, self.norm_weight, self.eps, gated, groups=self.norm_groups, count=n,
                     gate=proj[:, :inner], gate_mode="silu_before")
        ops.linear(gated, self.out_weight, None, residual, residual=True, rows=n)


@register_part("mixer", "mlstm")
class MLSTM(Mixer):
    """Matrix memory with exponential gating (the mLSTM of xLSTM).

    One fused projection gives ``q`` (times ``dim^-1/2``), ``k`` (``heads x dim``), ``v``
    (``heads x columns``), the output gate, and per head a raw input and forget gate. With
    ``i = cap tanh((i_raw + b_i) / cap)``, ``f = logsigmoid(cap tanh((f_raw + b_f) / cap))``
    and a running maximum ``m`` that starts at 0: ``m' = max(f + m, i)``,
    ``S <- e^(f + m - m') S + e^(i - m') k v^T``, ``n`` likewise with ``k`` alone,
    ``out = S^T q / (max(|n . q|, e^-m') + 1e-6)``. Each head's ``out`` is divided by its root
    mean square; the joined heads are weighted, multiplied by ``sigmoid(gate)`` and projected
    back into the residual stream.

    Spec parameters: ``width``, ``num_heads``, ``dim``, ``columns``, ``gate_cap``, ``eps``.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext, position: Part | None = None) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.num_heads = int(spec.num_heads)  # type: ignore[arg-type]
        self.dim = int(spec.dim)  # type: ignore[arg-type]
        self.columns = int(spec.columns)  # type: ignore[arg-type]
        self.gate_cap = float(spec.gate_cap)  # type: ignore[arg-type]
        self.eps = float(spec.eps)  # type: ignore[arg-type]
        if not 1 <= self.dim <= 512 or self.columns < 1 or not self.gate_cap > 0:
            raise ValueError("mlstm takes dim in [1, 512], columns >= 1 and a positive gate_cap")
        heads = self.num_heads
        self.qk = heads * self.dim
        self.inner = heads * self.columns
        # q, k, v, output gate, raw input gates, raw forget gates: one product
        self.proj_weight = self.add_param(
            "proj.weight", (2 * self.qk + 2 * self.inner + 2 * heads, self.width), "matrix")
        self.gate_bias = self.add_param("gate_bias", (2 * heads,), "vector")
        self.norm_weight = self.add_param("norm.weight", (self.inner,), "vector")
        self.out_weight = self.add_param("out.weight", (self.width, self.inner), "matrix")

    def state_need(self) -> StateNeed:
        return StateNeed((ops.scan_state_floats("mlstm", heads=self.num_heads, inner=self.dim,
                                                columns=self.columns),))

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache) -> None:
        n, work, heads = step.num_rows, step.workspace, self.num_heads
        state = cache.state
        assert state is not None
        proj = work.buffer("mlstm.proj", self.proj_weight.shape[0], torch.float32)
        answer = work.buffer("mlstm.answer", self.inner, torch.float32)
        gated = work.buffer("mlstm.gated", self.inner, self.ctx.dtype)
        gate_at = 2 * self.qk + self.inner
        ops.linear(hidden, self.proj_weight, None, proj, rows=n)
        ops.mlstm_scan(proj, self.gate_bias, state, answer, row_start=step.row_start,
                       state_slot=step.state_slot, requests=step.num_requests, heads=heads,
                       dim=self.dim, columns=self.columns, k_offset=self.qk,
                       v_offset=2 * self.qk, i_offset=gate_at + self.inner,
                       f_offset=gate_at + self.inner + heads, cap=self.gate_cap)
        # a head is a group of the norm: each divided by its own root mean square
        ops.rms_norm(answer, self.norm_weight, self.eps, gated, groups=heads, count=n,
                     gate=proj[:, gate_at:gate_at + self.inner], gate_mode="sigmoid_after")
        ops.linear(gated, self.out_weight, None, residual, residual=True, rows=n)


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    """Linear attention with a learned decay per key channel.

    One fused projection gives ``q`` (times ``dim^-1/2``), ``k`` (``heads x dim``), ``v``
    (``heads x columns``) and an output gate (``heads x columns``); a low-rank pair of
    projections gives the raw decays ``z = W_up (W_down h) + b`` (``heads x dim``). Per head
    ``alpha = sigmoid(z)^(1/tau)``, ``S <- diag(alpha) S + k v^T``, ``out = S^T q``; each head's
    ``out`` is normalised by its root mean square with one weight of ``columns`` entries that
    all heads share; the joined heads are multiplied by ``silu(gate)`` and projected back.
    Decays, their logarithms and the state are float32.

    State of a request: ``S`` per head, ``[heads][columns][dim]``.

    Spec parameters: ``width``, ``num_heads``, ``dim``, ``columns``, ``tau``, ``decay_rank``,
    ``eps``.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext, position: Part | None = None) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.num_heads = heads = int(spec.num_heads)  # type: ignore[arg-type]
        self.dim = int(spec.dim)  # type: ignore[arg-type]
        self.columns = int(spec.columns)  # type: ignore[arg-type]
        self.tau = float(spec.tau)  # type: ignore[arg-type]
        self.decay_rank = int(spec.decay_rank)  # type: ignore[arg-type]
        self.eps = float(spec.eps)  # type: ignore[arg-type]
        if not 1 <= self.dim <= 512 or self.columns < 1 or heads < 1 or self.decay_rank < 1 \
                or not self.tau > 0:
            raise ValueError("gated linear attention takes dim in [1, 512], columns, heads and "
                             "decay_rank >= 1 and a positive tau")
        self.qk = heads * self.dim
        self.inner = heads * self.columns
        # q, k, v, output gate: one product
        self.proj_weight = self.add_param("proj.weight", (2 * self.qk + 2 * self.inner,
                                                          self.width), "matrix")
        self.decay_down = self.add_param("decay_down.weight", (self.decay_rank, self.width),
                                         "matrix")
        self.decay_up = self.add_param("decay_up.weight", (self.qk, self.decay_rank), "matrix")
        self.decay_bias = self.add_param("decay_up.bias", (self.qk,), "vector")
        self.norm_weight = self.add_param("norm.weight", (self.columns,), "vector")
        self.out_weight = self.add_param("out.weight", (self.width, self.inner), "matrix")

    def state_need(self) -> StateNeed:
        return StateNeed((self.num_heads * self.dim * self.columns,))

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache) -> None:
        self._run(hidden, residual, step, cache, accumulate=True)

    def forward_into(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
                     cache: LayerCache) -> None:
        """The same, written into ``out`` (fp32 ``[N, width]``) instead of added to it."""
        self._run(hidden, out, step, cache, accumulate=False)

    def _run(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
             cache: LayerCache, accumulate: bool) -> None:
        n, work, heads = step.num_rows, step.workspace, self.num_heads
        state = cache.state
        assert state is not None
        proj = work.buffer("gla.proj", self.proj_weight.shape[0], torch.float32)
        low = work.buffer("gla.low", self.decay_rank, self.ctx.dtype)
        decay = work.buffer("gla.decay", self.qk, torch.float32)
        answer = work.buffer("gla.answer", self.inner, torch.float32)
        gated = work.buffer("gla.gated", self.inner, self.ctx.dtype)
        ops.linear(hidden, self.proj_weight, None, proj, rows=n)
        ops.linear(hidden, self.decay_down, None, low, rows=n)
        ops.linear(low, self.decay_up, self.decay_bias, decay, rows=n)
        ops.gla_scan(proj, decay, state, answer, row_start=step.row_start,
                     state_slot=step.state_slot, requests=step.num_requests, heads=heads,
                     dim=self.dim, columns=self.columns, k_offset=self.qk, v_offset=2 * self.qk,
                     tau=self.tau, q_scale=self.dim ** -0.5)
        # a head is a group of the norm; the weight's `columns` entries repeat for every head
        ops.rms_norm(answer, self.norm_weight, self.eps, gated, groups=heads, count=n,
                     gate=proj[:, 2 * self.qk + self.inner:], gate_mode="silu_after")
        ops.linear(gated, self.out_weight, None, out, residual=accumulate, rows=n)


@register_part("mixer", "delta_rule")
class DeltaRule(Mixer):
    """Matrix memory that forgets per key channel and removes along the key before it writes
    (a generalised delta rule).

    One fused projection gives the receptance ``r``, the key ``k`` and the raw removal rate
    (``heads x dim`` each), the value ``v`` and an output gate (``heads x columns`` each) and
    the low-rank input of the decay; ``z = W_up tanh(W_down h) + b`` (``heads x dim``) is the
    raw decay. Per head, with the unit key ``u = k / sqrt(k . k + 1e-6)``,
    ``w = exp(-decay_rate * sigmoid(z))`` and ``a = sigmoid(rate + rate_bias)``:
    ``S <- diag(w) S - (a * u)(u^T S) + k v^T`` (both terms read the old ``S``),
    ``out = S^T r``. Each head's ``out`` is divided by its root mean square; the joined heads
    are multiplied by a weight per entry and by ``sigmoid(gate)`` and projected back. Decays,
    rates, unit keys and the state are float32.

    State of a request: ``S`` per head, ``[heads][columns][dim]``.

    Spec parameters: ``width``, ``num_heads``, ``dim``, ``columns`` (``dim`` when absent),
    ``decay_rank``, ``decay_rate``, ``eps``.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext, position: Part | None = None) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.num_heads = heads = int(spec.num_heads)  # type: ignore[arg-type]
        self.dim = int(spec.dim)  # type: ignore[arg-type]
        self.columns = int(spec.get("columns", self.dim))  # type: ignore[arg-type]
        self.decay_rank = int(spec.decay_rank)  # type: ignore[arg-type]
        self.decay_rate = float(spec.decay_rate)  # type: ignore[arg-type]
        self.eps = float(spec.eps)  # type: ignore[arg-type]
        if not 1 <= self.dim <= 512 or self.columns < 1 or heads < 1 or self.decay_rank < 1 \
                or not self.decay_rate >= 0:
            raise ValueError("the delta rule takes dim in [1, 512], columns, heads and "
                             "decay_rank >= 1 and a decay_rate >= 0")
        self.qk = heads * self.dim
        self.inner = heads * self.columns
        # r, k, raw rate | v, gate | the decay's low-rank input: one product
        self.k_at, self.a_at = self.qk, 2 * self.qk
        self.v_at, self.g_at = 3 * self.qk, 3 * self.qk + self.inner
        self.low_at = 3 * self.qk + 2 * self.inner
        self.proj_weight = self.add_param("proj.weight", (self.low_at + self.decay_rank,
                                                          self.width), "matrix")
        self.rate_bias = self.add_param("rate.bias", (self.qk,), "vector")
        self.decay_up = self.add_param("decay_up.weight", (self.qk, self.decay_rank), "matrix")
        self.decay_bias = self.add_param("decay_up.bias", (self.qk,), "vector")
        self.norm_weight = self.add_param("norm.weight", (self.inner,), "vector")
        self.out_weight = self.add_param("out.weight", (self.width, self.inner), "matrix")

    def state_need(self) -> StateNeed:
        return StateNeed((self.num_heads * self.dim * self.columns,))

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache) -> None:
        self._run(hidden, residual, step, cache, accumulate=True)

    def forward_into(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
                     cache: LayerCache) -> None:
        """The same, written into ``out`` (fp32 ``[N, width]``) instead of added to it."""
        self._run(hidden, out, step, cache, accumulate=False)

    def _run(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
             cache: LayerCache, accumulate: bool) -> None:
        n, work, heads = step.num_rows, step.workspace, self.num_heads
        state = cache.state
        assert state is not None
        proj = work.buffer("delta.proj", self.proj_weight.shape[0], torch.float32)
        low = work.buffer("delta.low", self.decay_rank, self.ctx.dtype)
        decay = work.buffer("delta.decay", self.qk, torch.float32)
        answer = work.buffer("delta.answer", self.inner, torch.float32)
        gated = work.buffer("delta.gated", self.inner, self.ctx.dtype)
        ops.linear(hidden, self.proj_weight, None, proj, rows=n)
        ops.unary_rows(proj[:, self.low_at:], low, activation="tanh", rows=n)
        ops.linear(low, self.decay_up, self.decay_bias, decay, rows=n)
        ops.delta_scan(proj, decay, self.rate_bias, state, answer, row_start=step.row_start,
                       state_slot=step.state_slot, requests=step.num_requests, heads=heads,
                       dim=self.dim, columns=self.columns, k_offset=self.k_at,
                       v_offset=self.v_at, a_offset=self.a_at, decay_rate=self.decay_rate)
        # a head is a group of the norm: each divided by its own root mean square
        ops.rms_norm(answer, self.norm_weight, self.eps, gated, groups=heads, count=n,
                     gate=proj[:, self.g_at:self.g_at + self.inner], gate_mode="sigmoid_after")
        ops.linear(gated, self.out_weight, None, out, residual=accumulate, rows=n)
