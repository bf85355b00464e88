"""Softmax attention with a window that keeps the first tokens, and an output gate."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, CacheNeed, Part, register_part
from ayaka_b200.parts.context import LayerCache, StepContext
from ayaka_b200.parts.mixer import Mixer, leading_single_rows
from ayaka_b200.parts.spec import PartSpec

__all__ = ["GatedAttention"]


@register_part("mixer", "gated_attention")
class GatedAttention(Mixer):
    """Grouped softmax attention over paged keys and values, without positions in its scores.

    One fused projection gives queries (``num_heads x head_dim``), keys (``num_kv_heads x
    head_dim``), values (``num_kv_heads x value_dim``) and, with ``gate``, one raw gate per
    entry of the joined heads. With ``qk_norm`` the whole query projection and the whole key
    projection are each normalised by their root mean square (all heads at once, a plain weight
    per entry). Query head ``h`` uses key/value head ``h // (num_heads / num_kv_heads)``;
    ``score = scale * q . k``; the query at position ``p`` sees key ``j <= p`` when
    ``p - j < window`` (``window`` 0: every earlier key) or ``j < keep_first``: the sequence's
    first tokens stay in sight at their true positions; softmax in fp32; the joined heads are
    multiplied entry by entry by ``sigmoid(gate)``; then the output projection.

    Spec parameters: ``width``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``value_dim``,
    ``scale``, ``window``, ``keep_first``, ``qk_norm``, ``eps``, ``gate``.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext, position: Part | None = None) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.num_heads = heads = int(spec.num_heads)  # type: ignore[arg-type]
        self.num_kv_heads = kv_heads = int(spec.num_kv_heads)  # type: ignore[arg-type]
        self.head_dim = dim = int(spec.head_dim)  # type: ignore[arg-type]
        self.value_dim = vdim = int(spec.get("value_dim", dim))  # type: ignore[arg-type]
        self.scale = float(spec.scale)  # type: ignore[arg-type]
        self.window = int(spec.get("window", 0))  # type: ignore[arg-type]
        self.keep_first = int(spec.get("keep_first", 0))  # type: ignore[arg-type]
        self.eps = float(spec.get("eps", 1e-6))  # type: ignore[arg-type]
        self.gated = bool(spec.get("gate", False))
        if heads < 1 or kv_heads < 1 or heads % kv_heads:
            raise ValueError(f"num_kv_heads ({kv_heads}) must divide num_heads ({heads})")
        if dim < 1 or vdim < 1 or self.window < 0 or self.keep_first < 0:
            raise ValueError("gated attention needs head_dim, value_dim >= 1 and window, "
                             "keep_first >= 0")
        self.q_width, self.k_width, self.v_width = heads * dim, kv_heads * dim, kv_heads * vdim
        self.qkv_width = self.q_width + self.k_width + self.v_width
        self.out_width = heads * vdim
        out_features = self.qkv_width + (self.out_width if self.gated else 0)
        self.proj_weight = self.add_param("proj.weight", (out_features, self.width), "matrix")
        self.q_norm = self.k_norm = None
        if spec.get("qk_norm", False):
            self.q_norm = self.add_param("q_norm.weight", (self.q_width,), "vector")
            self.k_norm = self.add_param("k_norm.weight", (self.k_width,), "vector")
        self.out_weight = self.add_param("out.weight", (self.width, self.out_width), "matrix")

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window,
                         value_dim=0 if self.value_dim == self.head_dim else self.value_dim,
                         keep_first=self.keep_first if self.window else 0)

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache) -> None:
        self._run(hidden, residual, step, cache, accumulate=True)

    def forward_into(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
                     cache: LayerCache) -> None:
        """The same, written into ``out`` (fp32 ``[N, width]``) instead of added to it."""
        self._run(hidden, out, step, cache, accumulate=False)

    def _run(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
             cache: LayerCache, accumulate: bool) -> None:
        n, dtype, work = step.num_rows, self.ctx.dtype, step.workspace
        group = step.groups[cache.group]  # type: ignore[index]
        proj = work.buffer("gated_attention.proj", self.proj_weight.shape[0], torch.float32)
        q = work.buffer("gated_attention.q", self.q_width, dtype)
        attended = work.buffer("gated_attention.out", self.out_width, dtype)
        ops.linear(hidden, self.proj_weight, None, proj, rows=n)
        ops.gated_attention_prepare(
            proj, k_offset=self.q_width, v_offset=self.q_width + self.k_width,
            q_weight=self.q_norm, k_weight=self.k_norm, eps=self.eps,
            slot_mapping=group.slot_mapping, k_pages=cache.k_pages if cache.writes else None,
            v_pages=cache.v_pages if cache.writes else None, q=q, heads=self.num_heads,
            kv_heads=self.num_kv_heads, dim=self.head_dim, vdim=self.value_dim, rows=n)
        gate = proj[:, self.qkv_width:] if self.gated else None
        # Prompt portions in bfloat16, where the sizes are the tensor-core kernel's: the
        # engine's flash kernel, told of the kept keys, the value size and the gate. Single
        # rows (a decode step, or the decoding requests that lead a mixed step) and every
        # other size or type go to this part's own kernel.
        tiled = dtype == torch.bfloat16 and not step.decode_only and \
            self.head_dim % 16 == 0 and self.value_dim % 16 == 0 and \
            max(self.head_dim, self.value_dim) <= 256
        lead = (leading_single_rows(step.host_rows) if tiled else n)
        taken = 0
        if lead and (step.decode_only or tiled):
            # single rows: a row's keys in shares, a CTA per head and share
            reach = step.max_kv_len
            if self.window:
                reach = min(reach, self.window + self.keep_first)
            shares = ops.gated_decode_shares(lead, self.num_heads, reach, hidden.device)
            partial = None if shares == 1 else work.buffer(
                "gated_attention.partial", self.num_heads * (self.value_dim + 2),
                torch.float32, rows=n * shares)
            if ops.gated_decode(
                    q, cache.k_pages, cache.v_pages, group.block_table, step.request_of_row,
                    step.positions, attended, partial, heads=self.num_heads, scale=self.scale,
                    window=self.window, keep_first=self.keep_first, gate=gate, rows=lead,
                    shares=shares):
                lead, taken = 0, lead
        if lead:
            ops.gated_attention(
                q, cache.k_pages, cache.v_pages, group.block_table, step.request_of_row,
                step.positions, attended, heads=self.num_heads, scale=self.scale,
                window=self.window, keep_first=self.keep_first, gate=gate, rows=lead)
        lead = lead or taken
        if tiled:
            ops.attention_prefill(
                q, cache.k_pages, cache.v_pages, group.block_table[lead:],
                step.row_start[lead:], step.kv_len[lead:], attended, num_heads=self.num_heads,
                scale=self.scale, host_rows=step.host_rows[lead:], window=self.window,
                keep_first=self.keep_first, gate=gate)
        ops.linear(attended, self.out_weight, None, out, residual=accumulate, rows=n)
