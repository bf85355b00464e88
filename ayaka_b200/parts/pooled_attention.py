"""Softmax attention with a sliding window, pooled blocks behind the window, and a sink."""

from __future__ import annotations

import math

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, CacheNeed, Part, register_part
from ayaka_b200.parts.context import LayerCache, StepContext
from ayaka_b200.parts.mixer import Mixer, leading_single_rows
from ayaka_b200.parts.spec import PartSpec

__all__ = ["PooledWindowAttention", "blended_frequencies"]


def blended_frequencies(dims: int, base: float, *, factor: float = 1.0, original: float = 0.0,
                        fast: float = 0.0, slow: float = 0.0) -> tuple[list[float], float]:
    """Rotary frequencies ``f_i = base^(-2i / dims)`` for the ``dims / 2`` pairs and the gain on
    cosine and sine. With ``factor`` > 1 the frequencies are blended for contexts longer than
    ``original``: a pair that makes ``t`` turns over ``original`` positions has the index
    ``d(t) = dims * ln(original / (2 pi t)) / (2 ln base)``; with ``lo = max(floor(d(fast)), 0)``,
    ``hi = min(ceil(d(slow)), dims - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001),
    0, 1)`` the frequency is ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``, and the gain is
    ``0.1 * ln(factor) + 1``."""
    half = dims // 2
    freq = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if not factor or factor == 1.0 or not original:
        return freq, 1.0

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(freq):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


@register_part("mixer", "pooled_window_attention")
class PooledWindowAttention(Mixer):
    """Grouped softmax attention over paged keys whose far past is seen in pooled blocks.

    One fused projection gives queries (``num_heads x head_dim``) and keys (``num_kv_heads x
    head_dim``); with ``values_from_keys`` a token's value is its key as projected (before norm
    and rotation) and there is no value projection. With ``qk_norm`` every query head and key
    head is divided by its own root mean square and multiplied by one weight of ``head_dim``
    entries shared by the heads. The first ``rot_dims`` entries of each head are rotated by the
    position (entry ``i`` with ``i + rot_dims / 2``) with the frequencies and gain of
    :func:`blended_frequencies`. ``score = scale * q . k``. The query at position ``p`` sees
    the keys ``j`` with ``0 <= p - j < window`` and, with ``pool`` = P, one key and value for
    every block of P positions that lies wholly behind its window (block ``e`` when
    ``e P + P - 1 <= p - window``): the means of the block's cached keys and values. With
    ``sink`` the softmax's denominator also holds ``exp(sink_h)``, one learned number per head.

    The cache keeps every page (a pooled row lives in the page of its block's first token, and
    a block's mean is formed from the pages when its last token arrives), so ``window`` bounds
    what a row reads, not what a request holds.

    Spec parameters: ``width``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``,
    ``window``, ``pool``, ``qk_norm``, ``eps``, ``sink``, ``values_from_keys``, ``rot_dims``,
    ``rot_base``, ``rot_factor``, ``rot_original``, ``rot_fast``, ``rot_slow``.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext, position: Part | None = None) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.num_heads = heads = int(spec.num_heads)  # type: ignore[arg-type]
        self.num_kv_heads = kv_heads = int(spec.num_kv_heads)  # type: ignore[arg-type]
        self.head_dim = dim = int(spec.head_dim)  # type: ignore[arg-type]
        self.scale = float(spec.scale)  # type: ignore[arg-type]
        self.window = int(spec.get("window", 0))  # type: ignore[arg-type]
        self.pool = int(spec.get("pool", 0)) if self.window else 0  # type: ignore[arg-type]
        self.eps = float(spec.get("eps", 1e-6))  # type: ignore[arg-type]
        self.rot_dims = int(spec.get("rot_dims", 0))  # type: ignore[arg-type]
        if heads < 1 or kv_heads < 1 or heads % kv_heads:
            raise ValueError(f"num_kv_heads ({kv_heads}) must divide num_heads ({heads})")
        if dim < 1 or self.window < 0 or self.pool < 0 or self.rot_dims < 0 or \
                self.rot_dims % 2 or self.rot_dims > dim:
            raise ValueError("pooled window attention needs head_dim >= 1, window, pool >= 0 "
                             "and an even rot_dims of at most head_dim")
        if not spec.get("values_from_keys", True):
            raise ValueError("pooled window attention takes its values from the keys")
        self.q_width, self.k_width = heads * dim, kv_heads * dim
        self.proj_weight = self.add_param("proj.weight", (self.q_width + self.k_width,
                                                          self.width), "matrix")
        self.q_norm = self.k_norm = None
        if spec.get("qk_norm", False):
            self.q_norm = self.add_param("q_norm.weight", (dim,), "vector")
            self.k_norm = self.add_param("k_norm.weight", (dim,), "vector")
        self.sink = self.add_param("sink", (heads,), "vector") if spec.get("sink", False) \
            else None
        self.out_weight = self.add_param("out.weight", (self.width, self.q_width), "matrix")
        self.freq = None
        self.rot_gain = 1.0
        if self.rot_dims:
            values, self.rot_gain = blended_frequencies(
                self.rot_dims, float(spec.rot_base),  # type: ignore[arg-type]
                factor=float(spec.get("rot_factor", 1.0)),  # type: ignore[arg-type]
                original=float(spec.get("rot_original", 0.0)),  # type: ignore[arg-type]
                fast=float(spec.get("rot_fast", 0.0)),  # type: ignore[arg-type]
                slow=float(spec.get("rot_slow", 0.0)))  # type: ignore[arg-type]
            self.freq = torch.tensor(values, dtype=torch.float64, device=ctx.device)

    def cache_need(self) -> CacheNeed:
        # every page stays: the pooled rows lie in the pages of their blocks' first tokens
        return CacheNeed(self.num_kv_heads, self.head_dim, 0 if self.pool else self.window,
                         pool=self.pool)

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
        heads, dim = self.num_heads, self.head_dim
        proj = work.buffer("pooled_attention.proj", self.proj_weight.shape[0], torch.float32)
        q = work.buffer("pooled_attention.q", self.q_width, dtype)
        attended = work.buffer("pooled_attention.out", self.q_width, dtype)
        ops.linear(hidden, self.proj_weight, None, proj, rows=n)
        ops.pooled_prepare(
            proj, k_offset=self.q_width, q_weight=self.q_norm, k_weight=self.k_norm,
            eps=self.eps, positions=step.positions, freq=self.freq, rot_dims=self.rot_dims,
            rot_gain=self.rot_gain, slot_mapping=group.slot_mapping,
            k_pages=cache.k_pages if cache.writes else None,
            v_pages=cache.v_pages if cache.writes else None, q=q, heads=heads,
            kv_heads=self.num_kv_heads, dim=dim, rows=n)
        if self.pool and cache.writes:
            ops.pooled_blocks(cache.k_pages, cache.v_pages, cache.k_pool, cache.v_pool,
                              group.block_table, step.request_of_row, step.positions,
                              step.row_start, pool=self.pool, rows=n,
                              requests=step.num_requests)
        # Prompt portions in bfloat16, where the sizes are the tensor-core kernel's: the
        # engine's flash kernel, told of the pooled rows and the sink. Single rows (a decode
        # step, or the decoding requests that lead a mixed step) go to the kernel of shares,
        # every other size or type to the generic kernel.
        tiled = dtype == torch.bfloat16 and not step.decode_only and dim % 16 == 0 and \
            dim <= 256 and ops.POOLED_PREFILL == "mma"
        lead = leading_single_rows(step.host_rows) if tiled else n
        taken = 0
        if lead and (step.decode_only or tiled):
            reach = step.max_kv_len
            if self.window:
                reach = min(reach, self.window) + \
                    (max(0, step.max_kv_len - self.window) // self.pool if self.pool else 0)
            shares = ops.gated_decode_shares(lead, heads, reach, hidden.device)
            partial = None if shares == 1 else work.buffer(
                "pooled_attention.partial", heads * (dim + 2), torch.float32, rows=n * shares)
            if ops.pooled_attention(
                    q, cache.k_pages, cache.v_pages, cache.k_pool, cache.v_pool,
                    group.block_table, step.request_of_row, step.positions, attended,
                    heads=heads, scale=self.scale, window=self.window, pool=self.pool,
                    sink=self.sink, rows=lead, shares=shares, partial=partial):
                lead, taken = 0, lead
        if lead:
            ops.pooled_attention(
                q, cache.k_pages, cache.v_pages, cache.k_pool, cache.v_pool, group.block_table,
                step.request_of_row, step.positions, attended, heads=heads, scale=self.scale,
                window=self.window, pool=self.pool, sink=self.sink, rows=lead)
        lead = lead or taken
        if tiled:
            ops.attention_prefill(
                q, cache.k_pages, cache.v_pages, group.block_table[lead:],
                step.row_start[lead:], step.kv_len[lead:], attended, num_heads=heads,
                scale=self.scale, host_rows=step.host_rows[lead:], window=self.window,
                pool=self.pool, k_pool=cache.k_pool, v_pool=cache.v_pool, sink=self.sink)
        ops.linear(attended, self.out_weight, None, out, residual=accumulate, rows=n)
