"""Latent attention: keys and values are up-projections of one small cached row per token."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, CacheNeed, Part, register_part
from ayaka_b200.parts.context import LayerCache, StepContext
from ayaka_b200.parts.mixer import Mixer, attend_paged
from ayaka_b200.parts.spec import PartSpec

__all__ = ["LatentAttention"]


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Multi-head attention over a low-rank cache.

    One fused projection of the normed input gives, per row, the heads' queries
    (``[dim unrotated | rot rotated]`` each), a raw latent of ``rank`` entries with one raw
    key piece of ``rot`` entries that all heads share, and the output gate. The latent is
    normalised by its root mean square (plain weight), the key piece and the queries' rotated
    parts are turned by the position (``rot_dims`` of their ``rot`` entries), and only
    ``[latent | key piece]`` goes to the cache: ``rank + rot`` values per token whatever the
    number of heads. Head ``h`` scores ``scale * (q_plain . W_uk,h c + q_rot . kr)`` over the
    last ``window`` keys (0: all) and sums ``W_uv,h c`` with softmax weights; the joined heads
    are multiplied by ``sigmoid(gate)`` and projected back into the residual stream.

    The up-projections are applied on the query's side (``W_uk,h^T q_plain`` before the
    scores, ``W_uv,h`` after the weighted sum of latents), never to cached rows:
    ``csrc/latent_attention.cu``. What is left between the two is attention of ``num_heads``
    query heads over *one* key head whose rows are also its values (the sum over whole rows
    ``[c | kr]`` holds the sum over ``c`` in its first ``rank`` entries): when ``rank + rot``
    is a head size the engine's attention kernels take (a multiple of 16 up to 256), those run
    it, tensor cores and all, with the latent pages as keys and as values; any other size
    goes to the kernel of ``csrc/latent_attention.cu``.

    Options: with ``query_rank`` the queries go through a latent of their own,
    ``q = W_uq rms(W_dq h) * w`` (plain weight, the same ``eps``); ``gate=False`` leaves the
    output gate out; ``shares_latent=True`` is a layer without a down-projection of its own:
    it reads the latent rows another run of the order stored (``Run.reads_cache_of``) with its
    own up-projections, queries and window. ``rot`` may be 0 (no positions in the scores).

    Spec parameters: ``width``, ``num_heads``, ``dim``, ``rot``, ``value_dim``, ``rank``,
    ``scale``, ``window`` (0 = none), ``rot_dims``, ``rot_base``, ``rot_layout``
    (``neighbours`` when absent), ``eps`` (of the norms), ``query_rank`` (0 when absent),
    ``gate`` (true when absent), ``shares_latent`` (false when absent).
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext, position: Part | None = None) -> None:
        super().__init__(ctx)
        self.width = int(spec.width)  # type: ignore[arg-type]
        self.num_heads = int(spec.num_heads)  # type: ignore[arg-type]
        self.dim = int(spec.dim)  # type: ignore[arg-type]
        self.rot = int(spec.get("rot", 0))  # type: ignore[arg-type]
        self.value_dim = int(spec.value_dim)  # type: ignore[arg-type]
        self.rank = int(spec.rank)  # type: ignore[arg-type]
        self.scale = float(spec.scale)  # type: ignore[arg-type]
        self.window = int(spec.get("window", 0))  # type: ignore[arg-type]
        self.rot_dims = int(spec.get("rot_dims", self.rot))  # type: ignore[arg-type]
        self.rot_base = float(spec.get("rot_base", 10000.0))  # type: ignore[arg-type]
        self.rot_layout = str(spec.get("rot_layout", "neighbours"))
        self.eps = float(spec.eps)  # type: ignore[arg-type]
        self.query_rank = int(spec.get("query_rank", 0))  # type: ignore[arg-type]
        self.gated = bool(spec.get("gate", True))
        self.shares_latent = bool(spec.get("shares_latent", False))
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.rot:
            raise ValueError(f"rot_dims must be even and at most rot ({self.rot}), got "
                             f"{self.rot_dims}")
        if min(self.num_heads, self.rank, self.value_dim) < 1 or self.dim < 1 or \
                self.window < 0 or self.query_rank < 0:
            raise ValueError("latent attention needs heads, dim, rank and value_dim >= 1")
        self.q_width = self.num_heads * (self.dim + self.rot)
        self.kv_width = self.rank + self.rot
        self.out_width = self.num_heads * self.value_dim
        # one product of the layer's input: the queries (or their latent), then the raw
        # latent and key piece (a layer that stores them), then the gate
        own = 0 if self.shares_latent else self.kv_width
        first = self.query_rank or self.q_width
        self.kv_offset = self.q_width + self.query_rank
        self.gate_offset = self.kv_offset + own
        rows = first + own + (self.out_width if self.gated else 0)
        self.proj_weight = self.add_param("proj.weight", (rows, self.width), "matrix")
        self.q_norm = self.q_up = None
        if self.query_rank:
            self.q_norm = self.add_param("q_norm.weight", (self.query_rank,), "vector")
            self.q_up = self.add_param("q_up.weight", (self.q_width, self.query_rank), "matrix")
        self.latent_norm = None if self.shares_latent else \
            self.add_param("latent_norm.weight", (self.rank,), "vector")
        self.up_key = self.add_param("up_key.weight", (self.num_heads * self.dim, self.rank),
                                     "matrix")
        self.up_value = self.add_param("up_value.weight", (self.out_width, self.rank), "matrix")
        self.out_weight = self.add_param("out.weight", (self.width, self.out_width), "matrix")
        self._freq: torch.Tensor | None = None
        self._no_weight: torch.Tensor | None = None

    def cache_need(self) -> CacheNeed:
        return CacheNeed(1, self.kv_width, self.window, values=False)

    def forward(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                cache: LayerCache) -> None:
        self._run(hidden, residual, step, cache, accumulate=True)

    def forward_into(self, hidden: torch.Tensor, out: torch.Tensor, step: StepContext,
                     cache: LayerCache) -> None:
        """The same, written into ``out`` (fp32 ``[N, width]``) instead of added to it."""
        self._run(hidden, out, step, cache, accumulate=False)

    def _run(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
             cache: LayerCache, accumulate: bool) -> None:
        n, dtype, work = step.num_rows, self.ctx.dtype, step.workspace
        heads, rank = self.num_heads, self.rank
        if self._freq is None:
            self._freq = ops.rope_frequencies(max(self.rot_dims, 0), self.rot_base, hidden.device)
            self._no_weight = torch.ones(rank, dtype=torch.float32, device=hidden.device)
        if cache.writes == self.shares_latent:
            raise ValueError("a latent attention layer either stores its latents or reads "
                             "another run's (Run.reads_cache_of), as its spec says")
        group = step.groups[cache.group]  # type: ignore[index]
        proj = work.buffer(
            "latent.proj", self.proj_weight.shape[0] + (self.q_width if self.query_rank else 0),
            torch.float32)
        q_plain = work.buffer("latent.q_plain", heads * self.dim, dtype)
        qa = work.buffer("latent.query", heads * self.kv_width, dtype)
        shared = self.kv_width % 16 == 0 and self.kv_width <= 256
        mixed = work.buffer("latent.mixed", heads * (self.kv_width if shared else rank), dtype)
        attended = work.buffer("latent.out", self.out_width, dtype)
        if self.query_rank:
            # columns: [queries | query latent | raw latent, key piece | gate]
            low = work.buffer("latent.query_latent", self.query_rank, dtype)
            ops.linear(hidden, self.proj_weight, None, proj[:, self.q_width:], rows=n)
            ops.rms_norm(proj[:, self.q_width:self.kv_offset], self.q_norm, self.eps, low,
                         count=n)
            ops.linear(low, self.q_up, None, proj[:, :self.q_width], rows=n)
        else:
            ops.linear(hidden, self.proj_weight, None, proj[:, :self.proj_weight.shape[0]],
                       rows=n)
        ops.latent_prepare(
            proj, kv_offset=self.kv_offset,
            latent_weight=self._no_weight if self.latent_norm is None else self.latent_norm,
            eps=self.eps, positions=step.positions, slot_mapping=group.slot_mapping,
            freq=self._freq, layout=self.rot_layout,
            pages=cache.k_pages if cache.writes else None,
            q_plain=q_plain, qa=qa, heads=heads, dim=self.dim, rot=self.rot, rank=rank, rows=n)
        # the queries' unrotated parts, taken to latent space: qa[:, h, :rank] = W_uk,h^T q
        ops.head_linear(q_plain, self.up_key, qa, heads=heads, transposed=True, rows=n)
        taken = False
        if step.decode_only:
            # single rows: the kernel that fetches a latent row once for all heads
            reach = min(step.max_kv_len, self.window) if self.window else step.max_kv_len
            splits = ops.latent_decode_splits(n, heads, reach, hidden.device)
            partial = work.buffer("latent.partial", heads * (rank + 2), torch.float32,
                                  rows=n * splits)
            taken = ops.latent_decode(qa, cache.k_pages, group.block_table,
                                      step.request_of_row, step.positions, mixed, partial,
                                      num_heads=heads, rank=rank, scale=self.scale,
                                      window=self.window, rows=n, splits=splits)
        if taken:
            pass
        elif shared:
            attend_paged(qa, cache.k_pages, cache.k_pages, mixed, step, group, num_heads=heads,
                         scale=self.scale, window=self.window, dtype=dtype)
        else:
            ops.latent_attention(qa, cache.k_pages, group.block_table, step.request_of_row,
                                 step.positions, mixed, num_heads=heads, rank=rank,
                                 scale=self.scale, window=self.window, rows=n)
        gate = proj[:, self.gate_offset:self.gate_offset + self.out_width] if self.gated \
            else None
        ops.head_linear(mixed, self.up_value, attended, heads=heads, transposed=False, rows=n,
                        gate=gate, inner=rank)
        ops.linear(attended, self.out_weight, None, residual, residual=accumulate, rows=n)
