"""The cache's device tensors, and the plan that groups a model's runs by what they need.

Layout of a group's keys (and, separately, values):
``[cache slot, page, kv_head, token in page, head_dim]``. One cache slot per run of the
execution order that writes a cache; a run that reads another run's cache shares its slot.
All of one head's tokens in a page are contiguous (``page_size * head_dim`` elements), so an
attention kernel fetches a head's page in one bulk copy.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ayaka_b200.errors import ConfigError
from ayaka_b200.parts.base import CacheNeed, StateNeed
from ayaka_b200.parts.context import LayerCache
from ayaka_b200.parts.spec import Run

__all__ = ["CachePlan", "CacheStorage", "plan_cache"]


@dataclass(frozen=True, slots=True)
class CachePlan:
    """Which group and cache slot every run of the order uses.

    Attributes:
        groups: the distinct needs, in order of first use.
        run_group: per run, its group index or ``None`` (a mixer without pages).
        run_slot: per run, its slot inside the group's tensors or ``None``.
        run_writes: per run, whether it writes that slot (``False`` for a reader).
        slots_per_group: cache slots each group's tensors hold.
        run_state: per run, the fixed-size state its mixer asks for, or ``None``.
    """

    groups: tuple[CacheNeed, ...]
    run_group: tuple[int | None, ...]
    run_slot: tuple[int | None, ...]
    run_writes: tuple[bool, ...]
    slots_per_group: tuple[int, ...]
    run_state: tuple[StateNeed | None, ...]

    def bytes_per_page(self, group: int, itemsize: int, page_size: int) -> int:
        need = self.groups[group]
        entries = need.head_dim + (need.value_head_dim if need.values else 0)
        rows = page_size + (-(-page_size // need.pool) if need.pool else 0)
        return self.slots_per_group[group] * need.num_kv_heads * rows * entries * itemsize

    def bytes_per_token(self, itemsize: int) -> int:
        """Key and value bytes one cached token takes over all groups (windows ignored)."""
        return sum(self.bytes_per_page(g, itemsize, 1) for g in range(len(self.groups)))


def _same_rows(a: CacheNeed, b: CacheNeed) -> bool:
    """Whether two needs lay a token's rows out alike (how far back they look aside)."""
    return (a.num_kv_heads, a.head_dim, a.values, a.value_head_dim, a.pool) == \
        (b.num_kv_heads, b.head_dim, b.values, b.value_head_dim, b.pool)


def _covering(a: CacheNeed, b: CacheNeed) -> CacheNeed:
    """The need that keeps every page either of two needs with the same rows still sees."""
    if a == b:
        return a
    window = 0 if (not a.window or not b.window or a.chunk or b.chunk) \
        else max(a.window, b.window)
    chunk = a.chunk if a.chunk == b.chunk and not (a.window or b.window) else 0
    keep_first = max(a.keep_first, b.keep_first) if window else 0
    return CacheNeed(a.num_kv_heads, a.head_dim, window, a.values, chunk, a.value_dim,
                     keep_first, a.pool)


def plan_cache(order: tuple[Run, ...],
               needs: list[tuple[CacheNeed | None, StateNeed | None]]) -> CachePlan:
    """Group the runs by what they need. A run that reads another run's cache shares its
    slot; it may look back further or less far than the run that writes (a window, kept first
    tokens of its own): the slot's group then keeps what the furthest-looking of them sees."""
    owner_need: dict[int, CacheNeed] = {}
    for index, (run, (need, _)) in enumerate(zip(order, needs)):
        if need is None:
            continue
        if run.reads_cache_of is None:
            owner_need[index] = need
            continue
        owner = run.reads_cache_of
        if owner not in owner_need or order[owner].reads_cache_of is not None or \
                not _same_rows(owner_need[owner], need):
            raise ConfigError(
                "model.order", "CACHE_MISMATCH",
                f"run {index} reads the cache of run {owner}, whose geometry differs")
        owner_need[owner] = _covering(owner_need[owner], need)
    groups: list[CacheNeed] = []
    slots: list[int] = []
    run_group: list[int | None] = []
    run_slot: list[int | None] = []
    run_writes: list[bool] = []
    for index, (run, (need, _)) in enumerate(zip(order, needs)):
        if need is None:
            run_group.append(None)
            run_slot.append(None)
            run_writes.append(False)
            continue
        if run.reads_cache_of is not None:
            owner = run.reads_cache_of
            run_group.append(run_group[owner])
            run_slot.append(run_slot[owner])
            run_writes.append(False)
            continue
        need = owner_need[index]
        if need not in groups:
            groups.append(need)
            slots.append(0)
        group = groups.index(need)
        run_group.append(group)
        run_slot.append(slots[group])
        run_writes.append(True)
        slots[group] += 1
    return CachePlan(tuple(groups), tuple(run_group), tuple(run_slot), tuple(run_writes),
                     tuple(slots), tuple(state for _, state in needs))


class CacheStorage:
    """Keys, values and per-request state on the device, as the plan lays them out."""

    def __init__(self, plan: CachePlan, num_pages: list[int], page_size: int, max_requests: int,
                 dtype: torch.dtype, device: torch.device, poison: bool = False) -> None:
        self.plan = plan
        self.page_size = page_size
        self.keys: list[torch.Tensor] = []
        self.values: list[torch.Tensor | None] = []
        #: per group, the rows of pooled blocks beside the pages (keys, values) or ``None``
        self.pooled: list[tuple[torch.Tensor, torch.Tensor] | None] = []
        for need, slots, pages in zip(plan.groups, plan.slots_per_group, num_pages):
            shape = (slots, pages, need.num_kv_heads, page_size, need.head_dim)
            self.keys.append(torch.zeros(shape, dtype=dtype, device=device))
            # a group of latent rows keeps one tensor: its rows are keys and values at once
            self.values.append(torch.zeros((*shape[:-1], need.value_head_dim), dtype=dtype,
                                           device=device) if need.values else None)
            if need.pool and need.values:
                rows = -(-page_size // need.pool)
                self.pooled.append((
                    torch.zeros((slots, pages, need.num_kv_heads, rows, need.head_dim),
                                dtype=dtype, device=device),
                    torch.zeros((slots, pages, need.num_kv_heads, rows, need.value_head_dim),
                                dtype=dtype, device=device)))
            else:
                self.pooled.append(None)
        if poison:
            self.poison()
        self.states: list[torch.Tensor | None] = [
            None if need is None else
            torch.zeros((max_requests, *need.shape), dtype=need.dtype, device=device)
            for need in plan.run_state]

    def poison(self) -> None:
        """Fill every page with NaN (tests: a slot read before it is written then shows)."""
        pooled = [t for pair in self.pooled if pair is not None for t in pair]
        for tensor in (*self.keys, *self.values, *pooled):
            if tensor is not None:
                tensor.fill_(float("nan"))

    def layer_caches(self) -> list[LayerCache]:
        """One :class:`LayerCache` per run of the order."""
        out = []
        for index, group in enumerate(self.plan.run_group):
            if group is None:
                out.append(LayerCache(None, None, None, False, self.states[index]))
            else:
                slot = self.plan.run_slot[index]
                values = self.values[group]
                pooled = self.pooled[group]
                out.append(LayerCache(group, self.keys[group][slot],
                                      None if values is None else values[slot],
                                      self.plan.run_writes[index], self.states[index],
                                      None if pooled is None else pooled[0][slot],
                                      None if pooled is None else pooled[1][slot]))
        return out

    def zero_state_rows(self, rows: list[int]) -> None:
        if not rows:
            return
        for state in self.states:
            if state is not None:
                state[rows] = 0

    def nbytes(self) -> int:
        pooled = [t for pair in self.pooled if pair is not None for t in pair]
        total = sum(t.numel() * t.element_size() for t in (*self.keys, *self.values, *pooled)
                    if t is not None)
        return total + sum(t.numel() * t.element_size() for t in self.states if t is not None)
