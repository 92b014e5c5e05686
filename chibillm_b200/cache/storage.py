"""Device arrays behind the cache manager, and the views that mixers get.

Keys and values of a group: one array each per run step of the group,
``[pages, kv_heads, page_size, head_dim]`` in the runtime's activation type, so
the ``page_size * head_dim`` values of one (page, head) are contiguous.
Fixed state: one array per declared name and run step, ``[slots, *shape]``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import FixedStateNeed, PagedKVNeed, Runtime
from .manager import CacheError, GroupLayout


@dataclass
class PagedKVView:
    """What an attention-like mixer sees of the cache for one run step."""

    group: str
    keys: torch.Tensor
    values: torch.Tensor
    page_size: int
    writes: bool                 # False: this run step reads another step's cache


@dataclass
class FixedStateView:
    """Per-request arrays of one run step, indexed by state slot."""

    arrays: Dict[str, torch.Tensor]


@dataclass(frozen=True)
class CachePlan:
    groups: Tuple[GroupLayout, ...]
    # per run step: ("paged", group, entry, writes) | ("state", need) | None, or, for a run step
    # whose parts have several needs, ("several", (one of these per need, ...))
    steps: Tuple[Optional[tuple], ...]
    tied: Tuple[str, ...] = ()      # groups whose values are their keys (no value arrays)
    value_dims: Tuple[Tuple[str, int], ...] = ()     # groups whose value heads have another size than their keys
    value_heads: Tuple[Tuple[str, int], ...] = ()    # groups with fewer value heads than key heads


def group_name(need: PagedKVNeed) -> str:
    base = f"kv{need.num_kv_heads}x{need.head_dim}" if not need.tied_values else f"k{need.num_kv_heads}x{need.head_dim}"
    if need.value_dim is not None and need.value_dim != need.head_dim:
        base += f"v{need.value_dim}"
    if need.value_heads is not None and need.value_heads != need.num_kv_heads:
        base += f"h{need.value_heads}"
    return base if need.window is None else f"{base}w{need.window}"


def plan_cache(needs: Sequence[object], cache_of: Sequence[Optional[int]], page_size: int,
               pool_tokens: int, max_positions: int = 0) -> CachePlan:
    """Sort the run steps' needs into groups.  ``pool_tokens`` is how many
    tokens every group's pool can hold; it is rounded up to whole pages.
    ``max_positions`` (the model's limit; default: the pool's size) bounds the
    logical blocks of one request, which is the width of the device tables."""
    if page_size <= 0 or pool_tokens <= 0:
        raise CacheError("invalid_configuration", "page_size and pool_tokens must be positive")
    num_pages = (pool_tokens + page_size - 1) // page_size
    entries: Dict[str, int] = {}
    needs_of: Dict[str, PagedKVNeed] = {}
    steps: List[Optional[tuple]] = []
    def paged_of(step):
        """The paged member of a planned step (a step of several needs has at most one)."""
        if step is not None and step[0] == "several":
            found = [m for m in step[1] if m is not None and m[0] == "paged"]
            return found[0] if found else None
        return step

    def plan_one(i, need, src):
        if src is not None and isinstance(need, PagedKVNeed):
            owner = paged_of(steps[src]) if 0 <= src < i else None
            if owner is None or owner[0] != "paged" or not owner[3]:
                raise CacheError("invalid_configuration",
                                 f"run step {i} reads the cache of step {src}, which owns no paged cache")
            theirs = needs_of[owner[1]]
            if (need.num_kv_heads, need.head_dim, need.tied_values, need.value_dim or need.head_dim,
                    need.value_heads or need.num_kv_heads) != (
                    theirs.num_kv_heads, theirs.head_dim, theirs.tied_values, theirs.value_dim or theirs.head_dim,
                    theirs.value_heads or theirs.num_kv_heads):
                raise CacheError("invalid_configuration",
                                 f"run step {i} cannot read the cache of step {src}: shapes differ")
            if need.window != theirs.window:
                # the owner's window decides which pages are given back; a reader that looks
                # further back would meet pages that are gone
                raise CacheError("invalid_configuration",
                                 f"run step {i} (window {need.window}) cannot read the cache of step {src} "
                                 f"(window {theirs.window}): the windows differ")
            return ("paged", owner[1], owner[2], False)
        if isinstance(need, PagedKVNeed):
            name = group_name(need)
            needs_of[name] = need
            entry = entries.get(name, 0)
            entries[name] = entry + 1
            return ("paged", name, entry, True)
        if isinstance(need, FixedStateNeed):
            return ("state", need)
        if need is None:
            return None
        raise CacheError("invalid_configuration", f"run step {i}: unknown cache need {need!r}")

    for i, need in enumerate(needs):
        src = cache_of[i]
        if isinstance(need, (tuple, list)):
            if sum(isinstance(n, PagedKVNeed) for n in need) > 1:
                raise CacheError("invalid_configuration", f"run step {i} asks for more than one paged cache")
            steps.append(("several", tuple(plan_one(i, n, src) for n in need)))
            continue
        if src is not None and not isinstance(need, PagedKVNeed):
            raise CacheError("invalid_configuration",
                             f"run step {i} reads the cache of step {src} but has no paged cache need")
        steps.append(plan_one(i, need, src))
    max_blocks = (max(max_positions, 1) + page_size - 1) // page_size if max_positions else num_pages
    groups = tuple(GroupLayout(name, n.num_kv_heads, n.head_dim, n.window, page_size, num_pages,
                               entries[name], max_blocks) for name, n in needs_of.items())
    return CachePlan(groups, tuple(steps), tuple(name for name, n in needs_of.items() if n.tied_values),
                     tuple((name, n.value_dim) for name, n in needs_of.items()
                           if n.value_dim is not None and n.value_dim != n.head_dim),
                     tuple((name, n.value_heads) for name, n in needs_of.items()
                           if n.value_heads is not None and n.value_heads != n.num_kv_heads))


class CacheStorage:
    def __init__(self, plan: CachePlan, runtime: Runtime, num_slots: int):
        self.plan = plan
        self.runtime = runtime
        self.num_slots = num_slots
        self.keys: Dict[str, torch.Tensor] = {}
        self.values: Dict[str, torch.Tensor] = {}
        value_dims = dict(plan.value_dims)
        value_heads = dict(plan.value_heads)
        for g in plan.groups:
            shape = (g.num_entries, g.num_pages, g.num_kv_heads, g.page_size, g.head_dim)
            self.keys[g.name] = torch.zeros(shape, dtype=runtime.dtype, device=runtime.device)
            # a group whose values are its keys holds one array; readers get it under both names
            self.values[g.name] = self.keys[g.name] if g.name in plan.tied else \
                torch.zeros(shape[:2] + (value_heads.get(g.name, g.num_kv_heads), g.page_size,
                                         value_dims.get(g.name, g.head_dim)), dtype=runtime.dtype,
                            device=runtime.device)
        # the block tables' mirror on the device: row = a request's state slot
        self.tables: Dict[str, torch.Tensor] = {
            g.name: torch.full((num_slots, max(g.max_blocks, 1)), -1, dtype=torch.int32, device=runtime.device)
            for g in plan.groups}
        self.views: List[object] = []
        self._state_arrays: List[torch.Tensor] = []
        page_sizes = {g.name: g.page_size for g in plan.groups}

        def view_of(step):
            if step is None:
                return None
            if step[0] == "several":
                return tuple(view_of(member) for member in step[1])
            if step[0] == "paged":
                _, name, entry, writes = step
                return PagedKVView(name, self.keys[name][entry], self.values[name][entry],
                                   page_sizes[name], writes)
            arrays = {}
            for aname, shape, dtype in step[1].arrays:
                dtype = runtime.dtype if dtype is None else dtype       # None: the activations' type
                t = torch.zeros((num_slots,) + tuple(shape), dtype=dtype, device=runtime.device)
                arrays[aname] = t
                self._state_arrays.append(t)
            return FixedStateView(arrays)

        for step in plan.steps:
            self.views.append(view_of(step))

    def state_views(self) -> List["FixedStateView"]:
        """Every fixed-size state view, those inside a run step of several needs included."""
        out = []
        for v in self.views:
            for member in (v if isinstance(v, tuple) else (v,)):
                if isinstance(member, FixedStateView):
                    out.append(member)
        return out

    def zero_state_slot(self, slot: int) -> None:
        for t in self._state_arrays:
            t[slot].zero_()

    def poison(self, value: float = float("nan")) -> None:
        """Fill every page with a marker (tests use NaN so that a read of a
        position that was never written shows)."""
        for t in list(self.keys.values()) + [v for n, v in self.values.items() if n not in self.plan.tied]:
            t.fill_(value)

    def bytes(self) -> int:
        total = 0
        values = [v for n, v in self.values.items() if n not in self.plan.tied]
        for t in list(self.keys.values()) + values + self._state_arrays:
            total += t.numel() * t.element_size()
        return total
