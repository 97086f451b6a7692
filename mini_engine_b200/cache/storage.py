"""Device memory of the cache, laid out from what the model's mixers declare.

Every execution entry whose mixer keeps keys and values gets two page arrays ``[pages + 1,
kv_heads, block_size, head_dim]``: one page of one head is ``block_size * head_dim``
contiguous elements (4 KB at 16 x 128 bfloat16), which is what the attention kernels stream.
The reference keeps ``[kv_heads, pages + 1, block_size, head_dim]`` per layer
(src/mini_engine/engine.py:72-79 of YuvGev00/mini-engine) because its gather wants heads in
front; here nothing is gathered.  The last page is a spare that no request owns: padding
rows of a captured decode graph write to it and read from it.  Entries with equal needs
share a group, hence a page pool and block tables.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from mini_engine_b200.cache.manager import GroupSpec, SlotGroupSpec
from mini_engine_b200.parts.base import LayerCache, PagedCacheSpec, StateSpec


@dataclass
class CacheLayout:
    groups: list[GroupSpec]
    group_specs: list[PagedCacheSpec]
    views: list[LayerCache]  # one per execution entry
    arrays: list[torch.Tensor]  # per group [entries, 2, pages + 1, kv_heads, block_size, head_dim]
    slot_groups: list[SlotGroupSpec]  # one per execution entry whose mixer keeps per-request state
    bytes_per_token: int

    @property
    def has_state(self) -> bool:
        return bool(self.slot_groups)

    @property
    def spare_pages(self) -> list[int]:
        """Per group, the page that no request owns (the last of its array)."""
        return [g.num_blocks for g in self.groups]


def plan_groups(needs) -> tuple[list[PagedCacheSpec], list[int | None]]:
    """Group the execution entries by equal per-token need.  Returns the distinct needs and,
    per entry, its group index (``None`` for an entry without per-token cache)."""
    specs: list[PagedCacheSpec] = []
    group_of: list[int | None] = []
    for paged, _state, cache_of in needs:
        if paged is None:
            group_of.append(None)
            continue
        if cache_of is not None:
            owner = needs[cache_of][0]
            if owner != paged:
                raise ValueError(f"an entry reads a cache of {owner} but its mixer expects {paged}")
            group_of.append(group_of[cache_of])
            continue
        if paged not in specs:
            specs.append(paged)
        group_of.append(specs.index(paged))
    return specs, group_of


def pages_of_group(spec: PagedCacheSpec, num_blocks: int, block_size: int, max_num_seqs: int, max_step_tokens: int) -> int:
    """Pages of a group's pool.  A group that keeps every key gets ``num_blocks``.  A group with a
    window never holds more of a request than the window, the tokens of the step that is being
    computed (their pages are taken before the step and the pages behind the window go back after
    it) and the two pages that the ends of that range may share with their neighbours; so that
    much for every request that can be live is all it can ever use."""
    if spec.window is None:
        return num_blocks
    per_request = -(-(spec.window + max_step_tokens) // block_size) + 2
    return max(1, min(num_blocks, max_num_seqs * per_request))


def group_names(specs: list[PagedCacheSpec], pages: list[int]) -> list[GroupSpec]:
    return [
        GroupSpec(f"kv{i}:{s.kv_heads}x{s.head_dim}" + (f":w{s.window}" if s.window else ""), s.window, count)
        for i, (s, count) in enumerate(zip(specs, pages))
    ]


def bytes_per_token(
    needs: list[tuple[PagedCacheSpec | None, StateSpec | None, int | None]], dtype: torch.dtype
) -> int:
    """Bytes of keys and values that one token occupies over all order entries that own a cache."""
    element = torch.empty((), dtype=dtype).element_size()
    return sum(
        2 * paged.kv_heads * paged.head_dim * element
        for paged, _state, cache_of in needs
        if paged is not None and cache_of is None
    )


def blocks_for_budget(
    needs: list[tuple[PagedCacheSpec | None, StateSpec | None, int | None]],
    dtype: torch.dtype,
    block_size: int,
    budget_bytes: int,
) -> int:
    """Pages per group that ``budget_bytes`` of device memory hold (every group gets the same
    number of pages, and one spare page each is paid for first)."""
    per_page = bytes_per_token(needs, dtype) * block_size
    if per_page == 0:
        return 1
    blocks = budget_bytes // per_page - 1
    if blocks < 1:
        raise ValueError(
            f"{budget_bytes} bytes hold no KV page of {per_page} bytes (plus the spare page): "
            "raise kv_memory_fraction or lower block_size"
        )
    return int(blocks)


def allocate_cache(
    needs: list[tuple[PagedCacheSpec | None, StateSpec | None, int | None]],
    num_blocks: int,
    block_size: int,
    max_num_seqs: int,
    dtype: torch.dtype,
    device: str | torch.device = "cuda",
    max_step_tokens: int | None = None,
) -> CacheLayout:
    """``max_step_tokens`` (the token budget of a step) bounds what a group with a window can
    hold; without it such a group is sized like one that keeps every key."""
    specs, group_of = plan_groups(needs)
    pages = [
        pages_of_group(s, num_blocks, block_size, max_num_seqs, max_step_tokens) if max_step_tokens else num_blocks
        for s in specs
    ]
    owners: list[list[int]] = [[] for _ in specs]
    for entry, (paged, _state, cache_of) in enumerate(needs):
        if paged is not None and cache_of is None:
            owners[group_of[entry]].append(entry)
    element = torch.empty((), dtype=dtype).element_size()
    arrays = [
        torch.zeros(
            (len(entries), 2, count + 1, s.kv_heads, block_size, s.head_dim), dtype=dtype, device=device
        )
        for s, entries, count in zip(specs, owners, pages)
    ]
    views: list[LayerCache] = []
    slot_groups: list[SlotGroupSpec] = []
    for entry, (paged, state, cache_of) in enumerate(needs):
        view = LayerCache()
        if paged is not None:
            g = group_of[entry]
            owner = entry if cache_of is None else cache_of
            index = owners[g].index(owner)
            view.group, view.k, view.v = g, arrays[g][index, 0], arrays[g][index, 1]
            view.writes = cache_of is None
        if state is not None:
            slot_groups.append(SlotGroupSpec(f"state{entry}:{'x'.join(map(str, state.shape))}"))
            view.state = torch.zeros((max_num_seqs + 1, *state.shape), dtype=state.dtype, device=device)
        views.append(view)
    per_token = sum(2 * len(e) * s.kv_heads * s.head_dim * element for s, e in zip(specs, owners))
    return CacheLayout(group_names(specs, pages), specs, views, arrays, slot_groups, per_token)
