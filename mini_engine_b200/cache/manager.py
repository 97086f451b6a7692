"""Host-side bookkeeping of the cache: pages, block tables, prefix hashes, state slots.

Keys and values live in pages of ``block_size`` token slots; token ``i`` of a request lives
in slot ``block_table[i // block_size] * block_size + i % block_size``.  Mixers whose
per-token needs are equal form a **group**; every group has a page pool of its own and every
request a block table per group.  A group whose mixers read only a window of keys gives
pages back as soon as the window has passed them.  Beside the pages there is a pool of
**slots** for per-request state of fixed size; a request holds one slot from admission to
its end whether or not a mixer of the model uses it.

Pools follow the reference's block manager (src/mini_engine/block_manager.py:38-152 of
YuvGev00/mini-engine): reference counts, a free pool in eviction order (unhashed pages
first, then least recently freed), chained content hashes given to pages once they are
full and computed, prefix matching over whole pages that always leaves one token to
compute, all-or-nothing allocation, tail-first release.  Nothing here touches tensors.
"""

from __future__ import annotations

import hashlib
import itertools
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Sequence as Seq

NULL_PAGE = -1  # block-table entry of a page that a window has passed and that was given back
ROOT_HASH = b""


def hash_page(parent: bytes, token_ids: Seq[int]) -> bytes:
    """Chained 16-byte hash of a full page: equal hashes mean equal whole prefixes.
    Independent of the process, so hashes of different runs can be compared
    (src/mini_engine/block_manager.py:26-32)."""
    digest = hashlib.blake2b(parent, digest_size=16)
    digest.update(b"".join(int(t).to_bytes(4, "little", signed=False) for t in token_ids))
    return digest.digest()


@dataclass(frozen=True)
class GroupSpec:
    """What the manager needs to know of a cache group.

    ``num_blocks`` is the size of the group's own page pool (``None``: the manager's default); a
    group with a window needs far fewer pages than one that keeps every key.  ``shareable`` says
    whether what the group holds for a prefix can be found again by content hash; a group that
    cannot offer that (per-request state without snapshots, for one) says so here, and because a
    prefix hit skips the shared tokens in *every* layer, one such group means that requests of
    this model are always computed from their first token."""

    name: str
    window: int | None = None  # None: every key is kept
    num_blocks: int | None = None
    shareable: bool = True


@dataclass(frozen=True)
class SlotGroupSpec:
    """Per-request state of fixed size, kept in one slot per live request."""

    name: str
    shareable: bool = False  # no snapshot of the state exists at page boundaries


@dataclass
class RequestCache:
    """What one request holds: a block table per group, its page hashes, its state slot."""

    block_tables: list[list[int]]
    page_hashes: list[bytes] = field(default_factory=list)
    state_slot: int = -1
    version: int = 0  # grows whenever a block table changes: whoever keeps a copy knows when it is stale
    serial: int = field(default_factory=itertools.count().__next__)  # unlike id(), never used twice
    packed: object = field(default=None, repr=False, compare=False)  # the step function's copy of the tables

    def holds_nothing(self) -> bool:
        return self.state_slot < 0 and not any(self.block_tables)


class PagePool:
    """Pages of one group: reference counts, free pool, content hashes."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.ref_counts = [0] * num_pages
        self.page_hash: list[bytes | None] = [None] * num_pages
        self.hash_to_page: dict[bytes, int] = {}
        # Pages with no holder, front = handed out (and, if hashed, evicted) first.
        self.free_pool: OrderedDict[int, None] = OrderedDict((i, None) for i in range(num_pages))
        self.num_evictions = 0

    @property
    def num_free(self) -> int:
        return len(self.free_pool)

    def take_fresh(self) -> int:
        page, _ = self.free_pool.popitem(last=False)
        held = self.page_hash[page]
        if held is not None:  # its content is about to be overwritten
            del self.hash_to_page[held]
            self.page_hash[page] = None
            self.num_evictions += 1
        self.ref_counts[page] = 1
        return page

    def share(self, page: int) -> None:
        if self.ref_counts[page] == 0:
            del self.free_pool[page]
        self.ref_counts[page] += 1

    def release(self, page: int) -> None:
        if self.ref_counts[page] <= 0:
            raise AssertionError(f"page {page} freed twice")
        self.ref_counts[page] -= 1
        if self.ref_counts[page] == 0:
            self.free_pool[page] = None
            if self.page_hash[page] is None:
                self.free_pool.move_to_end(page, last=False)

    def set_hash(self, page: int, value: bytes) -> None:
        # First writer wins: a second page with the same content stays a private copy.
        if self.page_hash[page] is None and value not in self.hash_to_page:
            self.page_hash[page] = value
            self.hash_to_page[value] = page

    def reset_hashes(self) -> None:
        for value, page in self.hash_to_page.items():
            assert self.page_hash[page] == value
            self.page_hash[page] = None
        self.hash_to_page.clear()


class SlotPool:
    """Slots for per-request state of fixed size."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self.free: list[int] = list(range(num_slots - 1, -1, -1))
        self.held: set[int] = set()

    def take(self) -> int | None:
        if not self.free:
            return None
        slot = self.free.pop()
        self.held.add(slot)
        return slot

    def give_back(self, slot: int) -> None:
        if slot not in self.held:
            raise AssertionError(f"state slot {slot} freed twice")
        self.held.remove(slot)
        self.free.append(slot)


class CacheManager:
    def __init__(
        self,
        groups: Seq[GroupSpec],
        num_blocks: int,
        block_size: int,
        max_num_seqs: int,
        enable_prefix_caching: bool = True,
        slot_groups: Seq[SlotGroupSpec] = (),
    ):
        if num_blocks < 1 or block_size < 1 or max_num_seqs < 1:
            raise ValueError("num_blocks, block_size and max_num_seqs must be positive")
        self.groups = list(groups)
        self.slot_groups = list(slot_groups)
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.pools = [PagePool(g.num_blocks or num_blocks) for g in self.groups]
        self.slots = SlotPool(max_num_seqs)
        # A prefix hit skips the computation of the shared tokens in every layer.  That is only
        # sound when each group can supply what those tokens left behind: a group that keeps every
        # key, all their pages; a group with a window, the pages that the window still reaches at
        # the end of the shared prefix; a group that says it is not shareable, nothing.
        shareable = all(g.shareable for g in [*self.groups, *self.slot_groups])
        self.enable_prefix_caching = enable_prefix_caching and shareable and bool(self.groups)

    # ------------------------------------------------------------------ queries

    def new_request(self) -> RequestCache:
        return RequestCache(block_tables=[[] for _ in self.groups])

    def blocks_needed(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)

    @property
    def num_free_blocks(self) -> int:
        """Free pages of the tightest group."""
        return min((p.num_free for p in self.pools), default=self.num_blocks)

    @property
    def smallest_pool(self) -> int:
        """Pages that a single request could ever hold in a group that keeps every key (a group
        with a window never holds a whole request, so its pool does not bound a request)."""
        return min((p.num_pages for g, p in zip(self.groups, self.pools) if g.window is None), default=self.num_blocks)

    @property
    def num_evictions(self) -> int:
        return sum(p.num_evictions for p in self.pools)

    def _first_needed_page(self, group: GroupSpec, num_computed: int) -> int:
        """Pages below this index are behind the group's window once ``num_computed`` tokens
        are in the cache: the next query, at position ``num_computed``, reads keys at
        positions ``> num_computed - window``."""
        if group.window is None:
            return 0
        return max(0, num_computed - group.window + 1) // self.block_size

    def match_prefix(self, token_ids: Seq[int]) -> list[list[int]]:
        """Per group, the block table of the longest prefix of ``token_ids`` that the cache still
        holds, in whole pages (the same length in every group).  Only the first ``len - 1`` tokens
        are eligible: at least one token must be computed to have logits for the next
        (src/mini_engine/block_manager.py:62-79).  A group that keeps every key must hold every
        page of the prefix; a group with a window only those that the window still reaches from
        the prefix's end, and its table has ``NULL_PAGE`` before them."""
        if not self.enable_prefix_caching:
            return [[] for _ in self.groups]
        bs = self.block_size
        found: list[list[int | None]] = [[] for _ in self.groups]
        parent = ROOT_HASH
        best = 0
        for i in range((len(token_ids) - 1) // bs):
            parent = hash_page(parent, token_ids[i * bs : (i + 1) * bs])
            stop = False
            for group, pool, pages in zip(self.groups, self.pools, found):
                page = pool.hash_to_page.get(parent)
                pages.append(page)
                if page is None and group.window is None:
                    stop = True  # a full group has a gap: nothing longer can be whole
            if stop:
                break
            length = i + 1
            if all(
                None not in pages[self._first_needed_page(group, length * bs) : length]
                for group, pages in zip(self.groups, found)
            ):
                best = length
        hits: list[list[int]] = []
        for group, pages in zip(self.groups, found):
            first = self._first_needed_page(group, best * bs)
            hits.append([NULL_PAGE if i < first else pages[i] for i in range(best)])
        return hits

    # ---------------------------------------------------------------- mutations

    def try_allocate(
        self, req: RequestCache, num_tokens: int, cached: Seq[Seq[int]] | None = None
    ) -> bool:
        """Grow every block table of ``req`` to hold ``num_tokens`` tokens and make sure it
        has a state slot.  All or nothing: on failure nothing changes.  ``cached`` (from
        :meth:`match_prefix`) may only seed empty tables; those pages are shared, not taken
        (src/mini_engine/block_manager.py:83-105)."""
        cached = cached if cached is not None else [[] for _ in self.groups]
        target = self.blocks_needed(num_tokens)
        for pool, table, seed in zip(self.pools, req.block_tables, cached):
            if seed and table:
                raise ValueError("cached pages can only seed an empty block table")
            fresh = max(target - len(table) - len(seed), 0)
            revived = sum(1 for page in seed if page != NULL_PAGE and pool.ref_counts[page] == 0)
            if fresh + revived > pool.num_free:
                return False
        if req.state_slot < 0:
            slot = self.slots.take()
            if slot is None:
                return False
            req.state_slot = slot
        for pool, table, seed in zip(self.pools, req.block_tables, cached):
            for page in seed:
                if page != NULL_PAGE:
                    pool.share(page)
                table.append(page)
                req.version += 1
            while len(table) < target:
                table.append(pool.take_fresh())
                req.version += 1
        return True

    def release_behind_window(self, req: RequestCache, num_computed: int) -> int:
        """Give back the pages that a group's window has passed for good; their table
        entries become ``NULL_PAGE``.  Returns how many pages were given back."""
        count = 0
        for group, pool, table in zip(self.groups, self.pools, req.block_tables):
            for i in range(min(self._first_needed_page(group, num_computed), len(table))):
                if table[i] != NULL_PAGE:
                    pool.release(table[i])
                    table[i] = NULL_PAGE
                    count += 1
        req.version += count
        return count

    def free(self, req: RequestCache) -> None:
        """Drop everything the request holds.  Pages go back tail first, so that among
        pages freed together the more shareable head is evicted last
        (src/mini_engine/block_manager.py:107-118)."""
        for pool, table in zip(self.pools, req.block_tables):
            for page in reversed(table):
                if page != NULL_PAGE:
                    pool.release(page)
            table.clear()
        req.version += 1
        req.page_hashes.clear()
        if req.state_slot >= 0:
            self.slots.give_back(req.state_slot)
            req.state_slot = -1

    def register_computed(self, req: RequestCache, token_ids: Seq[int], num_computed: int) -> None:
        """Hash every page that became full and computed since the last call, generated
        tokens included (src/mini_engine/block_manager.py:120-134)."""
        if not self.enable_prefix_caching:
            return
        bs = self.block_size
        for i in range(len(req.page_hashes), num_computed // bs):
            parent = req.page_hashes[-1] if req.page_hashes else ROOT_HASH
            value = hash_page(parent, token_ids[i * bs : (i + 1) * bs])
            req.page_hashes.append(value)
            for pool, table in zip(self.pools, req.block_tables):
                if table[i] != NULL_PAGE:  # a page behind a window that a prefix hit never held
                    pool.set_hash(table[i], value)

    def reset_prefix_cache(self) -> None:
        for pool in self.pools:
            pool.reset_hashes()

    # ------------------------------------------------------------------- checks

    def check_invariants(self, live: Seq[RequestCache]) -> None:
        """No page lost, held twice without a count for it, or free while held; the same
        for state slots.  Raises AssertionError with the first violation."""
        for g, pool in enumerate(self.pools):
            uses = [0] * pool.num_pages
            for req in live:
                for page in req.block_tables[g]:
                    if page != NULL_PAGE:
                        uses[page] += 1
            for page in range(pool.num_pages):
                assert pool.ref_counts[page] == uses[page], (
                    f"group {g} page {page}: count {pool.ref_counts[page]} but {uses[page]} table entries"
                )
                assert (page in pool.free_pool) == (uses[page] == 0), f"group {g} page {page}: free pool wrong"
            for value, page in pool.hash_to_page.items():
                assert pool.page_hash[page] == value, f"group {g}: hash map and page {page} disagree"
            assert sum(h is not None for h in pool.page_hash) == len(pool.hash_to_page)
        held = [req.state_slot for req in live if req.state_slot >= 0]
        assert len(held) == len(set(held)), "a state slot is held twice"
        assert set(held) == self.slots.held, "state slots held do not match the live requests"
        assert len(self.slots.free) + len(held) == self.slots.num_slots, "a state slot was lost"
