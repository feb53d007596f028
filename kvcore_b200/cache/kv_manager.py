"""Cache manager: pages per group of layers, a block table per request and group, and a
state slot per request.  Pure bookkeeping on the host; it never touches device tensors.

What the reference does per layer (one manager and one block list per layer over a common
pool: kvcore/kv/kv_manager.py:105-113, 179-257; single_type_kv_manager.py:104-182;
block_table.py:87-236) is done here per *group*: schedule entries whose mixers have the same
cache needs (kv heads, head size, window) share one pool and one block table, and every
entry of the group stores its keys/values under the same page id in its own slice of the
group's storage.  A group that keeps all keys holds a request's pages until it ends; a
windowed group hands back pages that lie wholly behind the window while the request lives
(table entry becomes the null page).  Freed pages go to the tail of the free queue, a
finished request's pages in reverse order, so pages are used again.

Tables are persistent numpy rows indexed by the request's state slot and updated
incrementally; the step function gathers the rows of the requests it runs.

Prefix reuse (off unless asked for; reference: kv_utils.py:31-68, kv_manager.py:135-177,
single_type_kv_manager.py:148-175): the full pages of a request are registered under a sha256
chain over their token ids once computed; a new request whose prompt starts with registered
pages takes them over instead of computing them (at least its last token is always computed).
Only offered when there is one group that keeps all keys and no mixer has state of its own.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Sequence

import numpy as np

from .page_pool import NULL_PAGE, PagePool
from .state_slots import StateSlotPool


@dataclass(frozen=True)
class CacheGroupSpec:
    """One group of schedule entries with equal cache needs."""

    group_id: int
    entries: tuple[int, ...]
    planes: int                  # tensors a page consists of (keys and values: 2)
    heads: int                   # a page of a plane is [heads, page_size, width]
    width: int
    window: int | None = None

    @property
    def kind(self) -> str:
        return "full" if self.window is None else "window"

    @property
    def elements_per_token(self) -> int:
        """Elements one cached token takes in one entry of the group."""
        return self.planes * self.heads * self.width


@dataclass
class _RequestState:
    slot: int
    num_computed: int = 0
    # per group: number of logical blocks in the table (freed ones included) and how many
    # leading blocks were already handed back
    num_blocks: list[int] = field(default_factory=list)
    num_released: list[int] = field(default_factory=list)
    page_keys: list[bytes] = field(default_factory=list)   # chain keys of the full pages registered so far


class KVManagerError(RuntimeError):
    pass


class KVManager:
    def __init__(
        self,
        groups: list[CacheGroupSpec],
        *,
        num_pages: int | list[int],
        page_size: int,
        max_num_seqs: int,
        max_model_len: int,
        enable_prefix_caching: bool = False,
        track_released_pages: bool = False,
    ) -> None:
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.groups = list(groups)
        self.page_size = int(page_size)
        self.max_model_len = int(max_model_len)
        self.max_blocks_per_seq = -(-self.max_model_len // self.page_size)
        counts = [num_pages] * len(self.groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(self.groups):
            raise ValueError("num_pages must give one count per group")
        self.pools = [PagePool(count) for count in counts]
        self.slots = StateSlotPool(max_num_seqs)
        self.tables = [
            np.zeros((max_num_seqs, self.max_blocks_per_seq), dtype=np.int32) for _ in self.groups
        ]
        # row_versions[slot] changes whenever a table row of that slot changes (in any group), so
        # that a copy of a row made earlier can be recognised as still good
        self.row_versions = [0] * max_num_seqs
        self._version = 0
        self._requests: dict[str, _RequestState] = {}
        self._fresh_slots: list[int] = []
        # prefix reuse needs tables that keep every key (a windowed group has given pages back); with
        # several such groups a prefix counts only as far as every group still holds its pages
        self.prefix_caching = (bool(enable_prefix_caching) and len(self.groups) >= 1
                               and all(group.window is None for group in self.groups))
        self.num_prefix_hits = 0          # pages taken over instead of computed
        # per group, the pages that nobody holds any more since take_released_pages() was last called
        # (kept only on request: the debug fill of freed pages reads it)
        self._released: list[list[int]] | None = [[] for _ in self.groups] if track_released_pages else None

    # ---- queries ---------------------------------------------------------------------------
    def has_request(self, request_id: str) -> bool:
        return request_id in self._requests

    def num_computed(self, request_id: str) -> int:
        state = self._requests.get(request_id)
        return 0 if state is None else state.num_computed

    def state_slot(self, request_id: str) -> int:
        return self._requests[request_id].slot

    def step_place(self, request_id: str, num_new_tokens: int) -> tuple[int, int] | None:
        """(tokens computed so far, state slot) of a request whose next ``num_new_tokens`` tokens
        have their pages; ``None`` if the request is unknown or pages are missing."""
        state = self._requests.get(request_id)
        if state is None:
            return None
        target = -(-(state.num_computed + num_new_tokens) // self.page_size)
        for blocks in state.num_blocks:
            if blocks < target:
                return None
        return state.num_computed, state.slot

    def live_requests(self) -> list[str]:
        return list(self._requests)

    def num_free_pages(self) -> list[int]:
        return [pool.num_free for pool in self.pools]

    def block_ids(self, request_id: str) -> tuple[tuple[int, ...], ...]:
        """Per group, the request's table row up to the blocks it has (0 = handed back)."""
        state = self._requests[request_id]
        return tuple(
            tuple(int(x) for x in self.tables[g][state.slot, : state.num_blocks[g]])
            for g in range(len(self.groups))
        )

    def _new_pages_needed(self, state: _RequestState | None, num_new_tokens: int) -> list[int]:
        computed = 0 if state is None else state.num_computed
        total = computed + num_new_tokens
        target = -(-total // self.page_size)
        return [
            max(target - (0 if state is None else state.num_blocks[g]), 0)
            for g in range(len(self.groups))
        ]

    def pages_needed(self, request_id: str, num_new_tokens: int) -> list[int]:
        return self._new_pages_needed(self._requests.get(request_id), num_new_tokens)

    def can_fit(self, request_id: str, num_new_tokens: int, prefix_pages: Sequence[Sequence[int]] = ()) -> bool:
        """Whether ``num_new_tokens`` more tokens of the request can be given pages (and, for a
        request not yet seen, a state slot) right now.  Admission math as the reference's
        ``can_fit`` (kv_manager.py:179-201) per group instead of per layer: new pages, plus the
        taken-over pages that sit in the free queue now, must not exceed the free pages."""
        state = self._requests.get(request_id)
        computed = len(prefix_pages) * self.page_size if state is None else state.num_computed
        if computed + num_new_tokens > self.max_model_len:
            return False
        if state is None and self.slots.num_free == 0:
            return False
        if prefix_pages:
            if state is not None or not self.prefix_caching:
                return False
            target = -(-(computed + num_new_tokens) // self.page_size)
            for g, pool in enumerate(self.pools):
                queued = sum(1 for pages in prefix_pages if pool.is_queued(pages[g]))
                if target - len(prefix_pages) + queued > pool.num_free:
                    return False
            return True
        needed = self._new_pages_needed(state, num_new_tokens)
        return all(need <= pool.num_free for need, pool in zip(needed, self.pools))

    # ---- prefix reuse ----------------------------------------------------------------------
    def _chain_key(self, previous: bytes, tokens: Sequence[int]) -> bytes:
        return hashlib.sha256(previous + np.asarray(tokens, dtype=np.int64).tobytes()).digest()

    def find_prefix(self, token_ids: Sequence[int]) -> list[tuple[int, ...]]:
        """Pages whose registered contents are the leading full pages of ``token_ids``: one entry per
        page position, holding that position's page id in every group (a position counts only if
        every group still has it); at least the last token is left to compute."""
        if not self.prefix_caching:
            return []
        pages: list[tuple[int, ...]] = []
        key = b""
        for block in range((len(token_ids) - 1) // self.page_size):
            key = self._chain_key(key, token_ids[block * self.page_size : (block + 1) * self.page_size])
            found = tuple(pool.lookup(key) for pool in self.pools)
            if any(page is None for page in found):
                break
            pages.append(found)
        return pages

    def register_full_pages(self, request_id: str, token_ids: Sequence[int]) -> None:
        """Make the request's computed full pages findable (``token_ids``: all its tokens so far)."""
        if not self.prefix_caching:
            return
        state = self._requests.get(request_id)
        if state is None:
            return
        full = min(state.num_computed, len(token_ids)) // self.page_size
        while len(state.page_keys) < full:
            block = len(state.page_keys)
            previous = state.page_keys[-1] if state.page_keys else b""
            key = self._chain_key(previous, token_ids[block * self.page_size : (block + 1) * self.page_size])
            state.page_keys.append(key)
            for g, pool in enumerate(self.pools):
                pool.register(int(self.tables[g][state.slot][block]), key)   # a key already taken stays with its page

    # ---- changes ---------------------------------------------------------------------------
    def allocate_slots(self, request_id: str, num_new_tokens: int,
                       prefix_pages: Sequence[Sequence[int]] = ()) -> bool:
        """Give the request pages for ``num_new_tokens`` tokens beyond those computed.
        ``prefix_pages`` (a new request only, from ``find_prefix``): pages taken over as its
        first ones, in every group; their tokens count as computed.  Returns False (and changes nothing) if
        the pages do not fit."""
        if num_new_tokens <= 0:
            raise ValueError(f"num_new_tokens must be positive, got {num_new_tokens}")
        if not self.can_fit(request_id, num_new_tokens, prefix_pages):
            return False
        state = self._requests.get(request_id)
        if state is None:
            slot = self.slots.allocate(request_id)
            state = _RequestState(
                slot=slot,
                num_blocks=[0] * len(self.groups),
                num_released=[0] * len(self.groups),
            )
            self._requests[request_id] = state
            self._fresh_slots.append(slot)
            for table in self.tables:
                table[slot, :] = NULL_PAGE
            self._touch(slot)
            if prefix_pages:
                count = len(prefix_pages)
                for g, pool in enumerate(self.pools):
                    for pages in prefix_pages:
                        pool.share(pages[g])
                    self.tables[g][slot, :count] = [pages[g] for pages in prefix_pages]
                    state.num_blocks[g] = count
                state.num_computed = count * self.page_size
                self.num_prefix_hits += count
        needed = self._new_pages_needed(state, num_new_tokens)
        for g, need in enumerate(needed):
            if need:
                pages = self.pools[g].allocate(need)
                begin = state.num_blocks[g]
                self.tables[g][state.slot, begin : begin + need] = pages
                state.num_blocks[g] = begin + need
                self._touch(state.slot)
        return True

    def _touch(self, slot: int) -> None:
        self._version += 1
        self.row_versions[slot] = self._version

    def advance(self, request_id: str, num_tokens: int) -> None:
        """Record that ``num_tokens`` more tokens are computed; windowed groups hand back the
        pages that no later query can see (all positions < num_computed - window + 1)."""
        state = self._requests[request_id]
        state.num_computed += num_tokens
        for g, group in enumerate(self.groups):
            capacity = state.num_blocks[g] * self.page_size
            if state.num_computed > capacity:
                raise KVManagerError(
                    f"request {request_id!r} computed {state.num_computed} tokens but group "
                    f"{group.group_id} holds pages for only {capacity}"
                )
            if group.window is None:
                continue
            first_visible = state.num_computed - group.window + 1
            releasable = max(first_visible, 0) // self.page_size
            releasable = min(releasable, state.num_blocks[g])
            if releasable > state.num_released[g]:
                row = self.tables[g][state.slot]
                pages = [int(p) for p in row[state.num_released[g] : releasable] if p != NULL_PAGE]
                self.pools[g].free(pages)
                self._note_released(g, pages)
                row[state.num_released[g] : releasable] = NULL_PAGE
                state.num_released[g] = releasable
                self._touch(state.slot)

    def free(self, request_id: str) -> None:
        """Return everything the request holds: pages in reverse order, and its slot."""
        state = self._requests.pop(request_id, None)
        if state is None:
            return
        for g in range(len(self.groups)):
            row = self.tables[g][state.slot]
            pages = [int(p) for p in row[: state.num_blocks[g]] if p != NULL_PAGE]
            self.pools[g].free(reversed(pages))
            self._note_released(g, pages)
            row[:] = NULL_PAGE
        self._touch(state.slot)
        self.slots.free(state.slot)
        if state.slot in self._fresh_slots:
            self._fresh_slots.remove(state.slot)

    def _note_released(self, group: int, pages: Sequence[int]) -> None:
        if self._released is not None:
            self._released[group].extend(page for page in pages if not self.pools[group].is_held(page))

    def take_released_pages(self) -> list[list[int]]:
        """Per group, the pages that lost their last holder since the last call (empty lists unless the
        manager was built with ``track_released_pages``).  A page may have been handed out again since;
        whoever got it has not written to it yet, because no step has run in between."""
        if self._released is None:
            return [[] for _ in self.groups]
        released, self._released = self._released, [[] for _ in self.groups]
        return released

    def take_fresh_slots(self) -> list[int]:
        """Slots handed to new requests since the last call; their state must start at zero."""
        fresh, self._fresh_slots = self._fresh_slots, []
        return fresh

    # ---- checks ----------------------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, none held twice, tables and pools agree (used by tests)."""
        for g, pool in enumerate(self.pools):
            seen: dict[int, str] = {}
            holders: dict[int, int] = {}
            for request_id, state in self._requests.items():
                row = self.tables[g][state.slot]
                if np.any(row[state.num_blocks[g] :] != NULL_PAGE):
                    raise KVManagerError(f"request {request_id!r} has pages beyond its block count")
                for page in row[: state.num_blocks[g]]:
                    page = int(page)
                    if page == NULL_PAGE:
                        continue
                    if page in seen and not self.prefix_caching:
                        raise KVManagerError(
                            f"page {page} of group {g} is held by {seen[page]!r} and {request_id!r}"
                        )
                    if not pool.is_held(page):
                        raise KVManagerError(f"page {page} of group {g} is in a table but free")
                    seen[page] = request_id
                    holders[page] = holders.get(page, 0) + 1
            for page, count in holders.items():
                if pool.ref_count(page) != count:
                    raise KVManagerError(
                        f"page {page} of group {g} is in {count} table(s) but counts {pool.ref_count(page)} holder(s)"
                    )
            free = pool.free_pages()
            if len(set(free)) != len(free):
                raise KVManagerError(f"group {g}: a page is in the free queue twice")
            if set(free) & set(seen):
                raise KVManagerError(f"group {g}: a page is both free and held")
            if len(free) + len(seen) != pool.num_usable:
                raise KVManagerError(
                    f"group {g}: {pool.num_usable - len(free) - len(seen)} page(s) lost"
                )


def group_entries(requirements) -> tuple[list[CacheGroupSpec], dict[int, int]]:
    """Partition schedule entries into cache groups by equal ``CacheSpec``.

    ``requirements`` are the model's ``EntryRequirement``s.  Returns the groups and a map
    from entry index to group id; an entry that borrows a cache maps to its owner's group.
    """
    by_spec: dict[tuple, list[int]] = {}
    for req in requirements:
        if req.cache_spec is None or req.cache_of is not None:
            continue
        spec = req.cache_spec
        by_spec.setdefault((spec.planes, spec.heads, spec.width, spec.window), []).append(req.entry)
    groups = [
        CacheGroupSpec(group_id, tuple(entries), *key)
        for group_id, (key, entries) in enumerate(by_spec.items())
    ]
    entry_group: dict[int, int] = {}
    for group in groups:
        for entry in group.entries:
            entry_group[entry] = group.group_id
    for req in requirements:
        if req.cache_of is not None and req.cache_spec is not None:
            owner = requirements[req.cache_of]
            if owner.cache_spec != req.cache_spec:
                raise ValueError(
                    f"schedule entry {req.entry} borrows the cache of entry {req.cache_of}, "
                    "whose cache layout differs"
                )
            entry_group[req.entry] = entry_group[req.cache_of]
    return groups, entry_group


__all__ = ["CacheGroupSpec", "KVManager", "KVManagerError", "group_entries"]
