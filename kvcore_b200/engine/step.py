"""The step function: one batch of (request, its next tokens) run through the model from
the cache, returning 32-bit logits at the wanted places.

A step may mix portions of prompts with single decoded tokens, cut anywhere.  It runs only
the tokens it is given; everything earlier is read from the pages that earlier steps wrote.
The reference spreads this over its model runner (kvcore/model/model_runner.py:208-306,
411-580: flatten inputs, build metadata with per-layer block tables and slot mappings,
forward, gather logits rows).  Here the whole step's metadata is packed into one pinned
host buffer and uploaded with a single copy: per request its query start, cached length,
total length and state slot; per token its id, position and request row; the wanted rows;
and one block-table slice per cache group.  Kernels compute cache slots from the block
table and the position themselves, so no slot mapping is built.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from .. import kernels as K
from ..cache.kv_manager import CacheGroupSpec, KVManager
from ..parts.model import DecoderModel


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens, and which of them need logits.

    ``fed_from``: the entry's single token is not known to the host yet; it is row ``fed_from``
    of the sampler output handed to ``StepFunction.step`` as ``feedback`` (``token_ids`` then
    holds one placeholder)."""

    request_id: str
    token_ids: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)
    fed_from: int | None = None


@dataclass
class LayerCache:
    """What one schedule entry's mixer sees of the cache: the planes its ``CacheSpec`` declared, each
    ``[pages, heads, page_size, width]`` (none without a spec), and its state tensor
    ``[slots, *shape]`` if it declared a ``StateSpec``."""

    group: int | None
    planes: tuple[torch.Tensor, ...]
    owner: bool
    state: torch.Tensor | None
    page_size: int

    @property
    def k(self) -> torch.Tensor | None:
        """The first plane (the keys of a key/value cache)."""
        return self.planes[0] if self.planes else None

    @property
    def v(self) -> torch.Tensor | None:
        """The second plane (the values of a key/value cache)."""
        return self.planes[1] if len(self.planes) > 1 else None


class StepContext:
    """Device-side description of the step's batch, handed to every part."""

    def __init__(self) -> None:
        self.num_tokens = 0
        self.num_reqs = 0
        self.num_logits = 0
        self.page_size = 0
        self.token_ids: torch.Tensor | None = None
        self.positions: torch.Tensor | None = None
        self.req_index: torch.Tensor | None = None
        self.query_start: torch.Tensor | None = None
        self.context_lens: torch.Tensor | None = None
        self.seq_lens: torch.Tensor | None = None
        self.state_slots: torch.Tensor | None = None
        self.logits_indices: torch.Tensor | None = None
        self.tables: list[torch.Tensor] = []
        self.table_width = 0
        self.max_query_len = 0
        self.max_seq_len = 0
        self.max_seq_len_bound = 0  # table_width * page_size: a bound that is stable across steps
        self.decode_only = False
        # host copies, for parts that plan their launches (or toy parts written in torch)
        self.host_query_lens: list[int] = []
        self.host_context_lens: list[int] = []
        self.host_state_slots: list[int] = []
        self._shared: dict = {}

    def shared(self, key, make):
        """A value computed once per step and shared by the layers that ask for it under
        ``key`` (for example the cos/sin table of one rotary frequency table)."""
        if key not in self._shared:
            self._shared[key] = make()
        return self._shared[key]

    def block_table(self, group: int | None) -> torch.Tensor | None:
        """``[num_reqs, table_width]`` int32 page ids of the step's requests for ``group``."""
        return None if group is None else self.tables[group]


class CacheStorage:
    """Device tensors behind the cache manager's bookkeeping.

    Per group one tensor ``[entries, planes, pages, heads, page_size, width]`` as the group's
    ``CacheSpec`` has it (keys at plane 0, values at plane 1 for attention): every entry of the
    group stores a page id's tokens in its own slice.  Per schedule entry with a ``StateSpec``
    one tensor ``[slots, *shape]``.
    """

    def __init__(
        self,
        model: DecoderModel,
        groups: list[CacheGroupSpec],
        entry_group: dict[int, int],
        *,
        num_pages: list[int],
        page_size: int,
        num_slots: int,
        dtype: torch.dtype,
        device: torch.device,
    ) -> None:
        self.page_size = page_size
        self.group_tensors: list[torch.Tensor] = []
        for group, pages in zip(groups, num_pages):
            self.group_tensors.append(
                torch.zeros(
                    len(group.entries), group.planes, pages, group.heads, page_size, group.width,
                    dtype=dtype, device=device,
                )
            )
        self.layer_caches: list[LayerCache] = []
        self.state_tensors: list[torch.Tensor] = []
        for req in model.entry_requirements():
            planes: tuple[torch.Tensor, ...] = ()
            group_id = entry_group.get(req.entry)
            owner = req.cache_of is None
            if group_id is not None:
                owner_entry = req.entry if owner else req.cache_of
                index = groups[group_id].entries.index(owner_entry)
                planes = tuple(self.group_tensors[group_id][index].unbind(0))
            state = None
            if req.state_spec is not None:
                state = torch.zeros(
                    (num_slots, *req.state_spec.shape), dtype=req.state_spec.dtype, device=device
                )
                self.state_tensors.append(state)
            self.layer_caches.append(LayerCache(group_id, planes, owner, state, page_size))

    # what "poison" writes into freed pages: large enough that a read of a position nobody wrote
    # changes the logits by orders of magnitude, finite so that a masked probability of exactly
    # zero still cancels it
    POISON_VALUE = 3.0e4

    def fill_pages(self, group: int, pages: Sequence[int], value: float) -> None:
        """Overwrite ``pages`` of ``group`` in every entry and plane (the debug fill of freed pages)."""
        if not pages:
            return
        tensor = self.group_tensors[group]
        index = torch.as_tensor(sorted(set(int(p) for p in pages)), dtype=torch.long, device=tensor.device)
        tensor.index_fill_(2, index, value)

    def zero_slots(self, slots: Sequence[int]) -> None:
        if not slots or not self.state_tensors:
            return
        index = torch.as_tensor(list(slots), dtype=torch.long, device=self.state_tensors[0].device)
        for state in self.state_tensors:
            state.index_fill_(0, index, 0)

    def bytes_per_page(self) -> list[int]:
        return [
            t.shape[0] * t.shape[1] * t.shape[3] * t.shape[4] * t.shape[5] * t.element_size()
            for t in self.group_tensors
        ]


def _round4(n: int) -> int:
    return (n + 3) & ~3


class StepFunction:
    def __init__(
        self,
        model: DecoderModel,
        kv_manager: KVManager,
        storage: CacheStorage,
        *,
        max_num_tokens: int,
        max_num_seqs: int,
        use_cuda_graphs: bool = True,
        max_graphs: int = 24,
        fill_freed_pages: str | None = None,
    ) -> None:
        self.model = model
        self.kv = kv_manager
        self.storage = storage
        self.device = model.device
        self.max_num_tokens = int(max_num_tokens)
        self.max_num_seqs = int(max_num_seqs)
        self.vocab_size = model.spec.vocab_size
        if fill_freed_pages not in (None, "zero", "poison"):
            raise ValueError(f"fill_freed_pages must be None, 'zero' or 'poison', got {fill_freed_pages!r}")
        self.fill_freed_pages = fill_freed_pages
        width = kv_manager.max_blocks_per_seq
        capacity = (
            4 * _round4(self.max_num_seqs + 1)
            + 5 * _round4(self.max_num_tokens)
            + len(kv_manager.groups) * _round4(self.max_num_seqs * width)
        )
        self._capacity = capacity
        self._device_meta = torch.zeros(capacity, dtype=torch.int32, device=self.device)
        pin = self.device.type == "cuda"
        self._host_meta = [torch.zeros(capacity, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._host_arrays = [buffer.numpy() for buffer in self._host_meta]
        self._host_events: list[torch.cuda.Event | None] = [None, None]
        self._table_rows: list[list] = [[None, []], [None, []]]   # per buffer: layout stamp, (slot, version) per row
        self._turn = 0
        self._row_numbers = np.arange(self.max_num_seqs + 1, dtype=np.int32)
        self._views: dict[tuple[int, int, int, int], tuple] = {}
        self.last_context: StepContext | None = None
        self.num_steps = 0
        # decode-only steps of one shape (requests, wanted rows, table width) replay a CUDA graph
        self.use_cuda_graphs = bool(use_cuda_graphs) and self.device.type == "cuda" and model.graph_safe
        self.max_graphs = int(max_graphs)
        self._graphs: dict[tuple[int, int, int], object] = {}
        self._graph_seen: set[tuple[int, int, int]] = set()
        self.num_graph_replays = 0

    # ---- packing -----------------------------------------------------------------------------
    def _pack(self, entries: Sequence[StepEntry], feedback: torch.Tensor | None = None) -> StepContext:
        kv = self.kv
        num_reqs = len(entries)
        if num_reqs == 0:
            raise ValueError("a step needs at least one entry")
        if num_reqs > self.max_num_seqs:
            raise ValueError(f"{num_reqs} requests in one step exceed max_num_seqs {self.max_num_seqs}")
        # Inside the step the requests stand longest portion first (a stable order: a decode-only step
        # keeps the caller's), so that a mixer can hand the portions of prompts and the single decoded
        # tokens to different kernels as two contiguous runs of requests.  The wanted rows keep the
        # caller's order of entries: ``caller_order[i]`` is where the caller's entry i stands.
        if any(len(entry.token_ids) != len(entries[0].token_ids) for entry in entries):
            by_length = sorted(range(num_reqs), key=lambda i: -len(entries[i].token_ids))
            caller_order = [0] * num_reqs
            for place, index in enumerate(by_length):
                caller_order[index] = place
            entries = [entries[index] for index in by_length]
        else:
            caller_order = None
        query_lens = [len(entry.token_ids) for entry in entries]
        num_tokens = sum(query_lens)
        if num_tokens > self.max_num_tokens:
            raise ValueError(
                f"{num_tokens} tokens in one step exceed max_num_scheduled_tokens {self.max_num_tokens}"
            )
        seen: set[str] = set()
        context_lens: list[int] = []
        slots: list[int] = []
        for entry, n in zip(entries, query_lens):
            if n == 0:
                raise ValueError(f"request {entry.request_id!r} brings no tokens to the step")
            if entry.request_id in seen:
                raise ValueError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            place = kv.step_place(entry.request_id, n)
            if place is None:
                raise RuntimeError(
                    f"request {entry.request_id!r} has no pages for its next {n} tokens: "
                    "allocate_slots must succeed before the step"
                )
            context_lens.append(place[0])
            slots.append(place[1])
        seq_lens = [c + n for c, n in zip(context_lens, query_lens)]
        max_seq_len = max(seq_lens)
        width = -(-max_seq_len // kv.page_size)
        # decode-only steps round the table width up coarsely so that one captured graph serves
        # many consecutive steps (the width is part of the graph's shape)
        grain = 16 if max(query_lens) == 1 else 4
        width = max(1, min(-(-width // grain) * grain, kv.max_blocks_per_seq))
        num_logits = sum(len(entry.want) for entry in entries)

        # layout (int32 counts, each array starting on a 16-byte boundary)
        r4, t4 = _round4(num_reqs + 1), _round4(num_tokens)
        off_query_start = 0
        off_context = r4
        off_seq = 2 * r4
        off_slots = 3 * r4
        off_tokens = 4 * r4
        off_positions = off_tokens + t4
        off_req_index = off_positions + t4
        off_logits = off_req_index + t4
        off_feed = off_logits + _round4(max(num_logits, 1))
        off_tables = off_feed + t4
        table_len = _round4(num_reqs * width)
        used = off_tables + len(kv.groups) * table_len
        if used > self._capacity:
            raise RuntimeError("step metadata exceeds its buffer")  # cannot happen by construction

        turn = self._turn
        self._turn ^= 1
        event = self._host_events[turn]
        if event is not None:
            event.synchronize()
        host = self._host_arrays[turn]

        if num_tokens == num_reqs:
            host[off_query_start : off_query_start + num_reqs + 1] = self._row_numbers[: num_reqs + 1]
        else:
            starts = np.zeros(num_reqs + 1, dtype=np.int32)
            np.cumsum(query_lens, out=starts[1:])
            host[off_query_start : off_query_start + num_reqs + 1] = starts
        host[off_context : off_context + num_reqs] = context_lens
        host[off_seq : off_seq + num_reqs] = seq_lens
        host[off_slots : off_slots + num_reqs] = slots
        cursor = 0
        logit_rows: list[int] = []
        if num_tokens == num_reqs:
            # one token a request (a decode step): the per-token arrays are the per-request ones
            ids = np.fromiter((entry.token_ids[0] for entry in entries), dtype=np.int64, count=num_reqs)
            if ids.min() < 0 or ids.max() >= self.vocab_size:
                bad = entries[int(np.argmax((ids < 0) | (ids >= self.vocab_size)))]
                raise ValueError(f"request {bad.request_id!r} has a token id outside [0, {self.vocab_size})")
            host[off_tokens : off_tokens + num_reqs] = ids
            host[off_positions : off_positions + num_reqs] = context_lens
            host[off_req_index : off_req_index + num_reqs] = self._row_numbers[:num_reqs]
            for row, entry in enumerate(entries):
                for place in entry.want:
                    if place != 0:
                        raise ValueError(
                            f"request {entry.request_id!r} wants logits at place {place} of 1 tokens"
                        )
                    logit_rows.append(row)
        else:
            rows_of: list[list[int]] = []
            for row, (entry, n, context) in enumerate(zip(entries, query_lens, context_lens)):
                ids = np.asarray(entry.token_ids, dtype=np.int64)
                if ids.min() < 0 or ids.max() >= self.vocab_size:
                    raise ValueError(
                        f"request {entry.request_id!r} has a token id outside [0, {self.vocab_size})"
                    )
                host[off_tokens + cursor : off_tokens + cursor + n] = ids
                host[off_positions + cursor : off_positions + cursor + n] = np.arange(
                    context, context + n, dtype=np.int32
                )
                host[off_req_index + cursor : off_req_index + cursor + n] = row
                wanted = []
                for place in entry.want:
                    if not 0 <= place < n:
                        raise ValueError(
                            f"request {entry.request_id!r} wants logits at place {place} of {n} tokens"
                        )
                    wanted.append(cursor + int(place))
                rows_of.append(wanted)
                cursor += n
            # the logits come back in the caller's order of entries
            for place in (caller_order if caller_order is not None else range(num_reqs)):
                logit_rows.extend(rows_of[place])
        if logit_rows:
            host[off_logits : off_logits + num_logits] = logit_rows
        fed = any(entry.fed_from is not None for entry in entries)
        if fed:
            if feedback is None:
                raise ValueError("an entry takes its token from the step in front, but no sampler output was given")
            cursor = 0
            for entry, n in zip(entries, query_lens):
                if entry.fed_from is None:
                    host[off_feed + cursor : off_feed + cursor + n] = -1
                elif n != 1 or not 0 <= entry.fed_from < feedback.numel():
                    raise ValueError(f"request {entry.request_id!r}: a fed entry is one token from a row of the "
                                     f"sampler output, got {n} tokens from row {entry.fed_from}")
                else:
                    host[off_feed + cursor] = entry.fed_from
                cursor += n
        # block tables: a row of this buffer that still holds the same slot at the same version (the
        # buffer was last written two steps ago) is left as it is; a steady decode batch rewrites a
        # row only when its request got a page
        stamp = (off_tables, width, num_reqs)
        written = self._table_rows[turn]
        if written[0] != stamp:
            written[0] = stamp
            written[1] = [None] * num_reqs
        rows = written[1]
        versions = kv.row_versions
        for row, slot in enumerate(slots):
            mark = (slot, versions[slot])
            if rows[row] != mark:
                rows[row] = mark
                for g in range(len(kv.groups)):
                    begin = off_tables + g * table_len + row * width
                    host[begin : begin + width] = kv.tables[g][slot, :width]

        device_meta = self._device_meta
        device_meta[:used].copy_(self._host_meta[turn][:used], non_blocking=True)
        if self.device.type == "cuda":
            if event is None:
                event = self._host_events[turn] = torch.cuda.Event()
            event.record()
        if fed:  # the real ids replace the placeholders on the device, in stream order
            K.feed_tokens(device_meta[off_tokens : off_tokens + num_tokens],
                          device_meta[off_feed : off_feed + num_tokens], feedback)

        ctx = StepContext()
        ctx.num_tokens, ctx.num_reqs, ctx.num_logits = num_tokens, num_reqs, num_logits
        ctx.page_size = kv.page_size
        # the views into the metadata buffer depend on the layout only: steps of one shape (every
        # decode step of a steady batch) share them
        layout = (num_reqs, num_tokens, num_logits, width)
        views = self._views.get(layout)
        if views is None:
            if len(self._views) >= 256:
                self._views.clear()
            views = self._views[layout] = (
                device_meta[off_query_start : off_query_start + num_reqs + 1],
                device_meta[off_context : off_context + num_reqs],
                device_meta[off_seq : off_seq + num_reqs],
                device_meta[off_slots : off_slots + num_reqs],
                device_meta[off_tokens : off_tokens + num_tokens],
                device_meta[off_positions : off_positions + num_tokens],
                device_meta[off_req_index : off_req_index + num_tokens],
                device_meta[off_logits : off_logits + num_logits],
                [
                    device_meta[off_tables + g * table_len : off_tables + g * table_len + num_reqs * width].view(
                        num_reqs, width
                    )
                    for g in range(len(kv.groups))
                ],
            )
        (ctx.query_start, ctx.context_lens, ctx.seq_lens, ctx.state_slots, ctx.token_ids, ctx.positions,
         ctx.req_index, ctx.logits_indices, ctx.tables) = views
        ctx.table_width = width
        ctx.max_query_len = max(query_lens)
        ctx.max_seq_len = max_seq_len
        ctx.max_seq_len_bound = width * kv.page_size
        ctx.decode_only = ctx.max_query_len == 1
        ctx.host_query_lens = query_lens
        ctx.host_context_lens = context_lens
        ctx.host_state_slots = slots
        return ctx

    # ---- the step ------------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], feedback: torch.Tensor | None = None) -> torch.Tensor | None:
        """Run one batch; returns ``[wanted, vocab]`` 32-bit logits on the device (``None`` if
        nothing is wanted), rows in the order of the entries and of each entry's ``want``.
        ``feedback``: int32 tokens sampled from the step in front, for entries with ``fed_from``."""
        ctx = self._pack(entries, feedback)
        self.storage.zero_slots(self.kv.take_fresh_slots())
        if self.fill_freed_pages is not None:
            value = 0.0 if self.fill_freed_pages == "zero" else self.storage.POISON_VALUE
            for group, pages in enumerate(self.kv.take_released_pages()):
                self.storage.fill_pages(group, pages, value)
        if self.use_cuda_graphs and ctx.decode_only:
            logits = self._step_with_graph(ctx)
        else:
            logits = self._forward(ctx)
        for entry in entries:
            self.kv.advance(entry.request_id, len(entry.token_ids))
        self.last_context = ctx
        self.num_steps += 1
        return logits


    def _forward(self, ctx: StepContext) -> torch.Tensor | None:
        h, residual = self.model.forward(ctx, self.storage.layer_caches)
        if not ctx.num_logits:
            return None
        return self.model.compute_logits(h, residual, ctx.logits_indices)

    def _step_with_graph(self, ctx: StepContext) -> torch.Tensor | None:
        """Decode-only step through a CUDA graph.

        Every value a kernel takes from the host is fixed by the key (requests, wanted rows,
        table width); everything else (token ids, positions, lengths, block tables) sits at
        fixed addresses of the metadata buffer, which was just uploaded.  A shape is run
        eagerly the first time, captured the second time and replayed from then on.  The
        returned logits live in the graph's memory and are overwritten by its next replay.
        """
        key = (ctx.num_reqs, ctx.num_logits, ctx.table_width)
        graph = self._graphs.get(key)
        if graph is None:
            if key not in self._graph_seen:
                self._graph_seen.add(key)
                return self._forward(ctx)
            if len(self._graphs) >= self.max_graphs:
                self._graphs.pop(next(iter(self._graphs)))
            cuda_graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize(self.device)
            launches_before = K.api.launch_count
            with torch.cuda.graph(cuda_graph):
                static_logits = self._forward(ctx)
            graph = (cuda_graph, static_logits, K.api.launch_count - launches_before)
            K.api.launch_count = launches_before  # capturing launches nothing; replays are counted
            self._graphs[key] = graph
        cuda_graph, static_logits, launches = graph
        cuda_graph.replay()
        K.api.launch_count += launches
        self.num_graph_replays += 1
        return static_logits


__all__ = ["CacheStorage", "LayerCache", "StepContext", "StepEntry", "StepFunction"]
