"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.execute`` takes entries that may be whole prompts, portions of prompts cut
anywhere, and single decoded tokens, side by side.  It runs only the tokens it is given, as
one flat batch, reading everything earlier from the cache, writes the new tokens' keys and
values into their pages, and returns the logits at the wanted places.  It changes no host
state: counting computed tokens, hashing pages and freeing belong to the caller (the
scheduler's ``postprocess``, or the replay program), which is what lets a trace drive it
directly.

The reference's counterpart is ``LLMEngine._prepare`` plus the model call
(src/mini_engine/engine.py:200-226, src/mini_engine/attention.py:56-101 of
YuvGev00/mini-engine): there the batch becomes about ten small int64 tensors built token by
token; here it is one int32 block in pinned memory and one host-to-device copy.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence as Seq

import numpy as np
import torch

from mini_engine_b200.cache.manager import NULL_PAGE, RequestCache
from mini_engine_b200.cache.storage import CacheLayout, allocate_cache
from mini_engine_b200.csrc import ops
from mini_engine_b200.engine.batch import StepEntry  # noqa: F401  (re-exported: the step function's input)
from mini_engine_b200.engine.workspace import Workspace
from mini_engine_b200.parts.base import StepContext
from mini_engine_b200.parts.model import DecoderModel


@dataclass
class Prepacked:
    """A decode step laid out in a pinned block ahead of its token ids."""

    flip: int  # which pinned block
    used: int  # int32 values of the block that belong to the step
    ids_offset: int
    real: int  # entries without padding
    total_entries: int
    key: tuple  # (request serial, table version, start) of every entry, as laid out

    def matches(self, entries: Seq[StepEntry]) -> bool:
        """Whether `entries` (one token each) are the step that was laid out: the same requests
        in the same order at the same positions, their block tables unchanged since."""
        return len(entries) == self.real and self.key == tuple(
            (e.cache.serial, e.cache.version, e.start) for e in entries
        ) and all(len(e.token_ids) == 1 for e in entries)


class ModelRunner:
    def __init__(
        self,
        model: DecoderModel,
        *,
        dtype: torch.dtype,
        num_blocks: int,
        block_size: int,
        max_num_seqs: int,
        max_num_batched_tokens: int,
        max_model_len: int,
        device: str = "cuda",
        max_request_tokens: int | None = None,
    ):
        """``max_request_tokens``: the most tokens that ONE request brings to a step (the scheduler's
        budget), where that is less than the step's capacity; it sizes the pools of groups with a window."""
        if not torch.cuda.is_available():
            raise RuntimeError("mini_engine_b200 runs on a CUDA device only; none is available")
        self.model = model
        self.dtype = dtype
        self.device = torch.device(device)
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.max_entries = max_num_seqs
        self.max_tokens = max_num_batched_tokens
        self.table_width = -(-max_model_len // block_size)
        self.vocab_size = model.spec.vocab_size
        self.layout: CacheLayout = allocate_cache(
            model.cache_needs(), num_blocks, block_size, max_num_seqs, dtype, self.device,
            max_step_tokens=max_request_tokens or max_num_batched_tokens,
        )  # fmt: skip
        self.num_groups = len(self.layout.groups)
        self.workspace = Workspace(max_num_batched_tokens, self.device)
        self.spare_pages = self.layout.spare_pages  # per group, owned by no request: padding rows write and read here
        self.spare_slot = max_num_seqs
        # One int32 block holds every index array of a step; two pinned copies alternate so a
        # step never overwrites what an earlier copy may still be reading.
        g, t, b = self.num_groups, self.max_tokens, self.max_entries
        self._capacity = (3 + g) * t + (5 * b + 1) + t + g * b * self.table_width
        self._host = [torch.empty(self._capacity, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._host_np = [h.numpy() for h in self._host]
        self._device = torch.zeros(self._capacity, dtype=torch.int32, device=self.device)
        self._copied = [torch.cuda.Event(), torch.cuda.Event()]  # the copy out of each pinned block
        self._flip = 0
        self.last_h2d_bytes = 0
        # What each pinned block holds in its table region: where the region lies and, row by
        # row, whose tables (request, version) were written there last.
        self._token = object()  # marks the copies of block tables that this runner made (no reference back to it)
        self._row_layout: list[tuple[int, int] | None] = [None, None]
        self._row_owners: list[dict[int, tuple[int, int] | None]] = [{}, {}]

    # ------------------------------------------------------------------ packing

    def _tables_of(self, cache: RequestCache) -> list[np.ndarray]:
        """The request's block tables as int32 rows of the device table's width, ``NULL_PAGE``
        behind their ends; converted again only when the cache manager has changed them."""
        held = cache.packed
        if held is None or held[0] is not self._token or held[1] != cache.version:
            rows = []
            for table in cache.block_tables:
                row = np.full(self.table_width, NULL_PAGE, dtype=np.int32)
                row[: len(table)] = table
                rows.append(row)
            held = (self._token, cache.version, rows, [len(table) for table in cache.block_tables])
            cache.packed = held
        return held

    def pack(
        self,
        entries: Seq[StepEntry],
        pad_entries_to: int | None = None,
        want_every_entry: bool = False,
        build_context: bool = True,
        defer_copy: bool = False,
    ) -> tuple[StepContext | None, torch.Tensor | None] | "Prepacked":
        """Lay the batch out as int32 arrays on the device.  With ``pad_entries_to`` the batch
        is filled up with one-token dummy entries on the spare page (for a captured graph of
        that size); with ``want_every_entry`` the wanted rows are the last token of every entry,
        padding included, whatever the entries ask for.  Returns the context and the int32 row
        numbers of the wanted logits (both ``None`` without ``build_context``: a captured graph
        reads the arrays where they always lie).  With ``defer_copy`` the pinned block is filled
        but not copied: the :class:`Prepacked` that comes back takes the token ids later
        (:meth:`commit`), so that a decode step can be laid out while the one before it runs."""
        real = len(entries)
        total_entries = max(real, pad_entries_to or 0)
        counts = [len(e.token_ids) for e in entries]
        if real == 0 or min(counts) < 1:
            raise ValueError("a step needs at least one entry and every entry at least one token")
        real_tokens = sum(counts)
        tokens = real_tokens + (total_entries - real)
        if tokens > self.max_tokens or total_entries > self.max_entries:
            raise ValueError(
                f"step of {tokens} tokens / {total_entries} entries exceeds the capacity "
                f"({self.max_tokens} tokens, {self.max_entries} entries)"
            )
        g, bs, width = self.num_groups, self.block_size, self.table_width
        self._flip ^= 1
        flip = self._flip
        self._copied[flip].synchronize()  # the host may run ahead of the device by many steps
        host = self._host_np[flip]
        offset = 0

        def take(n: int) -> tuple[np.ndarray, int]:
            nonlocal offset
            view, start = host[offset : offset + n], offset
            offset += n
            return view, start

        ids, o_ids = take(tokens)
        pos, o_pos = take(tokens)
        ent, o_ent = take(tokens)
        slots = [take(tokens) for _ in range(g)]
        cu, o_cu = take(total_entries + 1)
        ctx_len, o_ctx = take(total_entries)
        state, o_state = take(total_entries)
        fresh, o_fresh = take(total_entries)
        tables = [take(total_entries * width) for _ in range(g)]
        table_rows = [t[0].reshape(total_entries, width) for t in tables]
        # A pinned block keeps the table rows it was given: a row is written again only when its
        # request, or that request's tables, differ from what the block holds at that place.
        layout = (tables[0][1] if g else 0, total_entries)
        owners = self._row_owners[flip]
        if self._row_layout[flip] != layout:
            self._row_layout[flip] = layout
            owners.clear()

        def put_row(b: int, cache: RequestCache | None, rows: list[np.ndarray] | None) -> None:
            key = (cache.serial, cache.version) if cache is not None else None
            if owners.get(b, 0) == key:
                return
            owners[b] = key
            for gi in range(g):
                if rows is None:
                    table_rows[gi][b] = self.spare_pages[gi]
                else:
                    table_rows[gi][b] = rows[gi]

        wanted_rows: list[int] = []
        starts = [e.start for e in entries]
        if real_tokens == real:
            # Every entry brings one token: the arrays are filled column-wise.
            start_arr = np.array(starts, dtype=np.int32)
            if int(start_arr.max()) >= width * bs:
                raise ValueError(f"request of {int(start_arr.max()) + 1} tokens exceeds max_model_len {width * bs}")
            ids[:real] = [e.token_ids[0] for e in entries]
            pos[:real] = start_arr
            ent[:real] = np.arange(real, dtype=np.int32)
            page_index = start_arr // bs
            for b, entry in enumerate(entries):
                held = self._tables_of(entry.cache)
                if held[3] and min(held[3]) <= page_index[b]:
                    raise ValueError(f"entry {b}: block table covers {min(held[3]) * bs} tokens, {starts[b] + 1} needed")
                put_row(b, entry.cache, held[2])
                slot = entry.cache.state_slot
                state[b] = slot if slot >= 0 else self.spare_slot
                for place in entry.want:
                    if place != 0:
                        raise ValueError(f"entry {b}: wanted place {place} is outside its 1 tokens")
                    wanted_rows.append(b)
            lanes = np.arange(real)
            for gi in range(g):
                pages = table_rows[gi][lanes, page_index]
                if (pages == NULL_PAGE).any():
                    raise ValueError("a new token falls on a page that was given back")
                slots[gi][0][:real] = pages * bs + start_arr % bs
            cu[: real + 1] = np.arange(real + 1, dtype=np.int32)
            ctx_len[:real] = start_arr + 1
            fresh[:real] = start_arr == 0
            cursor = real
            max_q, max_ctx = 1, int(start_arr.max()) + 1
        else:
            cursor = 0
            cu[0] = 0
            max_q = max_ctx = 1
            for b, entry in enumerate(entries):
                n = counts[b]
                end = entry.start + n
                if end > width * bs:
                    raise ValueError(f"request of {end} tokens exceeds max_model_len {width * bs}")
                ids[cursor : cursor + n] = entry.token_ids
                span = np.arange(entry.start, end, dtype=np.int32)
                pos[cursor : cursor + n] = span
                ent[cursor : cursor + n] = b
                held = self._tables_of(entry.cache)
                put_row(b, entry.cache, held[2])
                for gi in range(g):
                    if held[3][gi] * bs < end:
                        raise ValueError(f"entry {b}: block table covers {held[3][gi] * bs} tokens, {end} needed")
                    pages = held[2][gi][span // bs]
                    if (pages == NULL_PAGE).any():
                        raise ValueError(f"entry {b}: a new token falls on a page that was given back")
                    slots[gi][0][cursor : cursor + n] = pages * bs + span % bs
                cu[b + 1] = cursor + n
                ctx_len[b] = end
                state[b] = entry.cache.state_slot if entry.cache.state_slot >= 0 else self.spare_slot
                fresh[b] = 1 if entry.start == 0 else 0
                for place in entry.want:
                    if not 0 <= place < n:
                        raise ValueError(f"entry {b}: wanted place {place} is outside its {n} tokens")
                    wanted_rows.append(cursor + place)
                max_q, max_ctx = max(max_q, n), max(max_ctx, end)
                cursor += n
        if ids[:real_tokens].min() < 0 or ids[:real_tokens].max() >= self.vocab_size:
            raise ValueError(f"token ids must lie in [0, {self.vocab_size})")
        for b in range(real, total_entries):  # padding: one token at position 0 of the spare page
            ids[cursor], pos[cursor], ent[cursor] = 0, 0, b
            for gi in range(g):
                slots[gi][0][cursor] = self.spare_pages[gi] * bs
            put_row(b, None, None)
            cu[b + 1] = cursor + 1
            ctx_len[b], state[b], fresh[b] = 1, self.spare_slot, 1
            cursor += 1
        # Entries that bring one token and entries that bring more, for kernels that treat them
        # differently within one step.
        all_counts = counts + [1] * (total_entries - real)
        decode_list = [b for b, n in enumerate(all_counts) if n == 1]
        portion_list = [b for b, n in enumerate(all_counts) if n > 1]
        kinds_view, o_kinds = take(total_entries)
        kinds_view[: len(decode_list)] = decode_list
        kinds_view[len(decode_list) :] = portion_list
        if want_every_entry:
            wanted_rows = [int(cu[b + 1]) - 1 for b in range(total_entries)]
        rows_view, o_rows = take(len(wanted_rows))
        rows_view[:] = wanted_rows

        used = offset
        if defer_copy:
            key = tuple((e.cache.serial, e.cache.version, e.start) for e in entries)
            return Prepacked(flip, used, o_ids, real, total_entries, key)
        self._device[:used].copy_(self._host[flip][:used], non_blocking=True)
        self._copied[flip].record()
        self.last_h2d_bytes = used * 4
        if not build_context:
            return None, None
        dev = self._device

        def at(start: int, n: int) -> torch.Tensor:
            return dev[start : start + n]

        ctx = StepContext(
            dtype=self.dtype,
            num_tokens=tokens,
            num_entries=total_entries,
            max_query_len=max_q,
            max_context_len=max_ctx,
            token_ids=at(o_ids, tokens),
            positions=at(o_pos, tokens),
            entry_of_token=at(o_ent, tokens),
            cu_tokens=at(o_cu, total_entries + 1),
            context_lens=at(o_ctx, total_entries),
            state_slots=at(o_state, total_entries),
            fresh=at(o_fresh, total_entries),
            slot_mapping=[at(s[1], tokens) for s in slots],
            block_tables=[at(t[1], total_entries * width).view(total_entries, width) for t in tables],
            page_size=bs,
            workspace=self.workspace,
            all_decode=max_q == 1,
            num_decode_entries=len(decode_list),
            decode_entries=at(o_kinds, len(decode_list)),
            portion_entries=at(o_kinds + len(decode_list), len(portion_list)),
            host={
                "counts": all_counts,
                "starts": starts + [0] * (total_entries - real),
                "state_slots": [int(x) for x in state[:total_entries]],
            },
        )
        return ctx, at(o_rows, len(wanted_rows))

    def commit(self, prepacked: "Prepacked", token_ids: Seq[int] | torch.Tensor, rows: torch.Tensor | None = None) -> None:
        """Put the token ids into a block that :meth:`pack` laid out with ``defer_copy`` and copy
        it to the device.  Token ids that are still on the device (an int32 tensor: what the
        sampler drew in the step before) are copied there into the device's block, after the
        block itself, so the host need not know them yet; entry i takes ``token_ids[rows[i]]``
        when ``rows`` (int32, on the device) is given, else ``token_ids[i]``."""
        used = prepacked.used
        ids = slice(prepacked.ids_offset, prepacked.ids_offset + prepacked.real)
        on_device = isinstance(token_ids, torch.Tensor)
        if (len(token_ids) if rows is None else len(rows)) != prepacked.real:
            raise ValueError("one token id per entry of the prepacked step")
        if on_device:
            if token_ids.dtype != torch.int32 or not token_ids.is_cuda:
                raise ValueError("token ids on the device must be int32")
        else:
            if rows is not None:
                raise ValueError("rows pick among token ids on the device")
            if min(token_ids) < 0 or max(token_ids) >= self.vocab_size:
                raise ValueError(f"token ids must lie in [0, {self.vocab_size})")
            self._host_np[prepacked.flip][ids] = token_ids
        self._device[:used].copy_(self._host[prepacked.flip][:used], non_blocking=True)
        self._copied[prepacked.flip].record()
        if on_device and rows is not None:
            ops.pick_tokens(token_ids, rows, self._device[ids])
        elif on_device:
            self._device[ids].copy_(token_ids, non_blocking=True)
        self.last_h2d_bytes = used * 4

    # --------------------------------------------------------------------- step

    @torch.inference_mode()
    def execute(self, entries: Seq[StepEntry]) -> torch.Tensor:
        """Float32 logits ``[wanted, vocab]`` on the device, in the order of the entries and
        of each entry's ``want``.  The tensor is a view of a buffer that the next step
        overwrites."""
        ctx, rows = self.pack(entries)
        return self.model.forward(ctx, self.layout.views, rows)
