"""CUDA graphs for decode-only steps: the whole forward pass of a batch of single tokens is
captured once per batch-size bucket and replayed with one launch; and for steps that hold one
short prompt or portion (:class:`PromptGraphs`).

As in the reference (src/mini_engine/cuda_graphs.py:28-138 of YuvGev00/mini-engine): buckets
1, 2, 4, 8, then multiples of 16 up to the request cap; a batch is padded up to its bucket
with dummy rows that write to and read from a spare cache page that no request owns; every
buffer that a graph reads lives as long as the graph (here: the runner's index block and
workspace, whose addresses never change).
"""

from __future__ import annotations

from typing import Sequence as Seq

import torch

from mini_engine_b200.cache.manager import RequestCache
from mini_engine_b200.csrc import ops
from mini_engine_b200.engine.runner import ModelRunner, StepEntry


def batch_buckets(max_batch: int) -> list[int]:
    """Batch sizes that get a graph of their own: 1, 2, 4, 8, the multiples of 16, and the cap
    itself, so that no batch is padded by more than its own size or 15 rows."""
    sizes = {max_batch}
    size = 1
    while size < max_batch:
        sizes.add(size)
        size = size * 2 if size < 16 else size + 16
    return sorted(sizes)


class DecodeGraphs:
    def __init__(self, runner: ModelRunner, max_batch: int):
        self.runner = runner
        self.buckets = batch_buckets(max_batch)
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.logits: dict[int, torch.Tensor] = {}
        self.launches: dict[int, int] = {}  # kernels inside each bucket's graph
        self._capture_all()

    @property
    def max_batch(self) -> int:
        return self.buckets[-1]

    def _dummy_entries(self, count: int) -> list[StepEntry]:
        caches = [
            RequestCache(block_tables=[[page] for page in self.runner.spare_pages])
            for _ in range(count)
        ]
        return [StepEntry(c, 0, [0], (0,)) for c in caches]

    @torch.inference_mode()
    def _capture_all(self) -> None:
        runner = self.runner
        pool = None
        for bucket in reversed(self.buckets):  # largest first: smaller graphs reuse its memory pool
            entries = self._dummy_entries(bucket)
            ctx, rows = runner.pack(entries)
            # A captured launch must cover any context that a later replay may bring.
            ctx.max_context_len = runner.table_width * runner.block_size
            runner.model.forward(ctx, runner.layout.views, rows)  # warm-up: builds, descriptors, buffers
            torch.cuda.synchronize()
            ctx.memo.clear()  # what the warm-up computed once per step must be computed inside the graph too
            graph = torch.cuda.CUDAGraph()
            runner.workspace.frozen = True
            before = ops.launch_count()
            try:
                with torch.cuda.graph(graph, pool=pool):
                    self.logits[bucket] = runner.model.forward(ctx, runner.layout.views, rows)
            finally:
                runner.workspace.frozen = False
            self.launches[bucket] = ops.launch_count() - before
            pool = graph.pool()
            self.graphs[bucket] = graph
        torch.cuda.synchronize()

    def bucket_for(self, batch: int) -> int | None:
        for bucket in self.buckets:
            if bucket >= batch:
                return bucket
        return None

    def prepare(self, entries: Seq[StepEntry]):
        """Lay a decode step out ahead of its token ids (placeholders in `entries`)."""
        bucket = self.bucket_for(len(entries))
        return self.runner.pack(entries, pad_entries_to=bucket, want_every_entry=True, build_context=False, defer_copy=True)

    def run_prepared(self, prepacked, token_ids: Seq[int] | torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        """The step that :meth:`prepare` laid out, now that its token ids are known: to the host,
        or only to the device (an int32 tensor that the sampler wrote, of which ``rows`` picks the
        entries' tokens if given)."""
        self.runner.commit(prepacked, token_ids, rows)
        self.graphs[prepacked.total_entries].replay()
        return self.logits[prepacked.total_entries][: prepacked.real]

    def run(self, entries: Seq[StepEntry]) -> torch.Tensor:
        """Logits ``[len(entries), vocab]``: one decoded token per entry, the logits of each."""
        real = len(entries)
        bucket = self.bucket_for(real)
        self.runner.pack(entries, pad_entries_to=bucket, want_every_entry=True, build_context=False)
        self.graphs[bucket].replay()
        return self.logits[bucket][:real]


# Token counts that get a graph (each holds the request's tokens and a dummy entry of at least one).
# Up to 127 tokens the padded step's kernels take less time than the eager step's launches take
# the host (Qwen3-8B sizes: 32 tokens 4.1 -> 3.8 ms); from 128 tokens on the step is bound by its
# kernels and the padding only costs (128 tokens in the graph of 160: 5.0 ms against 4.6 eagerly).
PROMPT_BUCKETS = (32, 64, 96, 128)


class PromptGraphs:
    """Captured steps for ONE short prompt (or portion of one) alone in its step.

    An eager step costs the host about 15 us a launch, 330 launches for 36 layers: a prompt of a
    few dozen tokens then takes longer on the host than on the device.  A graph of a fixed shape replaces
    those launches: two entries that together bring exactly ``bucket`` tokens, the request's ``n``
    tokens (2 <= n < bucket) and a dummy entry of ``bucket - n`` tokens that lives on the spare page
    of every cache group.  What varies from replay to replay (token ids, positions, slots, block
    tables, lengths, the wanted row) lies in the runner's index arrays on the device; what a launch
    fixes on the host (grids) is set for the worst case: the longest entry the bucket can hold and
    the longest context the engine allows.  Both entries run through the kernels for portions
    whatever their lengths.  Graphs are captured when a bucket is first needed.  The reference
    captures decode steps only (src/mini_engine/cuda_graphs.py of YuvGev00/mini-engine)."""

    def __init__(self, runner: ModelRunner):
        self.runner = runner
        self.buckets = [b for b in PROMPT_BUCKETS if b <= runner.max_tokens]
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.logits: dict[int, torch.Tensor] = {}
        self.launches: dict[int, int] = {}
        self._pool = None
        width = runner.table_width
        self._dummy = RequestCache(block_tables=[[page] * width for page in runner.spare_pages])

    def bucket_for(self, tokens: int) -> int | None:
        """The smallest bucket that holds ``tokens`` and a dummy entry of at least one token."""
        if tokens < 2 or self.runner.max_entries < 2:
            return None
        for bucket in self.buckets:
            if tokens < bucket:
                return bucket
        return None

    def _entries(self, entry: StepEntry, bucket: int) -> list[StepEntry]:
        count = len(entry.token_ids)
        real = StepEntry(entry.cache, entry.start, entry.token_ids, (count - 1,))  # the last row is always computed
        return [real, StepEntry(self._dummy, 0, [0] * (bucket - count), ())]

    @torch.inference_mode()
    def _capture(self, bucket: int) -> None:
        runner = self.runner
        shape = [StepEntry(self._dummy, 0, [0] * (bucket - 2), (bucket - 3,)), StepEntry(self._dummy, 0, [0, 0], ())]
        ctx, rows = runner.pack(shape)
        # grids for whatever a replay may bring: one entry of up to bucket - 1 tokens, any context
        ctx.max_query_len = bucket
        ctx.max_context_len = runner.table_width * runner.block_size
        ctx.all_decode, ctx.num_decode_entries = False, 0
        runner.model.forward(ctx, runner.layout.views, rows)  # warm-up: builds, descriptors, buffers
        torch.cuda.synchronize()
        ctx.memo.clear()
        graph = torch.cuda.CUDAGraph()
        runner.workspace.frozen = True
        before = ops.launch_count()
        try:
            with torch.cuda.graph(graph, pool=self._pool):
                self.logits[bucket] = runner.model.forward(ctx, runner.layout.views, rows)
        finally:
            runner.workspace.frozen = False
        self.launches[bucket] = ops.launch_count() - before
        self._pool = graph.pool()
        self.graphs[bucket] = graph
        torch.cuda.synchronize()

    def run(self, entry: StepEntry) -> torch.Tensor | None:
        """Logits ``[1, vocab]`` at the entry's last token, or ``None`` when no bucket takes it."""
        bucket = self.bucket_for(len(entry.token_ids))
        if bucket is None:
            return None
        if bucket not in self.graphs:
            self._capture(bucket)
        self.runner.pack(self._entries(entry, bucket), build_context=False)
        self.graphs[bucket].replay()
        return self.logits[bucket][:1]
