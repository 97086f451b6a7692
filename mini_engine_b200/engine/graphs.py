"""CUDA graphs for decode-only steps: the whole forward pass of a batch of single tokens is
captured once per batch-size bucket and replayed with one launch.

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
