"""The engine loop: schedule -> pack -> forward -> sample -> postprocess.

Names and meanings follow ``LLMEngine`` of YuvGev00/mini-engine
(src/mini_engine/engine.py:59-299): ``from_pretrained``, ``add_request``, ``generate``,
``step``, ``stats``, ``scheduler``, ``block_manager``.  Token ids go in and come out;
tokenisation is the caller's business.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Iterable

import torch

from mini_engine_b200.cache.manager import CacheManager
from mini_engine_b200.cache.storage import blocks_for_budget
from mini_engine_b200.config.engine_config import EngineConfig
from mini_engine_b200.csrc import ops
from mini_engine_b200.engine.graphs import PROMPT_BUCKETS, DecodeGraphs, PromptGraphs
from mini_engine_b200.engine.loading import load_model, random_model
from mini_engine_b200.engine.runner import ModelRunner, Prepacked
from mini_engine_b200.engine.scheduler import ScheduledSeq, Scheduler, SchedulerConfig
from mini_engine_b200.engine.sequence import Sequence
from mini_engine_b200.parts.model import DecoderModel
from mini_engine_b200.sampling.params import SamplingParams
from mini_engine_b200.sampling.sampler import Draw, Sampler


DEVICE_CHECK_EVERY = 32  # steps between reads of the kernels' error flags (generate() also reads them at its end)


@dataclass
class EngineStats:
    steps: int = 0
    prompt_tokens: int = 0  # hits of the prefix cache are counted in scheduler.num_cached_tokens
    computed_tokens: int = 0  # tokens actually run through the model
    generated_tokens: int = 0
    graph_steps: int = 0  # decode steps that replayed a captured graph
    prompt_graph_steps: int = 0  # steps of one short prompt that replayed a captured graph
    prepacked_steps: int = 0  # of those, steps that were launched while the step before ran
    dropped_steps: int = 0  # steps launched ahead that turned out not to be the next step
    step_batch_sizes: list[int] = field(default_factory=list)


@dataclass
class StepInFlight:
    """A decode step that was launched before the token ids of the step before it were read."""

    prepacked: Prepacked
    draw: Draw


def kv_cache_bytes_per_token(runner: ModelRunner) -> int:
    """Bytes of keys and values that one token occupies over all layers
    (src/mini_engine/engine.py:54-56)."""
    return runner.layout.bytes_per_token


class LLMEngine:
    def __init__(self, model: DecoderModel, config: EngineConfig, eos_token_ids: Iterable[int] = ()):
        if config.kv_memory_fraction is not None:
            free_bytes, _total = torch.cuda.mem_get_info()
            blocks = blocks_for_budget(
                model.cache_needs(), config.dtype, config.block_size, int(free_bytes * config.kv_memory_fraction)
            )
            config = dataclasses.replace(config, num_blocks=blocks)
        self.config = config
        self.model = model
        capacity = config.max_num_batched_tokens
        if config.cuda_graphs and model.capturable:
            # room for the bucket that a portion as long as the token budget replays (one token more at least)
            capacity = max(capacity, min((b for b in PROMPT_BUCKETS if b > capacity), default=capacity))
        self.runner = ModelRunner(
            model,
            dtype=config.dtype,
            num_blocks=config.num_blocks,
            block_size=config.block_size,
            max_num_seqs=config.max_num_seqs,
            max_num_batched_tokens=capacity,
            max_model_len=config.max_model_len,
            max_request_tokens=config.max_num_batched_tokens,
        )
        self.block_manager = CacheManager(
            self.runner.layout.groups,
            config.num_blocks,
            config.block_size,
            config.max_num_seqs,
            config.enable_prefix_caching,
            slot_groups=self.runner.layout.slot_groups,
        )
        self.scheduler = Scheduler(
            SchedulerConfig(config.max_num_seqs, config.max_num_batched_tokens, config.max_model_len),
            self.block_manager,
            set(eos_token_ids),
            # A step launched ahead may have to be dropped and run again; that is only harmless when
            # a step leaves nothing behind but keys and values (a mixer's own state would advance twice).
            rerun_safe=not self.runner.layout.has_state,
        )
        self.sampler = Sampler(config.seed, max(config.max_num_seqs, 1))
        self.stats = EngineStats()
        self._in_flight: StepInFlight | None = None  # the decode step after the current one, already launched
        self._rows_host = torch.empty((2, max(config.max_num_seqs, 1)), dtype=torch.int32).pin_memory()
        self._rows = torch.empty(max(config.max_num_seqs, 1), dtype=torch.int32, device="cuda")
        self.decode_graphs: DecodeGraphs | None = None
        self.prompt_graphs: PromptGraphs | None = None
        if config.cuda_graphs:
            self.decode_graphs = DecodeGraphs(self.runner, config.max_num_seqs)
            if model.capturable:  # steps of one short prompt replay a graph too (captured at first use)
                self.prompt_graphs = PromptGraphs(self.runner)

    # ----------------------------------------------------------------- loading

    @classmethod
    def from_pretrained(cls, model_path: str | Path, config: EngineConfig | None = None) -> "LLMEngine":
        """Load a checkpoint from a local folder with ``config.json`` and safetensors files
        (and ``generation_config.json`` for the end-of-sequence ids, if present)."""
        config = config or EngineConfig()
        _arch, model_config, model = load_model(model_path, config.dtype)
        return cls(model, config, getattr(model_config, "eos_token_ids", ()))

    @classmethod
    def from_random(cls, model_config: Any, seed: int = 0, config: EngineConfig | None = None, scale: float = 1.0) -> "LLMEngine":
        """An engine on seeded random weights of the given typed configuration."""
        config = config or EngineConfig()
        model = random_model(model_config, seed, config.dtype, scale=scale)
        return cls(model, config, getattr(model_config, "eos_token_ids", ()))

    # -------------------------------------------------------------------- API

    def add_request(self, prompt_token_ids: list[int], params: SamplingParams | None = None) -> Sequence:
        seq = Sequence(prompt_token_ids, params or SamplingParams())
        vocab = self.runner.vocab_size
        if min(seq.token_ids) < 0 or max(seq.token_ids) >= vocab:
            raise ValueError(f"prompt token ids must lie in [0, {vocab})")
        self.scheduler.add(seq)
        self.stats.prompt_tokens += len(seq)
        return seq

    def generate(self, prompts: list[list[int]], params: SamplingParams | None = None) -> list[list[int]]:
        """Run all prompts to completion as one continuously batched workload; returns the
        generated ids of each."""
        seqs = [self.add_request(p, params) for p in prompts]
        while self.scheduler.has_unfinished():
            self.step()
        ops.raise_on_device_error()
        return [s.output_token_ids for s in seqs]

    @torch.inference_mode()
    def step(self) -> list[Sequence]:
        """One iteration; returns the requests that finished in it.

        Decode steps overlap: when it is certain what the step after this one holds unless a
        request ends on the token drawn now, that step is launched before this one's token ids
        are read, fed on the device with what the sampler drew; scheduling and bookkeeping then
        run while the device works.  If a request does end (or a new one arrives), the next call
        finds that the step in flight is not the one the scheduler wants and drops it: it wrote
        keys and values only to places that the rerun writes again with the same values, or that
        belonged to the ended request."""
        plan = self.scheduler.plan()
        batch, entries = plan.items, plan.entries
        if not batch:
            raise RuntimeError("scheduler produced an empty batch with work pending")
        flight, self._in_flight = self._in_flight, None
        if flight is not None and not flight.prepacked.matches(entries):
            self.stats.dropped_steps += 1
            flight = None
        if flight is not None:
            draw, graph_step = flight.draw, True
            self.stats.prepacked_steps += 1
        else:
            graph_step = self._graph_fits(batch)
            if graph_step:
                logits = self.decode_graphs.run(entries)
            else:
                logits = self._run_prompt_step(batch, entries)
            draw = self._draw(batch, logits, 0)
        if graph_step:
            self.stats.graph_steps += 1
            # host work while the device runs: the scheduler says whether the step after is certain
            ahead = self.scheduler.plan_ahead(plan) if self.config.overlap_steps else None
            if ahead is not None:
                prepacked = self.decode_graphs.prepare(ahead.entries)
                rows = None
                if len(ahead.staying) < len(batch):  # the tokens of the requests that go on are picked on the device
                    count = len(ahead.staying)
                    host = self._rows_host[self.stats.steps & 1]  # its copy of two steps ago has run by now
                    host[:count] = torch.tensor([row for row, _ in ahead.staying], dtype=torch.int32)
                    rows = self._rows[:count]
                    rows.copy_(host[:count], non_blocking=True)
                logits = self.decode_graphs.run_prepared(prepacked, draw.tokens, rows)
                self._in_flight = StepInFlight(prepacked, self._draw([item for _, item in ahead.staying], logits, 1))
        sampled = self.sampler.collect(draw)
        tokens = iter(sampled)
        next_tokens = [next(tokens) if item.samples else None for item in batch]
        self._update_stats(batch)
        if self.stats.steps % DEVICE_CHECK_EVERY == 0:
            ops.raise_on_device_error()
        return self.scheduler.postprocess(batch, next_tokens)

    # ---------------------------------------------------------------- private

    def _draw(self, batch: list[ScheduledSeq], logits: torch.Tensor, ahead: int):
        """Launch the draw of one token for every request of `batch` that samples; `ahead` = 1 for
        the step after the one that `batch` describes (every request one token further)."""
        sampling = [item.seq for item in batch if item.samples]
        return self.sampler.launch(
            logits,
            [seq.params.temperature for seq in sampling],
            [seq.seq_id for seq in sampling],
            [seq.num_output_tokens + ahead for seq in sampling],
        )

    def _run_prompt_step(self, batch: list[ScheduledSeq], entries) -> torch.Tensor:
        """A step that is no pure decode step: eagerly, or, when it is one short prompt or portion
        alone, through the captured graph of its token-count bucket."""
        if self.prompt_graphs is not None and len(entries) == 1:
            logits = self.prompt_graphs.run(entries[0])
            if logits is not None:
                self.stats.prompt_graph_steps += 1
                return logits if batch[0].samples else logits[:0]
        return self.runner.execute(entries)

    def _graph_fits(self, batch: list[ScheduledSeq]) -> bool:
        graphs = self.decode_graphs
        if graphs is None or len(batch) > graphs.max_batch:
            return False
        return all(item.num_tokens == 1 and item.samples for item in batch)

    def _update_stats(self, batch: list[ScheduledSeq]) -> None:
        stats = self.stats
        stats.steps += 1
        stats.step_batch_sizes.append(len(batch))
        for item in batch:
            stats.computed_tokens += item.num_tokens
            stats.generated_tokens += int(item.samples)
