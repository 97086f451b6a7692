"""Trace replay: feed given token ids step by step, write logits, sample nothing.

Every step's entries are one batch for :meth:`ModelRunner.execute`; pages come from the
engine's :class:`CacheManager` with a pool sized by ``--max-tokens``, so that pages of ended
requests are handed out again.  For a step in which something is wanted, ``<out>/<step>.f32``
holds the logits at the wanted places, in the order of the entries and of ``want``, as
little-endian float32 ``[wanted, vocab]``.  After every step ``done <step>`` is printed and
flushed.

The reference has no such program; its nearest pieces are the whole-prompt logits recipe of
tests/test_parity.py:67-77 and the hand-rolled step of benchmarks/profile_engine.py:33-58
(YuvGev00/mini-engine).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

PAGE_SIZE = 16  # tokens per page; --max-tokens counts requests rounded up to 64, a multiple of it
MAX_LIVE = 4


class Replayer:
    """The model, its step function and a cache manager whose pool holds ``max_tokens``."""

    def __init__(
        self,
        model_dir: str | Path,
        dtype: torch.dtype,
        max_tokens: int,
        block_size: int = PAGE_SIZE,
        max_step_tokens: int | None = None,
    ):
        from mini_engine_b200.cache.manager import CacheManager
        from mini_engine_b200.engine.loading import load_model
        from mini_engine_b200.engine.runner import ModelRunner

        self.block_size = block_size
        self.num_blocks = max(-(-max_tokens // block_size), 1)
        _arch, self.config, model = load_model(model_dir, dtype)
        self.runner = ModelRunner(
            model,
            dtype=dtype,
            num_blocks=self.num_blocks,
            block_size=block_size,
            max_num_seqs=MAX_LIVE * 2,
            max_num_batched_tokens=max_step_tokens or max(max_tokens, 64),
            max_model_len=self.num_blocks * block_size,
        )
        self.manager = CacheManager(
            self.runner.layout.groups,
            self.num_blocks,
            block_size,
            max_num_seqs=MAX_LIVE * 2,
            enable_prefix_caching=False,
            slot_groups=self.runner.layout.slot_groups,
        )
        self.live: dict[str, list] = {}  # id -> [RequestCache, tokens held]

    def step(self, record: dict) -> torch.Tensor | None:
        """Run one step record; return the wanted logits ``[wanted, vocab]`` on the host, or
        ``None`` when nothing was wanted."""
        from mini_engine_b200.csrc import ops
        from mini_engine_b200.engine.runner import StepEntry

        entries = []
        for item in record.get("entries", []):
            name = item["id"]
            if name not in self.live:
                self.live[name] = [self.manager.new_request(), 0]
            cache, held = self.live[name]
            tokens = [int(t) for t in item["tokens"]]
            if not self.manager.try_allocate(cache, held + len(tokens)):
                raise MemoryError(
                    f"step {record.get('step')}: request {name!r} needs {held + len(tokens)} tokens but the "
                    f"pool of {self.num_blocks * self.block_size} tokens (--max-tokens) is exhausted"
                )
            entries.append(StepEntry(cache, held, tokens, tuple(item.get("want", ()))))
            self.live[name][1] = held + len(tokens)
        result = None
        if entries:
            logits = self.runner.execute(entries)
            if logits.shape[0]:
                result = logits.to("cpu")
            else:
                torch.cuda.synchronize()
            ops.raise_on_device_error()
            for entry in entries:
                self.manager.release_behind_window(entry.cache, entry.start + len(entry.token_ids))
        for name in record.get("end", []):
            if name in self.live:
                self.manager.free(self.live.pop(name)[0])
        return result


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    parser.add_argument("--block-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    parser.add_argument("--max-step-tokens", type=int, default=None, help="most tokens in one step")
    args = parser.parse_args(argv)

    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    replayer = Replayer(args.model, dtype, args.max_tokens, args.block_size, args.max_step_tokens)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        try:
            logits = replayer.step(record)
        except MemoryError as error:
            print(f"error: {error}", file=sys.stderr)
            return 2
        if logits is not None:
            logits.contiguous().numpy().astype("<f4", copy=False).tofile(out_dir / f"{record['step']}.f32")
        print(f"done {record['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
