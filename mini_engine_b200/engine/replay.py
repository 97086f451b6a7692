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


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    parser.add_argument("--block-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    parser.add_argument("--max-step-tokens", type=int, default=None, help="most tokens in one step")
    args = parser.parse_args(argv)

    from mini_engine_b200.cache.manager import CacheManager
    from mini_engine_b200.engine.loading import load_model
    from mini_engine_b200.engine.runner import ModelRunner, StepEntry

    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    block_size = args.block_size
    num_blocks = max(-(-args.max_tokens // block_size), 1)
    step_tokens = args.max_step_tokens or max(args.max_tokens, 64)
    _arch, _config, model = load_model(args.model, dtype)
    runner = ModelRunner(
        model,
        dtype=dtype,
        num_blocks=num_blocks,
        block_size=block_size,
        max_num_seqs=MAX_LIVE * 2,
        max_num_batched_tokens=step_tokens,
        max_model_len=num_blocks * block_size,
    )
    manager = CacheManager(
        runner.layout.groups,
        num_blocks,
        block_size,
        max_num_seqs=MAX_LIVE * 2,
        enable_prefix_caching=False,
        has_state=runner.layout.has_state,
    )
    live: dict[str, tuple] = {}  # id -> (RequestCache, tokens so far)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            name = item["id"]
            if name not in live:
                live[name] = (manager.new_request(), 0)
            cache, held = live[name]
            tokens = [int(t) for t in item["tokens"]]
            if not manager.try_allocate(cache, held + len(tokens)):
                print(
                    f"error: step {step}: request {name!r} needs {held + len(tokens)} tokens but the pool of "
                    f"{num_blocks * block_size} (--max-tokens) is exhausted",
                    file=sys.stderr,
                )
                return 2
            entries.append(StepEntry(cache, held, tokens, tuple(item.get("want", ()))))
            live[name] = (cache, held + len(tokens))
        if entries:
            logits = runner.execute(entries)
            if logits.shape[0]:
                logits.to("cpu").contiguous().numpy().astype("<f4", copy=False).tofile(out_dir / f"{step}.f32")
            else:
                torch.cuda.synchronize()
            for entry in entries:
                manager.release_behind_window(entry.cache, entry.start + len(entry.token_ids))
        for name in record.get("end", []):
            if name in live:
                manager.free(live.pop(name)[0])
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
