"""Where does a decode step spend its time?  Phase timers around the engine's own step.

    python -m mini_engine_b200.cli.profile_engine [--model DIR | --size 0.6b|8b] [--steps 30]

The counterpart of benchmarks/profile_engine.py of YuvGev00/mini-engine (its options ``--model``,
``--num-blocks``, ``--steps`` with the same meanings; ``--device`` is always CUDA here): it runs the
throughput workload (64 requests, 256-token prompts by default) until every request is decoding,
then times decode steps phase by phase and counts the kernel launches of a step.  The reference
re-implements its step with a CUDA sync after every phase; here the engine's own ``step`` runs,
with timers around the calls it makes, twice: once as it is (the device works while the host
schedules, so the phases overlap and their sum exceeds the step) and once with a synchronize after
every phase and without launching ahead (the phases in isolation, the device's share included).
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import time
from collections import defaultdict

import torch

SIZES = {
    "0.6b": dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16, tie_word_embeddings=True),
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32, tie_word_embeddings=False),
}  # fmt: skip


def build_engine(args: argparse.Namespace, overlap: bool):
    from mini_engine_b200 import EngineConfig, LLMEngine
    from mini_engine_b200.config import Qwen3Config

    config = EngineConfig(
        block_size=16, num_blocks=args.num_blocks, max_num_seqs=max(args.requests, 1), max_num_batched_tokens=8192,
        max_model_len=args.prompt_len + args.steps + 64, dtype=torch.bfloat16, overlap_steps=overlap,
    )  # fmt: skip
    if args.model:
        return LLMEngine.from_pretrained(args.model, config)
    model = Qwen3Config(
        vocab_size=151936, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
        max_position_embeddings=40960, **SIZES[args.size],
    )  # fmt: skip
    return LLMEngine.from_random(model, 0, config)


def timed(obj, name: str, label: str, totals: dict[str, float], sync: bool) -> None:
    """Replace ``obj.name`` by a wrapper that adds its wall time (after a synchronize, if asked) to
    ``totals[label]``."""
    inner = getattr(obj, name)

    def wrapper(*args, **kwargs):
        start = time.perf_counter()
        result = inner(*args, **kwargs)
        if sync:
            torch.cuda.synchronize()
        totals[label] += time.perf_counter() - start
        return result

    setattr(obj, name, wrapper)


def profile(args: argparse.Namespace, isolated: bool) -> dict:
    from mini_engine_b200 import SamplingParams
    from mini_engine_b200.csrc import ops

    engine = build_engine(args, overlap=not isolated)
    rng = random.Random(0)
    vocab = engine.runner.vocab_size
    params = SamplingParams(max_tokens=args.steps + 40, ignore_eos=True)
    seqs = [engine.add_request([rng.randrange(vocab) for _ in range(args.prompt_len)], params) for _ in range(args.requests)]
    while any(s.num_computed_tokens < s.num_prompt_tokens for s in seqs):
        engine.step()
    for _ in range(5):
        engine.step()
    totals: dict[str, float] = defaultdict(float)
    timed(engine.scheduler, "plan", "schedule", totals, isolated)
    timed(engine.decode_graphs, "run", "lay out + H2D + graph launch", totals, isolated)
    timed(engine.decode_graphs, "run_prepared", "token ids + H2D + graph launch (laid out ahead)", totals, isolated)
    timed(engine.scheduler, "plan_ahead", "plan the next step", totals, isolated)
    timed(engine.decode_graphs, "prepare", "lay out the next step", totals, isolated)
    timed(engine.sampler, "launch", "sampling kernel + D2H", totals, isolated)
    timed(engine.sampler, "collect", "wait for the token ids", totals, isolated)
    timed(engine.scheduler, "postprocess", "postprocess", totals, isolated)
    launches_before = ops.launch_count()
    torch.cuda.synchronize()
    began = time.perf_counter()
    for _ in range(args.steps):
        engine.step()
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - began
    bucket = engine.decode_graphs.bucket_for(args.requests)
    per_step = (ops.launch_count() - launches_before) / args.steps + engine.decode_graphs.launches[bucket]
    return {
        "mode": "phases in isolation (synchronize after each, no step launched ahead)" if isolated else "as it runs (phases overlap)",
        "ms_per_step": round(elapsed / args.steps * 1e3, 3),
        "tokens_per_second": round(args.requests * args.steps / elapsed, 1),
        "kernel_launches_per_step": round(per_step, 1),
        "steps_launched_ahead": engine.stats.prepacked_steps,
        "phases_us_per_step": {label: round(seconds / args.steps * 1e6, 1) for label, seconds in sorted(totals.items(), key=lambda kv: -kv[1])},
    }  # fmt: skip


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", help="folder with config.json and safetensors files (default: random weights of --size)")
    parser.add_argument("--size", choices=sorted(SIZES), default="0.6b")
    parser.add_argument("--num-blocks", type=int, default=2048)
    parser.add_argument("--steps", type=int, default=30)
    parser.add_argument("--requests", type=int, default=64)
    parser.add_argument("--prompt-len", type=int, default=256)
    args = parser.parse_args(argv)
    for isolated in (False, True):
        print(json.dumps(profile(args, isolated)), flush=True)
        torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    sys.exit(main())
