"""The reference's end-to-end workloads with seeded synthetic tokens and random weights.

    python -m mini_engine_b200.cli.workloads [--layers N]

Shapes follow benchmarks/bench.py:56-62,113-123 of YuvGev00/mini-engine (Qwen3-0.6B layer sizes;
``block_size 16, num_blocks 2048, max_num_seqs 64, max_num_batched_tokens 8192, max_model_len
2048``; greedy, ``ignore_eos``; only output tokens count, wall time includes prompts and
scheduling):

* throughput: 64 requests, 256-token prompts, 128 output tokens each;
* prefix: 64 requests that share a 512-token prefix plus 32 tokens of their own, 64 output tokens,
  one request first and the other 63 together, with the prefix cache on and off.

Token ids are uniform random from a fixed seed (the reference draws its prompts the same way,
benchmarks/bench.py:52-53).
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import time

import torch


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--layers", type=int, default=28)
    parser.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    args = parser.parse_args(argv)

    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.config import Qwen3Config

    cfg = Qwen3Config(
        vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=args.layers,
        num_attention_heads=16, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
        max_position_embeddings=40960, tie_word_embeddings=True,
    )  # fmt: skip
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    rng = random.Random(0)

    def ids(n: int) -> list[int]:
        return [rng.randrange(100, cfg.vocab_size) for _ in range(n)]

    throughput = [ids(256) for _ in range(64)]
    shared = ids(512)
    prefix = [shared + ids(32) for _ in range(64)]

    def run(name: str, prompts, max_tokens: int, staged: bool, prefix_cache: bool) -> dict:
        engine = LLMEngine.from_random(
            cfg, 0,
            EngineConfig(block_size=16, num_blocks=2048, max_num_seqs=64, max_num_batched_tokens=8192,
                         max_model_len=2048, enable_prefix_caching=prefix_cache, dtype=dtype),
        )  # fmt: skip
        params = SamplingParams(max_tokens=max_tokens, ignore_eos=True)
        torch.cuda.synchronize()
        began = time.perf_counter()
        if staged:
            outputs = engine.generate(prompts[:1], params) + engine.generate(prompts[1:], params)
        else:
            outputs = engine.generate(prompts, params)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - began
        tokens = sum(len(o) for o in outputs)
        row = {
            "workload": name, "output_tokens": tokens, "seconds": round(elapsed, 4),
            "tokens_per_second": round(tokens / elapsed, 1), "steps": engine.stats.steps,
            "graph_steps": engine.stats.graph_steps, "prompt_tokens_from_cache": engine.scheduler.num_cached_tokens,
            "preemptions": engine.scheduler.num_preemptions,
        }  # fmt: skip
        print(json.dumps(row), flush=True)
        return row

    run("warm-up", throughput[:4], 4, False, True)
    run("throughput", throughput, 128, False, True)
    run("prefix, cache off", prefix, 64, True, False)
    run("prefix, cache on", prefix, 64, True, True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
