"""The reference's end-to-end workloads with seeded synthetic tokens and random weights.

    python -m mini_engine_b200.cli.workloads [--size 0.6b|8b|32b] [--layers N]

Shapes follow benchmarks/bench.py:56-62,113-123 of YuvGev00/mini-engine (Qwen3-0.6B layer sizes;
``block_size 16, num_blocks 2048, max_num_seqs 64, max_num_batched_tokens 8192, max_model_len
2048``; greedy, ``ignore_eos``; only output tokens count, wall time includes prompts and
scheduling):

* throughput: 64 requests, 256-token prompts, 128 output tokens each;
* prefix: 64 requests that share a 512-token prefix plus 32 tokens of their own, 64 output tokens,
  one request first and the other 63 together, with the prefix cache on and off.

With ``--size 32b`` (Qwen3-32B layer sizes, 65 GB of random bfloat16 weights) it runs the mixed
workload instead: steps of 8 prompt portions of 512 tokens beside 32 single decoded tokens at
4,096-token contexts, device-timed through the step function (the decoding requests' pages hold
random keys and values rather than computed ones); and the same mix through the scheduler with a
page pool too small for all requests, so that it has to preempt.

With ``--size 8b`` (Qwen3-8B layer sizes) it sweeps what ``bench.py`` measures at one point: one
prompt of 128 to 16,384 tokens through the step function (eager launches, host included), and
decode steps of a batch of 8 as captured graphs at contexts of 512 to 32,768 tokens.

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


def mixed_32b(layers: int) -> int:
    """8 prompt portions of 512 tokens beside 32 decoded tokens at 4,096-token contexts."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.config import Qwen3Config
    from mini_engine_b200.engine.runner import StepEntry

    cfg = Qwen3Config(
        vocab_size=151936, hidden_size=5120, intermediate_size=25600, num_hidden_layers=layers,
        num_attention_heads=64, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
        max_position_embeddings=40960, tie_word_embeddings=False,
    )  # fmt: skip
    rng = random.Random(0)

    def ids(n: int) -> list[int]:
        return [rng.randrange(100, cfg.vocab_size) for _ in range(n)]

    decodes, prompts, context, portion, steps = 32, 8, 4096, 512, 8
    engine = LLMEngine.from_random(
        cfg, 0,
        EngineConfig(block_size=16, num_blocks=decodes * (context // 16 + 2) + prompts * 64 + 8, max_num_seqs=64,
                     max_num_batched_tokens=8192, max_model_len=8192, dtype=torch.bfloat16, cuda_graphs=False),
    )  # fmt: skip
    runner, manager = engine.runner, engine.block_manager
    for array in runner.layout.arrays:
        array.normal_()  # the decoding requests' contexts: random keys and values
    deep = [manager.new_request() for _ in range(decodes)]
    fresh = [manager.new_request() for _ in range(prompts)]
    for cache in deep:
        assert manager.try_allocate(cache, context + 2 * steps + 2)
    for cache in fresh:
        assert manager.try_allocate(cache, 2 * portion)
    texts = [ids(2 * portion) for _ in range(prompts)]
    position = context

    def mixed_step(first_half: bool) -> None:
        nonlocal position
        lo = 0 if first_half else portion
        entries = [StepEntry(c, position, ids(1), (0,)) for c in deep]
        entries += [StepEntry(c, lo, t[lo : lo + portion], (portion - 1,) if not first_half else ()) for c, t in zip(fresh, texts)]
        runner.execute(entries)
        position += 1

    for i in range(2):
        mixed_step(i % 2 == 0)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(2 * steps):
        mixed_step(i % 2 == 0)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / (2 * steps)
    tokens = decodes + prompts * portion
    per_layer = cfg.hidden_size * (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    per_layer += cfg.num_attention_heads * cfg.head_dim * cfg.hidden_size + 3 * cfg.hidden_size * cfg.intermediate_size
    gemm_tflop = 2.0 * tokens * per_layer * layers / 1e12
    kv_gb = decodes * (context + steps) * 2 * cfg.num_key_value_heads * cfg.head_dim * 2 * layers / 1e9
    print(json.dumps({
        "workload": "mixed step, 32B sizes", "layers": layers, "tokens_per_step": tokens, "ms_per_step": round(ms, 3),
        "tokens_per_second": round(tokens / ms * 1e3, 1), "gemm_tflops": round(gemm_tflop / ms * 1e3, 1),
        "kv_gb_read_per_step": round(kv_gb, 2),
    }), flush=True)  # fmt: skip
    for cache in deep + fresh:
        manager.free(cache)
    manager.check_invariants([])
    del engine, runner, manager, deep, fresh, mixed_step
    torch.cuda.empty_cache()

    # The same mix through the scheduler, with too few pages for all requests at once.
    engine = LLMEngine.from_random(
        cfg, 0,
        EngineConfig(block_size=16, num_blocks=1400, max_num_seqs=64, max_num_batched_tokens=portion + decodes,
                     max_model_len=2048, dtype=torch.bfloat16, enable_prefix_caching=False),
    )  # fmt: skip
    params = SamplingParams(max_tokens=96, ignore_eos=True)
    requests = [ids(512) for _ in range(decodes)] + [ids(1024) for _ in range(prompts)]
    torch.cuda.synchronize()
    began = time.perf_counter()
    outputs = engine.generate(requests, params)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - began
    produced = sum(len(o) for o in outputs)
    engine.block_manager.check_invariants([])
    print(json.dumps({
        "workload": "32 x 512 in + 8 x 1,024 in, 96 out each, portions of 512, 1,400 pages", "layers": layers,
        "output_tokens": produced, "seconds": round(elapsed, 3), "tokens_per_second": round(produced / elapsed, 1),
        "steps": engine.stats.steps, "graph_steps": engine.stats.graph_steps,
        "preemptions": engine.scheduler.num_preemptions,
    }), flush=True)  # fmt: skip
    return 0


def sweep_8b(layers: int) -> int:
    """Prompt lengths, decode context lengths and decode batch sizes at Qwen3-8B layer sizes."""
    from mini_engine_b200 import EngineConfig, LLMEngine
    from mini_engine_b200.config import Qwen3Config
    from mini_engine_b200.engine.runner import StepEntry

    cfg = Qwen3Config(
        vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=layers,
        num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
        max_position_embeddings=40960, tie_word_embeddings=False,
    )  # fmt: skip
    batch, longest, most = 8, 32768, 128  # decode: 8 contexts of up to 32,768 tokens, up to 128 of 2,048
    engine = LLMEngine.from_random(
        cfg, 0,
        EngineConfig(block_size=16, num_blocks=max(batch * (longest // 16 + 8), most * (2048 // 16 + 4)) + 8, max_num_seqs=most,
                     max_num_batched_tokens=16384, max_model_len=longest + 64, enable_prefix_caching=False,
                     dtype=torch.bfloat16),
    )  # fmt: skip
    runner, manager, graphs = engine.runner, engine.block_manager, engine.decode_graphs
    rng = random.Random(0)

    def ids(n: int) -> list[int]:
        return [rng.randrange(100, cfg.vocab_size) for _ in range(n)]

    def timed(function, repeats: int) -> float:
        function()
        torch.cuda.synchronize()
        began = time.perf_counter()
        for _ in range(repeats):
            function()
        torch.cuda.synchronize()
        return (time.perf_counter() - began) / repeats * 1e3

    for tokens in (32, 60, 100, 127, 128, 512, 2048, 8192, 16384):
        cache = manager.new_request()
        assert manager.try_allocate(cache, tokens)
        entry = StepEntry(cache, 0, ids(tokens), (tokens - 1,))
        ms = timed(lambda: runner.execute([entry]), 3)
        row = {"prompt_tokens": tokens, "ms": round(ms, 2), "tokens_per_second": round(tokens / ms * 1e3)}
        if engine.prompt_graphs is not None and engine.prompt_graphs.bucket_for(tokens):
            # what LLMEngine.step does with a prompt that is alone in its step: the graph of its bucket
            row["ms_as_captured_graph"] = round(timed(lambda: engine.prompt_graphs.run(entry), 5), 2)
            row["bucket"] = engine.prompt_graphs.bucket_for(tokens)
        manager.free(cache)
        print(json.dumps(row), flush=True)
    weights = layers * (6144 * 4096 + 4096 * 4096 + 3 * 4096 * 12288) * 2 + cfg.vocab_size * 4096 * 2
    for array in runner.layout.arrays:
        array.normal_()  # contexts of random keys and values: only the time of a decode step is looked at
    caches = [manager.new_request() for _ in range(most)]
    shapes = [(batch, context) for context in (512, 2048, 8192, 32768)] + [(b, 2048) for b in (1, 2, 4, 16, 32, 64, 128)]
    for entries, context in shapes:
        for cache in caches:
            manager.free(cache)
        for cache in caches[:entries]:
            assert manager.try_allocate(cache, context + 40)
        position = [context]

        def step() -> None:
            graphs.run([StepEntry(c, position[0], [7], (0,)) for c in caches[:entries]])
            position[0] += 1

        ms = timed(step, 20)
        read = weights + entries * context * 2 * layers * 8 * 128 * 2
        print(json.dumps({"decode_batch": entries, "context": context, "ms_per_step": round(ms, 3),
                          "tokens_per_second": round(entries / ms * 1e3), "terabytes_per_second": round(read / ms / 1e9, 2)}), flush=True)  # fmt: skip
    return 0


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--size", choices=["0.6b", "8b", "32b"], default="0.6b")
    parser.add_argument("--layers", type=int, default=0, help="0: all layers of the size (28 or 64)")
    parser.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    args = parser.parse_args(argv)
    if args.size == "32b":
        return mixed_32b(args.layers or 64)
    if args.size == "8b":
        return sweep_8b(args.layers or 36)
    args.layers = args.layers or 28

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
        engine.block_manager.check_invariants([])  # every page is back and none is held twice
        row = {
            "workload": name, "output_tokens": tokens, "seconds": round(elapsed, 4),
            "tokens_per_second": round(tokens / elapsed, 1), "steps": engine.stats.steps,
            "graph_steps": engine.stats.graph_steps, "prompt_tokens_from_cache": engine.scheduler.num_cached_tokens,
            "preemptions": engine.scheduler.num_preemptions, "steps_launched_ahead": engine.stats.prepacked_steps,
            "steps_dropped": engine.stats.dropped_steps,
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
