"""Generate from the command line, in the manner of examples/generate.py of YuvGev00/mini-engine.

The reference's script takes ``--device`` and ``--max-tokens``, tokenises three questions that
share a long system prefix, runs the first request alone so that its prefix is cached before the
others arrive, and prints the answers and one line of statistics (examples/generate.py:26-49).
This one keeps those two options and that staging, and adds what a model folder without a
tokenizer or network needs: prompts as token ids, seeded random weights, and the engine's
options under the names of ``EngineConfig`` and ``SamplingParams``.

    python -m mini_engine_b200.cli.generate --model DIR --prompt-ids "1,2,3;4,5,6" --max-tokens 16
    python -m mini_engine_b200.cli.generate --random-weights CONFIG_DIR --seed 0 --max-tokens 8
"""

from __future__ import annotations

import argparse
import random
import sys
import tempfile
import time

import torch


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    source = parser.add_mutually_exclusive_group(required=True)
    source.add_argument("--model", help="folder with config.json and safetensors files")
    source.add_argument("--random-weights", metavar="CONFIG_DIR", help="folder with a config.json; weights are seeded random")
    parser.add_argument("--device", default="cuda", help="only 'cuda' is supported")
    parser.add_argument("--dtype", choices=["bf16", "fp32", "bfloat16", "float32"], default="bf16")
    parser.add_argument("--max-tokens", type=int, default=32)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--num-blocks", type=int, default=128)
    parser.add_argument("--kv-memory-fraction", type=float, default=None,
                        help="size the KV pool as this fraction of free device memory instead of --num-blocks")
    parser.add_argument("--max-num-seqs", type=int, default=16)
    parser.add_argument("--max-num-batched-tokens", type=int, default=2048)
    parser.add_argument("--max-model-len", type=int, default=4096)
    parser.add_argument("--no-prefix-cache", action="store_true")
    parser.add_argument("--no-cuda-graphs", action="store_true")
    parser.add_argument("--prompt", action="append", help="text prompt (needs tokenizer files in the model folder)")
    parser.add_argument("--prompt-ids", help="token ids: requests separated by ';', ids by ','")
    return parser


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    if not args.device.startswith("cuda"):
        print(f"error: this engine runs on CUDA only, not on {args.device!r}", file=sys.stderr)
        return 2
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.config import load_model_config
    from mini_engine_b200.weights import write_random_model

    dtype = torch.bfloat16 if args.dtype in ("bf16", "bfloat16") else torch.float32
    config = EngineConfig(
        block_size=args.block_size, num_blocks=args.num_blocks, max_num_seqs=args.max_num_seqs,
        max_num_batched_tokens=args.max_num_batched_tokens, max_model_len=args.max_model_len,
        enable_prefix_caching=not args.no_prefix_cache, dtype=dtype, seed=args.seed,
        cuda_graphs=not args.no_cuda_graphs, kv_memory_fraction=args.kv_memory_fraction,
    )  # fmt: skip
    scratch = None
    folder = args.model
    if args.random_weights:
        _arch, model_config = load_model_config(args.random_weights)
        scratch = tempfile.TemporaryDirectory()
        folder = write_random_model(scratch.name, model_config, args.seed, torch.bfloat16 if dtype == torch.bfloat16 else torch.float32)
    engine = LLMEngine.from_pretrained(folder, config)
    vocab = engine.runner.vocab_size

    tokenizer = None
    if args.prompt:
        from transformers import AutoTokenizer  # a tokenizer only; no model code of the library is used

        tokenizer = AutoTokenizer.from_pretrained(folder)
        prompts = [tokenizer(text).input_ids for text in args.prompt]
    elif args.prompt_ids:
        prompts = [[int(t) for t in part.split(",") if t.strip()] for part in args.prompt_ids.split(";") if part.strip()]
    else:
        # Three requests that share a prefix longer than a few pages, as the reference's demo does.
        rng = random.Random(args.seed)
        shared = [rng.randrange(vocab) for _ in range(4 * args.block_size + 3)]
        prompts = [shared + [rng.randrange(vocab) for _ in range(rng.randrange(3, 12))] for _ in range(3)]

    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, ignore_eos=args.ignore_eos)
    torch.cuda.synchronize()
    start = time.perf_counter()
    # The first request warms the prefix cache; the rest are batched and reuse it.
    outputs = engine.generate(prompts[:1], params) + (engine.generate(prompts[1:], params) if prompts[1:] else [])
    elapsed = time.perf_counter() - start
    for prompt, out in zip(prompts, outputs):
        if tokenizer is not None:
            print(f"Q: {tokenizer.decode(prompt)}\nA: {tokenizer.decode(out, skip_special_tokens=True).strip()}\n")
        else:
            print(f"prompt ({len(prompt)} tokens) -> {out}")
    stats = engine.stats
    print(
        f"{stats.generated_tokens} tokens in {elapsed:.1f}s over {stats.steps} steps | "
        f"prompt tokens {stats.prompt_tokens}, served from prefix cache {engine.scheduler.num_cached_tokens}"
    )
    if scratch is not None:
        scratch.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
