"""What each class of kernels costs INSIDE a captured decode step.

    python -m mini_engine_b200.cli.step_costs [--batch 8] [--context 2048] [--size 8b|0.6b] [--layers N]

Kernels of a replayed graph overlap each other's start and end (programmatic dependent launch), so
the time of a kernel alone says little about its share of the step.  This captures the decode step
several times, each time with one class of launches left out (the norms, the fused norm / rotation /
cache write, decode attention, or all three, which leaves the matrix products), and prints the
step's time for each; the difference to the whole step is the class's cost in place.  The results
of the shortened steps are wrong, only their time is looked at.  YuvGev00/mini-engine's
benchmarks/profile_engine.py times phases with a synchronize after each; a captured graph has no
place for one.
"""

from __future__ import annotations

import argparse
import json
import sys

import torch

CLASSES = {
    "norms": ("add_rmsnorm",),
    "norm_rotation_cache_write": ("qk_norm_rope_store",),
    "decode_attention": ("paged_attention",),
    "all_but_products": ("add_rmsnorm", "qk_norm_rope_store", "paged_attention"),
}


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=2048)
    parser.add_argument("--size", choices=["8b", "0.6b"], default="8b")
    parser.add_argument("--layers", type=int, default=0, help="0: all layers of the size")
    parser.add_argument("--steps", type=int, default=40)
    args = parser.parse_args(argv)

    from mini_engine_b200 import EngineConfig, LLMEngine
    from mini_engine_b200.cli.profile_engine import SIZES
    from mini_engine_b200.config import Qwen3Config
    from mini_engine_b200.csrc import ops
    from mini_engine_b200.engine.graphs import DecodeGraphs
    from mini_engine_b200.engine.runner import StepEntry

    sizes = dict(SIZES[args.size])
    if args.layers:
        sizes["num_hidden_layers"] = args.layers
    cfg = Qwen3Config(
        vocab_size=151936, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
        max_position_embeddings=40960, **sizes,
    )  # fmt: skip
    room = args.context + args.steps + 8  # every class starts again at the same position
    pages = -(-room // 16)
    engine = LLMEngine.from_random(
        cfg, 0,
        EngineConfig(block_size=16, num_blocks=args.batch * pages + 8, max_num_seqs=args.batch,
                     max_num_batched_tokens=max(args.batch, 64), max_model_len=pages * 16,
                     dtype=torch.bfloat16, enable_prefix_caching=False, cuda_graphs=False),
    )  # fmt: skip
    runner, manager = engine.runner, engine.block_manager
    for array in runner.layout.arrays:
        array.normal_()  # contexts of random keys and values: only the step's time is looked at
    caches = [manager.new_request() for _ in range(args.batch)]
    for cache in caches:
        assert manager.try_allocate(cache, room)

    real = {name: getattr(ops, name) for names in CLASSES.values() for name in names}
    left_out: set[str] = set()

    def wrapper(name: str):
        def call(*a, **k):
            return None if name in left_out else real[name](*a, **k)

        return call

    for name in real:
        setattr(ops, name, wrapper(name))
    position = [args.context]
    whole = None
    try:
        for label, names in [("whole step", ())] + list(CLASSES.items()):
            left_out.clear()
            left_out.update(names)
            position[0] = args.context
            graphs = DecodeGraphs(runner, args.batch)  # captured with these launches left out

            def step() -> None:
                graphs.run([StepEntry(c, position[0], [7], (0,)) for c in caches])
                position[0] += 1

            for _ in range(5):
                step()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(args.steps):
                step()
            end.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(end) / args.steps
            whole = ms if whole is None else whole
            row = {"left_out": label if names else None, "ms_per_step": round(ms, 4),
                   "launches": graphs.launches[graphs.bucket_for(args.batch)]}  # fmt: skip
            if names:
                row["cost_in_place_ms"] = round(whole - ms, 4)
            print(json.dumps(row), flush=True)
    finally:
        for name, function in real.items():
            setattr(ops, name, function)
    return 0


if __name__ == "__main__":
    sys.exit(main())
