#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

The default run builds the Qwen3-8B layer sizes with seeded random bfloat16 weights, fills the
cache of 8 requests with 2,048-token contexts, and times K decode steps (one token for every
request per step) as captured CUDA graphs, with CUDA events on the launching stream.  It
prints ONE JSON line: ``value`` is decoded tokens per second on the device; ``e2e`` is the
same through ``LLMEngine.step`` (host token ids in, sampled ids out, scheduler and copies
included); ``prefill`` times one 2,048-token prompt; ``roofline`` is the bytes a decode step
must read (every weight once plus the live requests' cache) over its time, against the
measured copy bandwidth; ``points`` adds decode at batch 1 and 64; ``workloads`` the reference's
own two end-to-end workloads at Qwen3-0.6B layer sizes (output tokens per second, wall time).
``fp32_check`` compares the bfloat16 logits of a 256-token prompt with the true 32-bit path of the
same full-size model.  ``--impl reference`` measures through the unmodified reference engine instead.

Every step reads about 15 GB of weights, far more than the 126 MB L2, so no flush is needed
between timed iterations (``config.l2`` says so).
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# BASELINE.json configs[2]: Qwen3-8B layer sizes.
QWEN3_8B = dict(
    vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
    max_position_embeddings=40960, tie_word_embeddings=False,
)  # fmt: skip
# BASELINE.json configs[3]: Qwen3-0.6B layer sizes, for the reference's own two end-to-end workloads.
QWEN3_0P6B = dict(
    vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
    num_attention_heads=16, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
    max_position_embeddings=40960, tie_word_embeddings=True,
)  # fmt: skip
# Engine settings of those workloads (benchmarks/bench.py:113-123 of YuvGev00/mini-engine).
WORKLOAD_ENGINE = dict(block_size=16, num_blocks=2048, max_num_seqs=64, max_num_batched_tokens=8192, max_model_len=2048)
CONTEXT = 2048  # tokens each request holds when decode is timed
REPEATS = 3  # the timed decode region is run this often; the median counts, the spread is printed
PREFILL_TOKENS = 2048
MAX_MODEL_LEN = 4096  # benchmark context length of the configuration
BLOCK_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {
                "hbm_gbs": float(raw["hbm_gbs"]),
                "bf16_tflops": float(raw["bf16_tflops"]),  # best single product (burst)
                # a product repeated for seconds under the power cap; the prefill is such a step
                "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained") or raw["bf16_tflops"]),
                "source": "measured",
            }
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = (
        "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5,
                ).stdout.strip()  # fmt: skip
                if out:
                    self.samples.append([f.strip() for f in out.splitlines()[0].split(",")])
            except (OSError, subprocess.SubprocessError):
                return
            self._stop.wait(0.2)

    def __enter__(self) -> "ClockSampler":
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc) -> None:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=6)

    def summary(self) -> dict:
        clocks = [int(s[0]) for s in self.samples if s and s[0].isdigit()]
        maxima = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        reasons = sorted(
            {name for s in self.samples for name, flag in zip(self.NAMES, s[2:]) if flag.lower().startswith("active")}
        )
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max(maxima) if maxima else None,
            "reasons": reasons,
            "samples": len(clocks),
        }


def workload_prompts(vocab: int) -> tuple[list[list[int]], list[list[int]]]:
    """Seeded synthetic prompts in the shapes of the reference's two workloads
    (benchmarks/bench.py:52-62): 64 x 256 tokens; 64 x (512 shared + 32 own)."""
    import random

    rng = random.Random(0)

    def ids(n: int) -> list[int]:
        return [rng.randrange(100, vocab) for _ in range(n)]

    shared = ids(512)
    return [ids(256) for _ in range(64)], [shared + ids(32) for _ in range(64)]


def run_workloads(make_engine, generate, synchronize) -> dict:
    """Output tokens per second of the two workloads, wall time with prompts and scheduling
    included, as the reference counts them (benchmarks/bench.py:18,267-277): 64 requests of 256 in
    and 128 out; 64 requests of 512 shared + 32 in and 64 out, one first and then the other 63,
    with the prefix cache on.  ``make_engine()`` builds a fresh engine, ``generate(engine, prompts,
    max_tokens)`` returns the generated ids."""
    throughput, prefix = workload_prompts(QWEN3_0P6B["vocab_size"])
    generate(make_engine(), throughput[:4], 4)  # warm-up: kernels built, graphs captured once
    out = {}
    engine = make_engine()
    synchronize()
    began = time.perf_counter()
    tokens = sum(len(o) for o in generate(engine, throughput, 128))
    synchronize()
    out["qwen3_0.6b_64x(256in,128out)_tok_s"] = round(tokens / (time.perf_counter() - began), 1)
    engine = make_engine()
    synchronize()
    began = time.perf_counter()
    tokens = sum(len(o) for o in generate(engine, prefix[:1], 64) + generate(engine, prefix[1:], 64))
    synchronize()
    out["qwen3_0.6b_64x(512shared+32in,64out)_tok_s"] = round(tokens / (time.perf_counter() - began), 1)
    out["published_on_L4_tok_s"] = [1982.4, 1691.0]  # the reference's own numbers for these two, another GPU
    return out


def decode_bytes(cfg, layers: int, batch: int, context: int) -> float:
    """Bytes one decode step has to read: every weight it uses once (the embedding table is
    only touched at ``batch`` rows) and the keys and values of the live requests."""
    d, h, inter = cfg.head_dim, cfg.hidden_size, cfg.intermediate_size
    per_layer = ((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * d * h + cfg.num_attention_heads * d * h + 3 * h * inter) * 2
    head = cfg.vocab_size * h * 2
    kv = 2 * layers * cfg.num_key_value_heads * d * 2 * context * batch
    return per_layer * layers + head + kv


def prefill_flops(cfg, layers: int, tokens: int) -> float:
    d, h, inter = cfg.head_dim, cfg.hidden_size, cfg.intermediate_size
    gemm = 2.0 * tokens * ((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * d * h + cfg.num_attention_heads * d * h + 3 * h * inter)
    attention = 2.0 * 2.0 * cfg.num_attention_heads * d * tokens * (tokens + 1) / 2  # causal QK^T and PV
    return layers * (gemm + attention) + 2.0 * cfg.vocab_size * h  # one row of logits


def run_ours(args) -> dict:
    import torch

    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.config import Qwen3Config
    from mini_engine_b200.csrc import ops, tensor_core
    from mini_engine_b200.engine.runner import StepEntry

    sizes = dict(QWEN3_8B)
    full_layers = sizes["num_hidden_layers"]
    if args.layers:
        sizes["num_hidden_layers"] = args.layers
    cfg = Qwen3Config(**sizes)
    layers = cfg.num_hidden_layers
    peaks = load_peaks()
    max_batch = max(args.batch, 64 if not args.skip_points else args.batch)
    steps_total = REPEATS * args.steps + args.warmup + 8
    pages_per_request = -(-(CONTEXT + steps_total + 1) // BLOCK_SIZE)
    engine_config = EngineConfig(
        block_size=BLOCK_SIZE, num_blocks=max_batch * pages_per_request + 8, max_num_seqs=max_batch,
        max_num_batched_tokens=max(PREFILL_TOKENS, max_batch), max_model_len=MAX_MODEL_LEN,
        enable_prefix_caching=False, dtype=torch.bfloat16, seed=0, cuda_graphs=True,
    )  # fmt: skip
    torch.manual_seed(0)
    engine = LLMEngine.from_random(cfg, seed=0, config=engine_config)
    runner, graphs = engine.runner, engine.decode_graphs
    generator = torch.Generator().manual_seed(1)
    sampled = torch.empty(max_batch, dtype=torch.int32, device="cuda")

    def random_prompt(n: int) -> list[int]:
        return torch.randint(0, cfg.vocab_size, (n,), generator=generator).tolist()

    # ---------------------------------------------------------------- prefill, device timed
    def time_prefill() -> float:
        cache = engine.block_manager.new_request()
        assert engine.block_manager.try_allocate(cache, PREFILL_TOKENS)
        entry = StepEntry(cache, 0, random_prompt(PREFILL_TOKENS), (PREFILL_TOKENS - 1,))
        times = []
        for i in range(3 + 3):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.execute([entry])
            end.record()
            torch.cuda.synchronize()
            if i >= 3:
                times.append(start.elapsed_time(end))
        engine.block_manager.free(cache)
        return statistics.median(times)

    prefill_ms = time_prefill()

    # ------------------------------------------------------------ decode, device timed
    def fill_contexts(batch: int) -> list:
        caches = []
        for _ in range(batch):
            cache = engine.block_manager.new_request()
            assert engine.block_manager.try_allocate(cache, CONTEXT + steps_total + 1)
            runner.execute([StepEntry(cache, 0, random_prompt(CONTEXT), ())])
            caches.append(cache)
        torch.cuda.synchronize()
        return caches

    def time_decode(batch: int, steps: int, warmup: int, repeats: int) -> tuple[list[float], int]:
        """Times ``repeats`` regions of ``steps`` decode steps each, one after the other (the
        contexts go on growing); returns the milliseconds per step of every region."""
        caches = fill_contexts(batch)
        tokens = random_prompt(batch)
        position = CONTEXT
        launches_before = 0

        def one_step() -> None:
            nonlocal position
            entries = [StepEntry(c, position, [tokens[i]], (0,)) for i, c in enumerate(caches)]
            logits = graphs.run(entries)
            ops.sample(logits, None, None, sampled[:batch])
            position += 1

        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        regions, launches = [], 0
        for _ in range(repeats):
            launches_before = ops.launch_count()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(steps):
                one_step()
            end.record()
            torch.cuda.synchronize()
            regions.append(start.elapsed_time(end) / steps)
            launches = ops.launch_count() - launches_before + graphs.launches[graphs.bucket_for(batch)] * steps
        for cache in caches:
            engine.block_manager.free(cache)
        return regions, launches

    with ClockSampler() as clocks:
        regions, launches = time_decode(args.batch, args.steps, args.warmup, REPEATS)
    clock_summary = clocks.summary()
    ms_per_step = statistics.median(regions)
    value = args.batch / (ms_per_step / 1e3)

    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            ms = statistics.median(time_decode(batch, max(args.steps // 2, 5), args.warmup, REPEATS)[0])
            points[f"decode_b{batch}"] = round(batch / (ms / 1e3), 1)
            points[f"decode_b{batch}_ms"] = round(ms, 4)

    # ------------------------------------------------- decode through the Python entry point
    def time_e2e(batch: int, steps: int, warmup: int) -> tuple[float, int, int]:
        # The first requests already decode while the later ones' prompts run (one step per prompt
        # under this token budget): room for those tokens too, so that nobody ends inside the timed steps.
        params = SamplingParams(max_tokens=steps + warmup + batch + 2, ignore_eos=True)
        seqs = [engine.add_request(random_prompt(CONTEXT), params) for _ in range(batch)]
        while any(s.num_computed_tokens < s.num_prompt_tokens for s in seqs):
            engine.step()  # prompts, in portions under the token budget
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        began = time.perf_counter()
        h2d = 0
        for _ in range(steps):
            engine.step()
            h2d = max(h2d, runner.last_h2d_bytes)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - began
        while engine.scheduler.has_unfinished():
            engine.step()
        return batch * steps / elapsed, h2d, 4 * batch

    e2e_value, h2d_bytes, d2h_bytes = time_e2e(args.batch, args.steps, args.warmup)
    device_error = tensor_core.take_error()
    fp32_check = None
    if args.fp32_check:
        fp32_check = check_against_fp32(engine, cfg, random_prompt(args.fp32_check))

    workloads = None
    if not args.skip_workloads:
        del engine, runner, graphs
        torch.cuda.empty_cache()
        small = Qwen3Config(**QWEN3_0P6B)
        workloads = run_workloads(
            lambda: LLMEngine.from_random(small, 0, EngineConfig(dtype=torch.bfloat16, **WORKLOAD_ENGINE)),
            lambda engine, prompts, n: engine.generate(prompts, SamplingParams(max_tokens=n, ignore_eos=True)),
            torch.cuda.synchronize,
        )
        device_error = device_error or tensor_core.take_error()
    return result_line(
        "ours", cfg, layers, full_layers, args, peaks, regions, e2e_value, h2d_bytes, d2h_bytes, prefill_ms, points,
        clock_summary, "captured CUDA graph per step + sampling kernel",
        gpu_launches=launches, device_error=device_error, **({"fp32_check": fp32_check} if fp32_check else {}),
        **({"workloads": workloads} if workloads else {}),
    )  # fmt: skip


def result_line(impl, cfg, layers, full_layers, args, peaks, regions, e2e_value, h2d_bytes, d2h_bytes, prefill_ms,
                points, clock_summary, decode_path, **more) -> dict:  # fmt: skip
    """The one JSON line of a run; both arms print the same keys from the same formulas."""
    ms_per_step = statistics.median(regions)
    middle = CONTEXT + args.warmup + len(regions) * args.steps // 2  # mean context length of the timed steps
    achieved_gbs = decode_bytes(cfg, layers, args.batch, middle) / (ms_per_step / 1e3) / 1e9
    tflops = prefill_flops(cfg, layers, PREFILL_TOKENS) / (prefill_ms / 1e3) / 1e12
    return {
        "metric": "decode tok/s at batch 8, 2,048-token contexts (Qwen3-8B layer sizes)",
        "value": round(args.batch / (ms_per_step / 1e3), 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4),
        "ms_per_step_regions": [round(r, 4) for r in regions],
        "spread": round((max(regions) - min(regions)) / ms_per_step, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded random token ids, random-init weights N(0, 0.02)",
        "impl": impl,
        "config": {
            "model": "Qwen3-8B layer sizes",
            "layers": layers,
            "layers_of_configuration": full_layers,
            "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size,
            "vocab": cfg.vocab_size,
            "global_batch": args.batch,
            "seq_len": CONTEXT,
            "max_model_len": MAX_MODEL_LEN,
            "kv_block_size": BLOCK_SIZE,
            "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single GPU",
            "l2": "inputs larger than L2: each step reads all weights",
            "peaks": peaks["source"],
        },
        "decode_path": decode_path,
        "e2e": {
            "value": round(e2e_value, 1),
            "unit": "tokens/s",
            "h2d_bytes_per_step": h2d_bytes,
            "d2h_bytes_per_step": d2h_bytes,
        },
        "prefill": {
            "value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1),
            "tokens": PREFILL_TOKENS,
            "ms": round(prefill_ms, 3),
            "tflops": round(tflops, 1),
            # a 2,048-token step lasts tens of milliseconds under the power cap: the sustained peak
            "frac": round(tflops / peaks["bf16_tflops_sustained"], 4),
            "frac_of_burst": round(tflops / peaks["bf16_tflops"], 4),
            "peak_tflops_sustained": peaks["bf16_tflops_sustained"],
            "peak_tflops_burst": peaks["bf16_tflops"],
        },
        "roofline": {
            "bound": "hbm",
            "achieved": round(achieved_gbs, 1),
            "peak": peaks["hbm_gbs"],
            "unit": "GB/s",
            "frac": round(achieved_gbs / peaks["hbm_gbs"], 4),
        },
        "points": points,
        "clocks": clock_summary,
        **more,
    }


def check_against_fp32(engine, cfg, prompt: list[int]) -> dict:
    """Logits of one prompt from the bfloat16 engine against the true 32-bit path of the same
    model (the same weights, widened to float32; CUDA-core products, no tensor cores)."""
    import torch

    from mini_engine_b200.cache.manager import CacheManager
    from mini_engine_b200.engine.loading import random_model
    from mini_engine_b200.engine.runner import ModelRunner, StepEntry

    def logits_of(runner, manager) -> "torch.Tensor":
        cache = manager.new_request()
        assert manager.try_allocate(cache, len(prompt))
        out = runner.execute([StepEntry(cache, 0, prompt, tuple(range(len(prompt))))]).float().cpu()
        manager.free(cache)
        return out

    low = logits_of(engine.runner, engine.block_manager)
    pages = -(-len(prompt) // BLOCK_SIZE) + 1
    began = time.perf_counter()
    model32 = random_model(cfg, seed=0, dtype=torch.float32, store=torch.bfloat16)
    runner32 = ModelRunner(model32, dtype=torch.float32, num_blocks=pages, block_size=BLOCK_SIZE, max_num_seqs=1,
                           max_num_batched_tokens=len(prompt), max_model_len=pages * BLOCK_SIZE)  # fmt: skip
    manager32 = CacheManager(runner32.layout.groups, pages, BLOCK_SIZE, 1, False)
    high = logits_of(runner32, manager32)
    torch.cuda.synchronize()
    scale = float(high.abs().max())
    return {
        "tokens": len(prompt),
        "max_abs_err": round(float((low - high).abs().max()), 5),
        "max_abs_logit": round(scale, 4),
        "rel_err": round(float((low - high).abs().max()) / scale, 5),
        "argmax_agree": round(float((low.argmax(-1) == high.argmax(-1)).float().mean()), 4),
        "fp32_seconds": round(time.perf_counter() - began, 1),
    }


REFERENCE_DIR = ROOT / "baseline" / "_ref"


def locate_reference() -> str | None:
    """Puts the reference's package on the path and returns None, or says why it cannot.

    The package is pure Python; its offline ``pip install`` fails only because its build backend
    is not in the image, so ``baseline/_ref/mini_engine`` is an unmodified file copy of its
    ``src/mini_engine`` (made here from ``$MINI_ENGINE_REF`` when the folder is not there yet)."""
    import os
    import shutil

    package = REFERENCE_DIR / "mini_engine"
    if not (package / "engine.py").is_file():
        source = os.environ.get("MINI_ENGINE_REF", "")
        if not (source and (Path(source) / "mini_engine" / "engine.py").is_file()):
            return "no copy of YuvGev00/mini-engine under baseline/_ref and MINI_ENGINE_REF does not name its src folder"
        REFERENCE_DIR.mkdir(parents=True, exist_ok=True)
        shutil.copytree(Path(source) / "mini_engine", package)
    sys.path.insert(0, str(REFERENCE_DIR))
    return None


def run_reference(args) -> dict:
    """The same measurement through YuvGev00/mini-engine's own engine, unmodified.

    Its ``Qwen3ForCausalLM(ModelConfig(...))`` is built from the same numbers with N(0, 0.02)
    weights, wrapped in its ``LLMEngine`` with its stock CUDA options (Triton paged attention,
    captured decode graphs, ``engine.py:59-108``), and driven through ``add_request`` and
    ``step`` (``engine.py:145-196``) only.  Nothing of this repository's package is imported."""
    import types

    why = locate_reference()
    if why:
        return {"impl": "reference", "unavailable": why}
    import torch

    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device in this process"}
    from mini_engine.engine import EngineConfig, LLMEngine
    from mini_engine.model import ModelConfig, Qwen3ForCausalLM
    from mini_engine.sequence import SamplingParams

    sizes = dict(QWEN3_8B)
    full_layers = sizes["num_hidden_layers"]
    if args.layers:
        sizes["num_hidden_layers"] = args.layers
    cfg = types.SimpleNamespace(**sizes)
    layers = cfg.num_hidden_layers
    peaks = load_peaks()
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = Qwen3ForCausalLM(ModelConfig(
            vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
            num_layers=layers, num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta,
            max_position_embeddings=cfg.max_position_embeddings, tie_word_embeddings=cfg.tie_word_embeddings,
        ))  # fmt: skip
    with torch.no_grad():
        for name, parameter in model.named_parameters():
            if parameter.dim() == 2:  # linear and embedding weights; the norms keep their ones
                parameter.normal_(0.0, 0.02)
    model = model.to(dtype=torch.bfloat16)
    generator = torch.Generator().manual_seed(1)

    def random_prompt(n: int) -> list[int]:
        return torch.randint(0, cfg.vocab_size, (n,), generator=generator).tolist()

    def new_engine(batch: int, budget: int, tokens_per_request: int) -> "LLMEngine":
        pages = -(-tokens_per_request // BLOCK_SIZE)
        return LLMEngine(model, EngineConfig(
            block_size=BLOCK_SIZE, num_blocks=batch * pages + 8, max_num_seqs=batch, max_num_batched_tokens=budget,
            max_model_len=MAX_MODEL_LEN, enable_prefix_caching=False, device="cuda", dtype=torch.bfloat16, seed=0,
            cuda_graphs=True,
        ))  # fmt: skip

    def timed(function) -> float:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        function()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end)

    # ------------------------------------------------------------------ prefill: one whole prompt per step
    engine = new_engine(1, PREFILL_TOKENS, PREFILL_TOKENS + 16)
    prefill_times = []
    for i in range(3 + 3):
        engine.add_request(random_prompt(PREFILL_TOKENS), SamplingParams(max_tokens=1, ignore_eos=True))
        torch.cuda.synchronize()
        ms = timed(engine.step)  # the prompt, its one sampled token, finished
        if i >= 3:
            prefill_times.append(ms)
    prefill_ms = statistics.median(prefill_times)
    del engine

    # ------------------------------------------------------------------ decode
    def decode_engine(batch: int, steps_needed: int):
        """An engine whose ``batch`` requests all hold CONTEXT tokens and decode.  Prompts run in
        portions of 512 tokens: its padded prompt attention (``attention.py:128-157``) makes
        scores of batch x longest-portion x context, which a 2,048-token portion beside 63
        decoding requests would not fit."""
        engine = new_engine(batch, 512 if batch > 8 else PREFILL_TOKENS, CONTEXT + steps_needed + batch * 4 + 16)
        params = SamplingParams(max_tokens=min(steps_needed + batch * 4 + 8, MAX_MODEL_LEN - CONTEXT), ignore_eos=True)
        seqs = [engine.add_request(random_prompt(CONTEXT), params) for _ in range(batch)]
        while any(s.num_computed_tokens < s.num_prompt_tokens for s in seqs):
            engine.step()
        return engine

    def time_decode(batch: int, steps: int, warmup: int, repeats: int, e2e: bool):
        engine = decode_engine(batch, warmup + (repeats + int(e2e)) * steps)
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        regions = [timed(lambda: [engine.step() for _ in range(steps)]) / steps for _ in range(repeats)]
        wall = None
        if e2e:
            torch.cuda.synchronize()
            began = time.perf_counter()
            for _ in range(steps):
                engine.step()
            torch.cuda.synchronize()
            wall = time.perf_counter() - began
        return regions, wall, engine

    with ClockSampler() as clocks:
        regions, wall, engine = time_decode(args.batch, args.steps, args.warmup, REPEATS, True)
    clock_summary = clocks.summary()
    e2e_value = args.batch * args.steps / wall
    # what its graph path copies per step (cuda_graphs.py:124-136): int64 ids, positions, slots;
    # context and query lengths; the block-table rows of the batch.  Back: the sampled ids.
    backend, graphs = engine.attention_backend, engine.decode_graphs
    bucket = next(b for b in graphs.buckets if b >= args.batch) if graphs else args.batch
    width = -(-(CONTEXT + args.warmup + (REPEATS + 1) * args.steps) // BLOCK_SIZE)
    h2d_bytes = 8 * (3 * bucket + 2 * bucket + bucket * width)
    d2h_bytes = 8 * args.batch
    decode_path = (
        f"its attention backend {backend!r}, "
        + ("its captured CUDA graph per step" if graphs else "eager launches (it captured no graphs)")
        + ", library matrix products, torch argmax"
    )
    del engine, graphs

    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            try:
                ms = statistics.median(time_decode(batch, max(args.steps // 2, 5), args.warmup, REPEATS, False)[0])
                points[f"decode_b{batch}"] = round(batch / (ms / 1e3), 1)
                points[f"decode_b{batch}_ms"] = round(ms, 4)
            except (RuntimeError, AssertionError) as error:  # e.g. out of memory in its padded attention
                points[f"decode_b{batch}_error"] = str(error).splitlines()[0][:200]
                torch.cuda.empty_cache()

    workloads = None
    if not args.skip_workloads:
        del model
        torch.cuda.empty_cache()
        small = types.SimpleNamespace(**QWEN3_0P6B)
        with torch.device("cuda"):
            small_model = Qwen3ForCausalLM(ModelConfig(
                vocab_size=small.vocab_size, hidden_size=small.hidden_size, intermediate_size=small.intermediate_size,
                num_layers=small.num_hidden_layers, num_heads=small.num_attention_heads,
                num_kv_heads=small.num_key_value_heads, head_dim=small.head_dim, rms_norm_eps=small.rms_norm_eps,
                rope_theta=small.rope_theta, max_position_embeddings=small.max_position_embeddings,
                tie_word_embeddings=small.tie_word_embeddings,
            ))  # fmt: skip
        with torch.no_grad():
            for parameter in small_model.parameters():
                if parameter.dim() == 2:
                    parameter.normal_(0.0, 0.02)
        small_model = small_model.to(dtype=torch.bfloat16)
        try:
            workloads = run_workloads(
                lambda: LLMEngine(small_model, EngineConfig(device="cuda", dtype=torch.bfloat16, enable_prefix_caching=True,
                                                            seed=0, cuda_graphs=True, **WORKLOAD_ENGINE)),
                lambda engine, prompts, n: engine.generate(prompts, SamplingParams(max_tokens=n, ignore_eos=True)),
                torch.cuda.synchronize,
            )  # fmt: skip
        except (RuntimeError, AssertionError) as error:
            workloads = {"error": str(error).splitlines()[0][:200]}
    return result_line(
        "reference", cfg, layers, full_layers, args, peaks, regions, e2e_value, h2d_bytes, d2h_bytes, prefill_ms,
        points, clock_summary, decode_path, **({"workloads": workloads} if workloads else {}),
    )  # fmt: skip


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all)")
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--skip-points", action="store_true", help="do not time batch 1 and 64")
    parser.add_argument("--skip-workloads", action="store_true", help="do not run the two Qwen3-0.6B end-to-end workloads")
    parser.add_argument("--fp32-check", type=int, default=256, metavar="TOKENS",
                        help="also run a prompt of this many tokens through the true 32-bit path of the same model and "
                             "compare the bfloat16 logits with it (0: skip; needs 33 GB more device memory for a second)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        print(json.dumps(run_reference(args)))
        return 0
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
