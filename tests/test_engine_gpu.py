"""Generation through the Python entry point against the plain implementation."""

from __future__ import annotations

import pytest
import torch

import plain_qwen3 as plain
from conftest import load_plain
from tiny_configs import PAGE_SIZE, random_ids

pytestmark = pytest.mark.gpu


def engine_for(folder, name, dtype=torch.float32, **overrides):
    from mini_engine_b200 import EngineConfig, LLMEngine

    options = dict(block_size=PAGE_SIZE[name], num_blocks=64, max_model_len=256, max_num_seqs=8, dtype=dtype)
    options.update(overrides)
    return LLMEngine.from_pretrained(folder, EngineConfig(**options))


def plain_greedy(folder, prompts, steps):
    weights, cfg = load_plain(folder)
    return [plain.greedy_generate(weights, cfg, p, steps) for p in prompts]


def assert_same_tokens(got, expected, min_gap=1e-3):
    """Tokens must be equal wherever the plain implementation's choice was not a near-tie."""
    for tokens, (want, gaps) in zip(got, expected):
        for i, (a, b) in enumerate(zip(tokens, want)):
            if a != b:
                assert gaps[i] < min_gap, f"token {i}: engine {a}, plain {b}, top-2 gap {gaps[i]:.4g}"
                break  # after a legitimate near-tie flip the continuations differ
        assert len(tokens) == len(want)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_matches_plain(name, graphs, peaked_model_folders):
    from mini_engine_b200 import SamplingParams

    folder = peaked_model_folders[name]
    _, cfg = load_plain(folder)
    lengths = (5, 17, 33) if name == "A" else (1, 24, 70, 9, 40)
    prompts = [random_ids(500 + i, n, cfg["vocab"]) for i, n in enumerate(lengths)]
    expected = plain_greedy(folder, prompts, 8)
    engine = engine_for(folder, name, cuda_graphs=graphs)
    got = engine.generate(prompts, SamplingParams(max_tokens=8))
    assert_same_tokens(got, expected)
    assert engine.block_manager.num_free_blocks == 64
    engine.block_manager.check_invariants([])
    if graphs:
        assert engine.stats.graph_steps > 0
        assert 0 < engine.stats.prepacked_steps < engine.stats.graph_steps  # laid out while the step before ran


def test_every_way_of_running_gives_the_same_tokens(peaked_model_folders):
    """Unbatched, batched, portions under a small token budget, preemption under a small pool
    and prefix-cache hits all give the tokens of the plain implementation
    (tests/test_parity.py:80-119 of YuvGev00/mini-engine)."""
    from mini_engine_b200 import SamplingParams

    folder = peaked_model_folders["B"]
    _, cfg = load_plain(folder)
    shared = random_ids(600, 24, cfg["vocab"])
    prompts = [shared + random_ids(601 + i, n, cfg["vocab"]) for i, n in enumerate((6, 30, 46))]
    prompts += [random_ids(610, 1, cfg["vocab"]), random_ids(611, 70, cfg["vocab"])]
    params = SamplingParams(max_tokens=12)
    expected = plain_greedy(folder, prompts, 12)

    one_by_one = engine_for(folder, "B")
    assert_same_tokens([one_by_one.generate([p], params)[0] for p in prompts], expected)
    assert one_by_one.scheduler.num_cached_tokens == 2 * 24  # the shared prefix was reused twice

    batched = engine_for(folder, "B")
    assert_same_tokens(batched.generate(prompts, params), expected)

    portions = engine_for(folder, "B", max_num_batched_tokens=32)
    assert_same_tokens(portions.generate(prompts, params), expected)
    assert portions.stats.steps > batched.stats.steps

    squeezed = engine_for(folder, "B", num_blocks=22, enable_prefix_caching=False)
    assert_same_tokens(squeezed.generate(prompts, params), expected)
    assert squeezed.scheduler.num_preemptions > 0
    squeezed.block_manager.check_invariants([])

    squeezed_cached = engine_for(folder, "B", num_blocks=22)
    assert_same_tokens(squeezed_cached.generate(prompts, params), expected)
    assert squeezed_cached.scheduler.num_preemptions > 0


def test_temperature_sampling_is_reproducible_and_batch_independent(model_folders):
    from mini_engine_b200 import SamplingParams

    folder = model_folders["B"]
    _, cfg = load_plain(folder)
    prompts = [random_ids(700 + i, n, cfg["vocab"]) for i, n in enumerate((12, 40, 3))]
    params = SamplingParams(max_tokens=10, temperature=0.8)
    first = engine_for(folder, "B", seed=5)
    seqs = [first.add_request(p, params) for p in prompts]
    while first.scheduler.has_unfinished():
        first.step()
    ids = [s.seq_id for s in seqs]
    batched = [s.output_token_ids for s in seqs]
    assert len({tuple(t) for t in batched}) > 1
    # the same requests (same ids, same seed) run one at a time sample the same tokens
    from mini_engine_b200.engine.sequence import Sequence

    alone_engine = engine_for(folder, "B", seed=5)
    alone = []
    for prompt, seq_id in zip(prompts, ids):
        seq = Sequence(prompt, params, seq_id=seq_id)
        alone_engine.scheduler.add(seq)
        while alone_engine.scheduler.has_unfinished():
            alone_engine.step()
        alone.append(seq.output_token_ids)
    assert alone == batched
    other_seed = engine_for(folder, "B", seed=6)
    seqs2 = [Sequence(p, params, seq_id=i) for p, i in zip(prompts, ids)]
    for s in seqs2:
        other_seed.scheduler.add(s)
    while other_seed.scheduler.has_unfinished():
        other_seed.step()
    assert [s.output_token_ids for s in seqs2] != batched


def test_steps_launched_ahead_never_change_the_tokens(peaked_model_folders):
    """The decode step after the current one is launched before the current one's tokens are
    read.  When a request then ends on an end-of-sequence token, the step in flight is dropped and
    run again without it: greedy and sampled tokens equal those of an engine whose steps run strictly
    one after the other, for requests that end early, at different times, and for those that go on."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.engine.loading import load_model
    from mini_engine_b200.engine.sequence import Sequence

    folder = peaked_model_folders["B"]
    _, cfg = load_plain(folder)
    prompts = [random_ids(1200 + i, n, cfg["vocab"]) for i, n in enumerate((9, 30, 2, 17, 44))]
    _arch, _cfg, model = load_model(folder, torch.float32)

    def generate(engine, params, lengths=None):  # the same request ids in every run: sampled tokens depend on them
        seqs = []
        for i, prompt in enumerate(prompts):
            mine = params if lengths is None else SamplingParams(max_tokens=lengths[i], temperature=params.temperature)
            seqs.append(Sequence(prompt, mine, seq_id=7000 + i))
            engine.scheduler.add(seqs[-1])
        while engine.scheduler.has_unfinished():
            engine.step()
        return [seq.output_token_ids for seq in seqs]

    for temperature in (0.0, 0.9):
        params = SamplingParams(max_tokens=24, temperature=temperature)
        options = dict(block_size=PAGE_SIZE["B"], num_blocks=64, max_model_len=256, max_num_seqs=8, seed=3)
        free_run = generate(LLMEngine(model, EngineConfig(**options), []), params)
        # tokens that end some requests early and at different steps, and leave others running
        eos = [free_run[0][5], free_run[1][11], free_run[3][2]]
        runs = {}
        for overlap in (False, True):
            engine = LLMEngine(model, EngineConfig(overlap_steps=overlap, **options), eos)
            runs[overlap] = generate(engine, params)
            engine.block_manager.check_invariants([])
            assert engine.block_manager.num_free_blocks == 64
            if overlap:
                assert engine.stats.prepacked_steps > 0 and engine.stats.dropped_steps > 0
            else:
                assert engine.stats.prepacked_steps == 0 and engine.stats.dropped_steps == 0
        assert runs[True] == runs[False]
        assert any(len(tokens) < 24 for tokens in runs[True]) and any(len(tokens) == 24 for tokens in runs[True])
        for tokens, free in zip(runs[True], free_run):
            assert tokens == free[: len(tokens)]
        # Requests that end at their own max_tokens: known ahead, so the step after goes on without
        # them, launched ahead like any other, and none is dropped.
        lengths = [24, 7, 15, 24, 3]
        engine = LLMEngine(model, EngineConfig(**options), [])
        limited = generate(engine, params, lengths)
        assert [len(tokens) for tokens in limited] == lengths
        for tokens, free in zip(limited, free_run):
            assert tokens == free[: len(tokens)]
        assert engine.stats.dropped_steps == 0
        assert engine.stats.prepacked_steps == engine.stats.graph_steps - 1  # all but the first decode step
        engine.block_manager.check_invariants([])


@pytest.mark.parametrize("seed", range(8))
def test_overlapped_steps_with_arrivals_small_pools_and_early_ends(seed, peaked_model_folders):
    """Random workloads (requests that arrive while others decode, pools that force preemption,
    shared prefixes, end-of-sequence tokens, own max_tokens and temperatures): steps launched
    ahead give the tokens of strictly serial steps, and every page comes back."""
    import random

    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.engine.loading import load_model
    from mini_engine_b200.engine.sequence import Sequence

    folder = peaked_model_folders["B"]
    _, cfg = load_plain(folder)
    _arch, _cfg, model = load_model(folder, torch.float32)
    rng = random.Random(seed)
    page, vocab = PAGE_SIZE["B"], cfg["vocab"]
    count = rng.randint(3, 10)
    shared = [rng.randrange(vocab) for _ in range(rng.choice([0, 2 * page, 5 * page]))]
    prompts = [shared + [rng.randrange(vocab) for _ in range(rng.randint(1, 50))] for _ in range(count)]
    lengths = [rng.randint(1, 30) for _ in range(count)]
    temperatures = [rng.choice([0.0, 0.0, 0.7, 1.3]) for _ in range(count)]
    arrivals = sorted(rng.randint(0, 12) for _ in range(count))  # the step before which each request is added
    blocks = rng.choice([24, 40])
    eos = [rng.randrange(vocab) for _ in range(rng.choice([0, 3, 40]))]
    options = dict(
        block_size=page, num_blocks=blocks, max_model_len=128, max_num_seqs=rng.choice([3, 8]),
        max_num_batched_tokens=rng.choice([16, 64, 512]), seed=seed, enable_prefix_caching=rng.random() < 0.7,
    )  # fmt: skip
    runs = {}
    for overlap in (False, True):
        engine = LLMEngine(model, EngineConfig(overlap_steps=overlap, **options), eos)
        seqs = [
            Sequence(p, SamplingParams(max_tokens=m, temperature=t), seq_id=9000 + i)
            for i, (p, m, t) in enumerate(zip(prompts, lengths, temperatures))
        ]
        step = added = 0
        while added < count or engine.scheduler.has_unfinished():
            while added < count and arrivals[added] <= step:
                engine.scheduler.add(seqs[added])
                added += 1
            if engine.scheduler.has_unfinished():
                engine.step()
            step += 1
        engine.block_manager.check_invariants([])
        assert engine.block_manager.num_free_blocks == blocks
        runs[overlap] = [seq.output_token_ids for seq in seqs]
    assert runs[True] == runs[False]


def test_eos_stops_generation_and_is_kept(peaked_model_folders):
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.engine.loading import load_model

    folder = peaked_model_folders["A"]
    _, cfg = load_plain(folder)
    prompt = random_ids(800, 20, cfg["vocab"])
    free_run = engine_for(folder, "A").generate([prompt], SamplingParams(max_tokens=10))[0]
    eos = free_run[4]
    _arch, _cfg, model = load_model(folder, torch.float32)
    config = EngineConfig(block_size=16, num_blocks=64, max_model_len=256, max_num_seqs=8)
    stopped = LLMEngine(model, config, [eos]).generate([prompt], SamplingParams(max_tokens=10))[0]
    assert stopped == free_run[: free_run.index(eos) + 1]
    ignoring = LLMEngine(model, config, [eos]).generate([prompt], SamplingParams(max_tokens=10, ignore_eos=True))[0]
    assert ignoring == free_run


def test_bfloat16_generation_runs_and_mostly_agrees(peaked_model_folders):
    """bfloat16 is compared by tolerance on logits elsewhere; here generation must run through
    graphs and portions and agree with float32 on peaked logits up to near-ties."""
    from mini_engine_b200 import SamplingParams

    folder = peaked_model_folders["B"]
    _, cfg = load_plain(folder)
    prompts = [random_ids(900 + i, n, cfg["vocab"]) for i, n in enumerate((8, 33, 64))]
    params = SamplingParams(max_tokens=6)
    reference = engine_for(folder, "B").generate(prompts, params)
    got = engine_for(folder, "B", dtype=torch.bfloat16, max_num_batched_tokens=40).generate(prompts, params)
    agree = sum(a == b for x, y in zip(got, reference) for a, b in zip(x[:1], y[:1]))
    assert agree >= 2  # the first generated token of at least two of three requests


def test_command_line(peaked_model_folders):
    import subprocess
    import sys

    from conftest import ROOT

    folder = peaked_model_folders["A"]
    proc = subprocess.run(
        [sys.executable, str(ROOT / "examples" / "generate.py"), "--model", str(folder), "--dtype", "fp32",
         "--max-tokens", "5", "--block-size", "16", "--num-blocks", "32", "--max-model-len", "256"],
        capture_output=True, text=True, timeout=600,
    )  # fmt: skip
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = proc.stdout.strip().splitlines()
    assert len(lines) == 4 and lines[-1].startswith("15 tokens in")
    assert "served from prefix cache 128" in lines[-1]  # two later requests reuse four pages each
    refused = subprocess.run(
        [sys.executable, str(ROOT / "examples" / "generate.py"), "--model", str(folder), "--device", "cpu"],
        capture_output=True, text=True, timeout=600,
    )  # fmt: skip
    assert refused.returncode == 2 and "CUDA only" in refused.stderr


def test_pool_sized_from_free_memory(peaked_model_folders):
    """``kv_memory_fraction`` replaces ``num_blocks``: the pool takes that share of what is free."""
    from mini_engine_b200 import SamplingParams
    from mini_engine_b200.engine.llm_engine import kv_cache_bytes_per_token

    folder = peaked_model_folders["A"]
    free_before, _ = torch.cuda.mem_get_info()
    engine = engine_for(folder, "A", num_blocks=3, kv_memory_fraction=0.001)
    blocks = engine.config.num_blocks
    page_bytes = kv_cache_bytes_per_token(engine.runner) * PAGE_SIZE["A"]
    assert blocks == engine.block_manager.num_free_blocks != 3
    assert 0.5 * 0.001 * free_before <= (blocks + 1) * page_bytes <= 0.001 * free_before
    _, cfg = load_plain(folder)
    prompts = [random_ids(900, 21, cfg["vocab"])]
    assert_same_tokens(engine.generate(prompts, SamplingParams(max_tokens=4)), plain_greedy(folder, prompts, 4))


def test_engine_profiler_reports_phases(capsys):
    """The phase profiler runs the engine's own step both ways and prints one JSON line each."""
    import json

    from mini_engine_b200.cli import profile_engine

    assert profile_engine.main(["--steps", "4", "--requests", "3", "--prompt-len", "20", "--num-blocks", "64"]) == 0
    rows = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert len(rows) == 2
    running, isolated = rows
    assert running["steps_launched_ahead"] > 0 and isolated["steps_launched_ahead"] == 0
    assert running["kernel_launches_per_step"] > 100  # 28 layers of eight kernels and more
    assert "wait for the token ids" in running["phases_us_per_step"]
    assert "lay out + H2D + graph launch" in isolated["phases_us_per_step"]
