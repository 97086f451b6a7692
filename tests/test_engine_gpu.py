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


# Largest |engine logit - plain logit| that the replay tests allow, relative to the largest |logit|
# of the request (tests/test_replay_gpu.py); a generated token may therefore lie below the plain
# implementation's best logit by at most twice that.
TOLERANCE = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def plain_weights(folder, dtype):
    weights, cfg = load_plain(folder)
    weights = {k: v.to(torch.float32) for k, v in weights.items()}
    if dtype == torch.bfloat16:
        weights = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in weights.items()}
    return weights, cfg


def assert_follows_plain(folder, dtype, prompts, outputs, temperature=0.0, seed=0, request_ids=None):
    """Teacher-forced check of generated tokens, every one of them: the request's final token ids
    go through the plain implementation once (float64), and at each generated position the
    engine's token must be one that the plain logits allow.  Greedy: its plain logit lies within
    twice the logit tolerance of the best one.  With a temperature: it is the token that the
    plain cumulative distribution gives for the same uniform number, or that number lies so
    close to an edge of the token's interval that the logit tolerance can move the edge past it."""
    from mini_engine_b200.sampling.sampler import uniform_for

    weights, cfg = plain_weights(folder, dtype)
    tolerance = TOLERANCE[dtype]
    checked = 0
    for index, (prompt, out) in enumerate(zip(prompts, outputs)):
        full = list(prompt) + list(out)
        logits = plain.forward_logits(weights, cfg, full[:-1], torch.float64)
        slack = 2 * tolerance * float(logits.abs().max())
        for i, token in enumerate(out):
            row = logits[len(prompt) - 1 + i]
            if temperature == 0:
                gap = float(row.max() - row[token])
                assert gap <= slack, f"request {index} token {i}: engine {token}, plain best {int(row.argmax())}, gap {gap:.4g} > {slack:.4g}"
            else:
                u = uniform_for(seed, request_ids[index], i)
                if plain.sample_from_logits(row, temperature, u) != token:
                    cdf = torch.cumsum(torch.softmax(row / temperature, dim=-1), dim=-1)
                    low = float(cdf[token - 1]) if token > 0 else 0.0
                    high = float(cdf[token])
                    # probabilities move by a factor exp(+-2 slack / T) at most, so an edge by about that much
                    moved = 2.0 * (torch.exp(torch.tensor(slack / temperature)).item() - 1.0) + 1e-5
                    assert low - moved <= u <= high + moved, (
                        f"request {index} token {i}: engine drew {token} at u={u:.6f}, plain interval [{low:.6f}, {high:.6f}]"
                    )
            checked += 1
    assert checked == sum(len(o) for o in outputs)


def assert_same_tokens(got, expected, folder, prompts, min_gap=1e-3):
    """The engine's float32 tokens are the plain implementation's greedy tokens.  Where the plain
    choice was a near-tie the engine may take the other token; from there on the two continuations
    differ, so the rest of that request is checked teacher-forced (every token against the plain
    logits of the engine's own sequence) instead of being left unchecked."""
    for index, (tokens, (want, gaps)) in enumerate(zip(got, expected)):
        assert len(tokens) == len(want)
        for i, (a, b) in enumerate(zip(tokens, want)):
            if a != b:
                assert gaps[i] < min_gap, f"request {index} token {i}: engine {a}, plain {b}, top-2 gap {gaps[i]:.4g}"
                assert_follows_plain(folder, torch.float32, [prompts[index]], [tokens])
                break


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
    assert_same_tokens(got, expected, folder, prompts)
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
    assert_same_tokens([one_by_one.generate([p], params)[0] for p in prompts], expected, folder, prompts)
    assert one_by_one.scheduler.num_cached_tokens == 2 * 24  # the shared prefix was reused twice

    batched = engine_for(folder, "B")
    assert_same_tokens(batched.generate(prompts, params), expected, folder, prompts)

    portions = engine_for(folder, "B", max_num_batched_tokens=32)
    assert_same_tokens(portions.generate(prompts, params), expected, folder, prompts)
    assert portions.stats.steps > batched.stats.steps

    squeezed = engine_for(folder, "B", num_blocks=22, enable_prefix_caching=False)
    assert_same_tokens(squeezed.generate(prompts, params), expected, folder, prompts)
    assert squeezed.scheduler.num_preemptions > 0
    squeezed.block_manager.check_invariants([])

    squeezed_cached = engine_for(folder, "B", num_blocks=22)
    assert_same_tokens(squeezed_cached.generate(prompts, params), expected, folder, prompts)
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


# The paths that steps launched ahead run through: float32 (generic attention) and bfloat16 at head
# sizes 64 and 128, where the decode kernel fetches its first tile of keys and values before it waits
# for the step before it.
OVERLAP_CASES = [("B", torch.float32), ("C", torch.bfloat16), ("D", torch.bfloat16)]
OVERLAP_IDS = ["B-float32", "C-bfloat16", "D-bfloat16"]


@pytest.mark.parametrize("name,dtype", OVERLAP_CASES, ids=OVERLAP_IDS)
def test_steps_launched_ahead_never_change_the_tokens(name, dtype, peaked_model_folders):
    """The decode step after the current one is launched before the current one's tokens are
    read.  When a request then ends on an end-of-sequence token, the step in flight is dropped and
    run again without it: greedy and sampled tokens equal those of an engine whose steps run strictly
    one after the other, for requests that end early, at different times, and for those that go on.
    In bfloat16 the contexts grow across positions 96 and 128, the edges of the decode kernel's
    tiles, so that the tile fetched ahead of the wait holds the key that the step before wrote."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.engine.loading import load_model
    from mini_engine_b200.engine.sequence import Sequence

    folder = peaked_model_folders[name]
    _, cfg = load_plain(folder)
    prompt_lengths = (9, 30, 2, 17, 44) if name == "B" else (90, 120, 2, 125, 44)
    prompts = [random_ids(1200 + i, n, cfg["vocab"]) for i, n in enumerate(prompt_lengths)]
    _arch, _cfg, model = load_model(folder, dtype)
    bitwise_across_batches = dtype == torch.float32  # bfloat16 sums depend on the batch size

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
        options = dict(block_size=PAGE_SIZE[name], num_blocks=64, max_model_len=256, max_num_seqs=8, seed=3, dtype=dtype)
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
            assert not bitwise_across_batches or tokens == free[: len(tokens)]
        # Requests that end at their own max_tokens: known ahead, so the step after goes on without
        # them, launched ahead like any other, and none is dropped.
        lengths = [24, 7, 15, 24, 3]
        engine = LLMEngine(model, EngineConfig(**options), [])
        limited = generate(engine, params, lengths)
        assert [len(tokens) for tokens in limited] == lengths
        for tokens, free in zip(limited, free_run):
            assert not bitwise_across_batches or tokens == free[: len(tokens)]
        assert engine.stats.dropped_steps == 0
        assert engine.stats.prepacked_steps == engine.stats.graph_steps - 1  # all but the first decode step
        engine.block_manager.check_invariants([])


@pytest.mark.parametrize("name,dtype", OVERLAP_CASES, ids=OVERLAP_IDS)
@pytest.mark.parametrize("seed", range(8))
def test_overlapped_steps_with_arrivals_small_pools_and_early_ends(seed, name, dtype, peaked_model_folders):
    """Random workloads (requests that arrive while others decode, pools that force preemption,
    shared prefixes, end-of-sequence tokens, own max_tokens and temperatures): steps launched
    ahead give the tokens of strictly serial steps, and every page comes back."""
    import random

    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.engine.loading import load_model
    from mini_engine_b200.engine.sequence import Sequence

    folder = peaked_model_folders[name]
    _, cfg = load_plain(folder)
    _arch, _cfg, model = load_model(folder, dtype)
    rng = random.Random(seed)
    page, vocab = PAGE_SIZE[name], cfg["vocab"]
    count = rng.randint(3, 10)
    shared_pages = rng.choice([0, 2, 5])
    if page > 8:
        shared_pages = min(shared_pages, 2)  # larger pages: keep prompt + output inside max_model_len
    shared = [rng.randrange(vocab) for _ in range(shared_pages * page)]
    prompts = [shared + [rng.randrange(vocab) for _ in range(rng.randint(1, 50))] for _ in range(count)]
    lengths = [rng.randint(1, 30) for _ in range(count)]
    temperatures = [rng.choice([0.0, 0.0, 0.7, 1.3]) for _ in range(count)]
    arrivals = sorted(rng.randint(0, 12) for _ in range(count))  # the step before which each request is added
    blocks = rng.choice([24, 40]) * 8 // page  # pools of 192 or 320 tokens: some requests get preempted
    eos = [rng.randrange(vocab) for _ in range(rng.choice([0, 3, 40]))]
    options = dict(
        block_size=page, num_blocks=blocks, max_model_len=128 if name == "B" else 160, max_num_seqs=rng.choice([3, 8]),
        max_num_batched_tokens=rng.choice([16, 64, 512]), seed=seed, enable_prefix_caching=rng.random() < 0.7, dtype=dtype,
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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_every_way_of_running_follows_plain(name, dtype, peaked_model_folders):
    """Head sizes 64 and 128 (the tensor-core attention kernels in bfloat16) through the scheduler:
    batched with captured graphs and steps launched ahead, portions under a budget of 32 tokens,
    a pool so small that requests are preempted, and prefix-cache hits.  Every generated token
    of every run is checked against the plain implementation's logits at its position."""
    from mini_engine_b200 import SamplingParams

    folder = peaked_model_folders[name]
    _, cfg = load_plain(folder)
    page = PAGE_SIZE[name]
    shared = random_ids(1600, 3 * page, cfg["vocab"])
    prompts = [shared + random_ids(1601 + i, n, cfg["vocab"]) for i, n in enumerate((6, 30, 46))]
    prompts += [random_ids(1610, 1, cfg["vocab"]), random_ids(1611, 70, cfg["vocab"]), random_ids(1612, 120, cfg["vocab"])]
    params = SamplingParams(max_tokens=14)
    blocks = 2 * sum(-(-(len(p) + 14) // page) for p in prompts)

    batched = engine_for(folder, name, dtype=dtype, num_blocks=blocks)
    assert_follows_plain(folder, dtype, prompts, batched.generate(prompts, params))
    assert batched.stats.graph_steps > 0 and batched.stats.prepacked_steps > 0

    portions = engine_for(folder, name, dtype=dtype, num_blocks=blocks, max_num_batched_tokens=32)
    assert_follows_plain(folder, dtype, prompts, portions.generate(prompts, params))
    assert portions.stats.steps > batched.stats.steps

    # a pool that holds the prompts of the first four requests and one page more: as they decode 40 tokens
    # each they need several pages more, so the ones admitted last are preempted and recomputed
    tight = sum(-(-len(p) // page) for p in prompts[:4]) + 1
    assert tight >= max(-(-(len(p) + 40) // page) for p in prompts)
    long_params = SamplingParams(max_tokens=40)
    squeezed = engine_for(folder, name, dtype=dtype, num_blocks=tight, enable_prefix_caching=False)
    assert_follows_plain(folder, dtype, prompts, squeezed.generate(prompts, long_params))
    assert squeezed.scheduler.num_preemptions > 0
    squeezed.block_manager.check_invariants([])

    one_by_one = engine_for(folder, name, dtype=dtype, num_blocks=blocks)
    outputs = [one_by_one.generate([p], params)[0] for p in prompts]
    assert one_by_one.scheduler.num_cached_tokens == 2 * 3 * page  # the shared prefix was reused twice
    assert_follows_plain(folder, dtype, prompts, outputs)

    squeezed_cached = engine_for(folder, name, dtype=dtype, num_blocks=tight)
    assert_follows_plain(folder, dtype, prompts, squeezed_cached.generate(prompts, long_params))
    assert squeezed_cached.scheduler.num_preemptions > 0
    assert squeezed_cached.block_manager.num_free_blocks == tight


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_temperature_draws_are_the_plain_distributions(name, dtype, model_folders):
    """The token drawn for (seed, request id, token index) is the one that the plain implementation's
    cumulative distribution gives for the same uniform number, through the engine's own sampler
    path (host buffers that alternate, steps launched ahead), batched and under a small budget."""
    from mini_engine_b200 import SamplingParams
    from mini_engine_b200.engine.sequence import Sequence

    folder = model_folders[name]
    _, cfg = load_plain(folder)
    prompts = [random_ids(1700 + i, n, cfg["vocab"]) for i, n in enumerate((12, 40, 3, 77))]
    for temperature, budget in ((0.8, 2048), (1.4, 24)):
        engine = engine_for(folder, name, dtype=dtype, seed=9, max_num_batched_tokens=budget)
        seqs = [Sequence(p, SamplingParams(max_tokens=12, temperature=temperature), seq_id=8800 + i) for i, p in enumerate(prompts)]
        for seq in seqs:
            engine.scheduler.add(seq)
        while engine.scheduler.has_unfinished():
            engine.step()
        outputs = [seq.output_token_ids for seq in seqs]
        assert len({tuple(o) for o in outputs}) == len(outputs)
        assert_follows_plain(folder, dtype, prompts, outputs, temperature, seed=9, request_ids=[s.seq_id for s in seqs])


@pytest.mark.parametrize("name", ["B", "D"])
def test_a_replayed_graph_gives_the_bits_of_the_eager_step(name, model_folders):
    """In float32 the logits of a captured decode graph, padded buckets included (batches of 3 and 5
    run in the buckets of 4 and 8), are bit for bit those of the same entries run eagerly
    (tests/test_gpu.py:46-64 of YuvGev00/mini-engine compares its graphs with its eager step)."""
    from mini_engine_b200.engine.runner import StepEntry

    folder = model_folders[name]
    _, cfg = load_plain(folder)
    engine = engine_for(folder, name, max_num_seqs=8)
    manager, runner, graphs = engine.block_manager, engine.runner, engine.decode_graphs
    lengths = [37, 5, 64, 19, 90, 33, 1, 48]
    caches, prompts = [], []
    for i, n in enumerate(lengths):
        cache = manager.new_request()
        assert manager.try_allocate(cache, n + 4)
        prompts.append(random_ids(1800 + i, n + 3, cfg["vocab"]))
        runner.execute([StepEntry(cache, 0, prompts[-1][:n], ())])
        caches.append(cache)
    for round_number, batch in enumerate((1, 3, 5, 8)):
        assert graphs.bucket_for(batch) in (1, 4, 8)
        chosen = list(range(8))[-batch:] if round_number % 2 else list(range(batch))
        entries = [StepEntry(caches[i], lengths[i], [prompts[i][lengths[i]]], (0,)) for i in chosen]
        eager = runner.execute(entries).clone()
        replayed = graphs.run(entries).clone()  # writes the same keys and values again
        assert replayed.shape == (batch, cfg["vocab"])
        assert torch.equal(eager, replayed), f"batch {batch}: the graph's logits differ from the eager step's"
    for cache in caches:
        manager.free(cache)
    manager.check_invariants([])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_random_weights_in_memory_equal_those_of_a_written_folder(dtype, tmp_path):
    """`LLMEngine.from_random(config, seed)` makes its weights on the device, `write_random_model`
    on the host; both are the same function of (seed, tensor name, element index), so the two
    engines give the same logits bit for bit."""
    from tiny_configs import CONFIGS

    from mini_engine_b200 import EngineConfig, LLMEngine
    from mini_engine_b200.config import Qwen3Config
    from mini_engine_b200.engine.runner import StepEntry
    from mini_engine_b200.weights import write_random_model

    cfg = Qwen3Config.from_dict(CONFIGS["C"])
    options = EngineConfig(block_size=16, num_blocks=16, max_model_len=128, max_num_seqs=2, dtype=dtype, cuda_graphs=False)
    in_memory = LLMEngine.from_random(cfg, seed=21, config=options)
    folder = write_random_model(tmp_path / "m", cfg, seed=21, dtype=torch.bfloat16 if dtype == torch.bfloat16 else torch.float32)
    from_folder = LLMEngine.from_pretrained(folder, options)
    tokens = random_ids(2100, 70, cfg.vocab_size)
    logits = []
    for engine in (in_memory, from_folder):
        cache = engine.block_manager.new_request()
        assert engine.block_manager.try_allocate(cache, len(tokens))
        logits.append(engine.runner.execute([StepEntry(cache, 0, tokens, tuple(range(len(tokens))))]).clone())
    assert torch.equal(logits[0], logits[1])
    assert float(logits[0].abs().max()) > 0


@pytest.mark.parametrize("name", ["B", "D"])
def test_a_short_prompt_alone_replays_a_graph_with_the_eager_bits(name, model_folders):
    """A step that holds one short prompt (or one portion of a longer one) replays a graph of its
    token-count bucket, padded with a dummy entry on the spare page.  In float32 its logits are
    bit for bit those of the eager step, whatever the length, the position it starts at and what
    the graph's buffers held before; a prompt too long for the buckets runs eagerly."""
    from mini_engine_b200.engine.runner import StepEntry

    folder = model_folders[name]
    _, cfg = load_plain(folder)
    engine = engine_for(folder, name, max_model_len=512, num_blocks=96, max_num_batched_tokens=512)
    manager, runner, graphs = engine.block_manager, engine.runner, engine.prompt_graphs
    assert graphs is not None and graphs.buckets == [32, 64, 96, 128]
    assert graphs.bucket_for(1) is None and graphs.bucket_for(31) == 32 and graphs.bucket_for(32) == 64
    assert graphs.bucket_for(100) == 128 and graphs.bucket_for(127) == 128 and graphs.bucket_for(128) is None
    for i, (start, count) in enumerate([(0, 100), (0, 2), (0, 31), (0, 32), (40, 90), (0, 127), (7, 5), (100, 64)]):
        tokens = random_ids(1900 + i, start + count, cfg["vocab"])
        cache = manager.new_request()
        assert manager.try_allocate(cache, start + count)
        if start:
            runner.execute([StepEntry(cache, 0, tokens[:start], ())])
        entry = StepEntry(cache, start, tokens[start:], (count - 1,))
        eager = runner.execute([entry]).clone()
        replayed = graphs.run(entry).clone()  # writes the same keys and values again
        assert torch.equal(eager, replayed), f"start {start}, {count} tokens: the graph's logits differ from the eager step's"
        manager.free(cache)
    assert sorted(graphs.graphs) == [32, 64, 96, 128]
    manager.check_invariants([])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_short_prompts_through_the_engine_use_their_graphs(dtype, peaked_model_folders):
    """Requests that arrive one at a time: each prompt is a step of its own and replays a graph;
    portions under a small budget do too; the tokens follow the plain implementation."""
    from mini_engine_b200 import SamplingParams

    folder = peaked_model_folders["D"]
    _, cfg = load_plain(folder)
    prompts = [random_ids(2000 + i, n, cfg["vocab"]) for i, n in enumerate((17, 90, 2, 140, 33))]
    params = SamplingParams(max_tokens=6)
    engine = engine_for(folder, "D", dtype=dtype, num_blocks=64)
    outputs = [engine.generate([p], params)[0] for p in prompts]
    assert engine.stats.prompt_graph_steps == len(prompts) - 1  # the prompt of 140 tokens runs eagerly
    assert_follows_plain(folder, dtype, prompts, outputs)
    cut = engine_for(folder, "D", dtype=dtype, num_blocks=64, max_num_batched_tokens=48, enable_prefix_caching=False)
    outputs = [cut.generate([p], params)[0] for p in prompts]
    # portions of 48 tokens replay the graph of 64: 17 and 2 whole, 90 as 48 + 42, 140 as 48 + 48 + 44, 33 whole
    assert cut.stats.prompt_graph_steps == 1 + 2 + 1 + 3 + 1
    assert_follows_plain(folder, dtype, prompts, outputs)
    without = engine_for(folder, "D", dtype=dtype, num_blocks=64, cuda_graphs=False)
    assert without.prompt_graphs is None and without.generate([prompts[1]], params)[0] == outputs[1]


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
    assert_same_tokens(engine.generate(prompts, SamplingParams(max_tokens=4)), plain_greedy(folder, prompts, 4), folder, prompts)


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


def test_requests_arriving_over_time_on_a_layer_of_real_sizes(tmp_path_factory):
    """One layer of Qwen3-8B's own sizes through the whole engine in bfloat16: requests arrive while
    others run, some share a prefix, some are short enough to replay a prompt graph when they are
    alone in a step, the longest are cut by the token budget into portions of several hundred
    tokens (the CTA-pair products and the tensor-core attention), and the pool is so small that
    requests are preempted.  Every generated token is checked teacher-forced against the plain
    implementation."""
    import random

    from conftest import make_model_folder
    from tiny_configs import LAYER_OF_8B

    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.csrc import ops

    folder = make_model_folder(tmp_path_factory, "8B_engine", seed=17, dtype=torch.bfloat16, raw=LAYER_OF_8B)
    vocab = LAYER_OF_8B["vocab_size"]
    rng = random.Random(5)
    shared = random_ids(40, 200, vocab)
    prompts, limits = [], []
    for i in range(14):
        kind = i % 3
        if i == 0:
            prompt = random_ids(50, 50, vocab)  # alone in the first step: a prompt graph
        elif kind == 0:
            prompt = shared[: rng.choice([64, 160])] + random_ids(50 + i, rng.randrange(1, 30), vocab)
        elif kind == 1:
            prompt = random_ids(70 + i, rng.randrange(2, 100), vocab)
        else:
            prompt = random_ids(90 + i, rng.randrange(300, 420), vocab)
        prompts.append(prompt)
        limits.append(rng.randrange(1, 24))
    engine = LLMEngine.from_pretrained(
        folder,
        EngineConfig(block_size=16, num_blocks=40, max_num_seqs=6, max_num_batched_tokens=384, max_model_len=512, dtype=torch.bfloat16),
    )  # fmt: skip
    pending = list(zip(prompts, limits))
    seqs = [engine.add_request(pending[0][0], SamplingParams(max_tokens=pending[0][1], ignore_eos=True))]
    pending.pop(0)
    engine.step()
    assert engine.stats.prompt_graph_steps == 1
    while pending or engine.scheduler.has_unfinished():
        if not engine.scheduler.has_unfinished() or rng.random() < 0.3:
            for _ in range(rng.randrange(1, 4)):
                if pending:
                    prompt, limit = pending.pop(0)
                    seqs.append(engine.add_request(prompt, SamplingParams(max_tokens=limit, ignore_eos=True)))
        engine.step()
    ops.raise_on_device_error()
    engine.block_manager.check_invariants([])
    outputs = [s.output_token_ids for s in seqs]
    assert [len(o) for o in outputs] == limits
    assert engine.scheduler.num_preemptions > 0 and engine.scheduler.num_cached_tokens > 0
    assert engine.stats.prompt_graph_steps > 0 and engine.stats.prepacked_steps > 0 and engine.stats.graph_steps > 0
    assert_follows_plain(folder, torch.bfloat16, prompts, outputs)


def test_step_costs_reports_every_class(capsys):
    """The in-place cost tool captures the decode step with each class of launches left out and
    puts the kernels back when it is done."""
    import json

    from mini_engine_b200.cli import step_costs
    from mini_engine_b200.csrc import ops

    before = (ops.add_rmsnorm, ops.qk_norm_rope_store, ops.paged_attention)
    assert step_costs.main(["--size", "0.6b", "--layers", "2", "--batch", "3", "--context", "64", "--steps", "3"]) == 0
    assert (ops.add_rmsnorm, ops.qk_norm_rope_store, ops.paged_attention) == before
    rows = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert [r["left_out"] for r in rows] == [None, "norms", "norm_rotation_cache_write", "decode_attention", "all_but_products"]
    whole = rows[0]["launches"]
    assert [whole - r["launches"] for r in rows] == [0, 5, 2, 2, 9]  # two layers: 2 x 2 + 1 norms, 2 rotations, 2 attentions
