"""Each part of a layer alone against the plain implementation, at sizes of its own; models
whose order repeats a layer, reads another entry's cache or uses a window; and a toy mixer
with state of its own that is registered, built and stepped from here without touching the
framework's files; likewise a toy position encoding and a toy routed feed-forward."""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------ a small harness


def make_runner(spec, dtype=torch.float32, page=4, pages=64, seed=0, scale=5.0):
    """A model of `spec` with seeded random weights, its runner and a cache manager."""
    from mini_engine_b200.cache import CacheManager
    from mini_engine_b200.engine.runner import ModelRunner
    from mini_engine_b200.parts.model import DecoderModel
    from mini_engine_b200.weights.loader import place_tensors
    from mini_engine_b200.weights.random_init import random_tensors

    model = DecoderModel(spec)
    specs = model.weight_specs()
    host = random_tensors(specs, seed, torch.float32, scale=scale)
    model.load(place_tensors(dict(host), specs, dtype, "cuda"))
    runner = ModelRunner(model, dtype=dtype, num_blocks=pages, block_size=page, max_num_seqs=4,
                         max_num_batched_tokens=256, max_model_len=pages * page)  # fmt: skip
    manager = CacheManager(runner.layout.groups, pages, page, 4, False, slot_groups=runner.layout.slot_groups)
    return model, runner, manager, host


def one_layer_spec(hidden, heads, kv_heads, head_dim, inter, vocab=50, window=None, theta=777.0, eps=2e-5, layers=1,
                   order=None):
    from mini_engine_b200.config.model_spec import LayerSpec, ModelSpec, OrderEntry, PartSpec

    rope = PartSpec("rope", {"head_dim": head_dim, "theta": theta})
    layer_specs = tuple(
        LayerSpec(
            prefix=f"model.layers.{i}.",
            block="prenorm",
            mixer=PartSpec("gqa_attention", {
                "num_heads": heads, "kv_heads": kv_heads, "head_dim": head_dim, "qk_norm_eps": eps,
                "position_encoding": rope, "window": window,
                "names": {k: f"self_attn.{k}_proj.weight" for k in "qkvo"} | {
                    "q_norm": "self_attn.q_norm.weight", "k_norm": "self_attn.k_norm.weight"},
            }),
            feed_forward=PartSpec("gated_mlp", {"intermediate_size": inter, "names": {
                "gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight"}}),
            mixer_norm=PartSpec("rmsnorm", {"name": "input_layernorm.weight", "eps": eps}),
            feed_forward_norm=PartSpec("rmsnorm", {"name": "post_attention_layernorm.weight", "eps": eps}),
        )
        for i in range(layers)
    )  # fmt: skip
    return ModelSpec(
        vocab_size=vocab, hidden_size=hidden,
        embedding=PartSpec("token_embedding", {"weight": "model.embed_tokens.weight"}),
        layers=layer_specs, order=tuple(order or [OrderEntry(i) for i in range(layers)]),
        final_norm=PartSpec("rmsnorm", {"name": "model.norm.weight", "eps": eps}),
        head=PartSpec("linear_head", {"weight": "lm_head.weight", "tied_to": None}),
    )  # fmt: skip


def plain_cfg(hidden, heads, kv_heads, head_dim, inter, vocab=50, window=None, theta=777.0, eps=2e-5, layers=1):
    return {"vocab": vocab, "hidden": hidden, "inter": inter, "layers": layers, "heads": heads, "kv_heads": kv_heads,
            "head_dim": head_dim, "eps": eps, "theta": theta, "tied": False, "window": window}  # fmt: skip


def context_for(runner, manager, lengths):
    from mini_engine_b200.engine.runner import StepEntry

    entries = []
    for n in lengths:
        cache = manager.new_request()
        assert manager.try_allocate(cache, n)
        entries.append(StepEntry(cache, 0, [1] * n, ()))
    ctx, _ = runner.pack(entries)
    return ctx


SIZES = dict(hidden=48, heads=6, kv_heads=2, head_dim=16, inter=72)


# ----------------------------------------------------------------------- parts alone


def test_rmsnorm_part_alone():
    from mini_engine_b200.parts.base import Residual

    model, runner, manager, host = make_runner(one_layer_spec(**SIZES))
    norm = model.blocks[0].mixer_norm
    ctx = context_for(runner, manager, [5, 3])
    torch.manual_seed(0)
    x, delta = torch.randn(8, 48, device="cuda"), torch.randn(2, 8, 48, device="cuda")
    state = Residual(x.clone(), delta)
    out = norm.forward(state, ctx, torch.float32)
    summed = x + delta.sum(0)
    want = plain.rms_norm(summed.cpu(), host["model.layers.0.input_layernorm.weight"], 2e-5)
    assert state.pending is None and torch.allclose(state.x, summed, atol=1e-6)
    assert torch.allclose(out.cpu(), want, atol=1e-5, rtol=1e-5)


def test_rotary_part_alone():
    from mini_engine_b200.parts.rotary import RotaryEncoding

    part = RotaryEncoding("", 0, head_dim=48, theta=12345.0)
    want = 1.0 / (12345.0 ** (torch.arange(0, 48, 2, dtype=torch.float32) / 48))
    assert torch.equal(part.fused_rotary_table().cpu(), want)


@pytest.mark.parametrize("window", [None, 5])
def test_attention_mixer_alone(window):
    model, runner, manager, host = make_runner(one_layer_spec(**SIZES, window=window))
    mixer = model.blocks[0].mixer
    lengths = [13, 1, 7]
    ctx = context_for(runner, manager, lengths)
    torch.manual_seed(1)
    h = torch.randn(sum(lengths), 48, device="cuda")
    out = mixer.forward(h, ctx, runner.layout.views[0]).sum(0).cpu()
    cfg = plain_cfg(**SIZES, window=window)
    start = 0
    for n in lengths:
        want = plain.attention_block(h[start : start + n].cpu(), host, "model.layers.0.self_attn.", cfg, torch.arange(n))
        assert torch.allclose(out[start : start + n], want, atol=2e-5, rtol=1e-4)
        start += n


@pytest.mark.parametrize("head_dim,rotary_dim", [(16, 8), (128, 64), (48, 48)])
def test_attention_mixer_with_a_partial_rotation(head_dim, rotary_dim):
    """`rope` with `rotary_dim` < head_dim rotates the first rotary_dim elements of every head (in two
    halves of rotary_dim / 2) and passes the rest through, inside the same fused kernel (norm,
    rotation, cache write); a spec switches it on.  Whole == cut bitwise, equal to a plain restatement."""
    from mini_engine_b200.config.model_spec import LayerSpec, PartSpec

    sizes = dict(hidden=48, heads=4, kv_heads=2, head_dim=head_dim, inter=72)
    base = one_layer_spec(**sizes)
    layer = base.layers[0]
    rope = PartSpec("rope", {"head_dim": head_dim, "theta": 777.0, "rotary_dim": rotary_dim})
    mixer = PartSpec(layer.mixer.kind, {**layer.mixer.params, "position_encoding": rope})
    spec = type(base)(**{**base.__dict__, "layers": (type(layer)(**{**layer.__dict__, "mixer": mixer}),)})
    model, runner, manager, host = make_runner(spec)
    tokens = [3, 14, 15, 9, 2, 6, 5, 35, 8, 9, 7, 9, 3]
    whole, cut = run_whole_and_cut(runner, manager, tokens)
    assert torch.equal(whole, cut)

    cfg = plain_cfg(**sizes)
    t, eps = len(tokens), cfg["eps"]
    positions = torch.arange(t)
    p = "model.layers.0."
    x = host["model.embed_tokens.weight"][torch.tensor(tokens)]
    h = plain.rms_norm(x, host[p + "input_layernorm.weight"], eps)
    q = plain.rms_norm((h @ host[p + "self_attn.q_proj.weight"].T).view(t, 4, head_dim), host[p + "self_attn.q_norm.weight"], eps)
    k = plain.rms_norm((h @ host[p + "self_attn.k_proj.weight"].T).view(t, 2, head_dim), host[p + "self_attn.k_norm.weight"], eps)
    v = (h @ host[p + "self_attn.v_proj.weight"].T).view(t, 2, head_dim)
    cos, sin = plain.rope_angles(positions, rotary_dim, 777.0, torch.float32)

    def partly_rotated(z):
        return torch.cat((plain.apply_rope(z[..., :rotary_dim], cos, sin), z[..., rotary_dim:]), dim=-1)

    attended = plain.causal_attention(partly_rotated(q), partly_rotated(k), v)
    x = x + attended.reshape(t, -1) @ host[p + "self_attn.o_proj.weight"].T
    x = x + plain.swiglu_mlp(plain.rms_norm(x, host[p + "post_attention_layernorm.weight"], eps), host, p + "mlp.")
    want = plain.rms_norm(x, host["model.norm.weight"], eps) @ host["lm_head.weight"].T
    assert torch.allclose(whole, want, atol=3e-5, rtol=1e-4)
    if rotary_dim < head_dim:  # and the rotation of only a part is not the rotation of the whole
        full = plain.rope_angles(positions, head_dim, 777.0, torch.float32)
        assert not torch.allclose(partly_rotated(q), plain.apply_rope(q, *full), atol=1e-3)


@pytest.mark.parametrize("head_dim,qk_norm", [(16, False), (128, False), (128, True)])
def test_attention_mixer_with_projection_biases(head_dim, qk_norm):
    """`qkv_bias` adds a bias to the q, k and v projections (and `qk_norm_eps=None` drops the per-head
    norms): the attention of models that have biases instead of q/k norms, by spec alone.  The bias
    is added inside the fused kernel, to the sum of the product's partial sums."""
    from mini_engine_b200.config.model_spec import PartSpec

    sizes = dict(hidden=48, heads=4, kv_heads=2, head_dim=head_dim, inter=72)
    base = one_layer_spec(**sizes)
    layer = base.layers[0]
    names = {**layer.mixer.params["names"], "q_bias": "self_attn.q_proj.bias", "k_bias": "self_attn.k_proj.bias",
             "v_bias": "self_attn.v_proj.bias"}  # fmt: skip
    params = {**layer.mixer.params, "qkv_bias": True, "names": names}
    if not qk_norm:
        params["qk_norm_eps"] = None
    spec = type(base)(**{**base.__dict__, "layers": (type(layer)(**{**layer.__dict__, "mixer": PartSpec(layer.mixer.kind, params)}),)})
    model, runner, manager, host = make_runner(spec)
    p = "model.layers.0."
    assert (p + "self_attn.q_norm.weight" in host) == qk_norm and host[p + "self_attn.k_proj.bias"].shape == (2 * head_dim,)
    tokens = [3, 14, 15, 9, 2, 6, 5, 35, 8, 9, 7, 9, 3]
    whole, cut = run_whole_and_cut(runner, manager, tokens)
    assert torch.equal(whole, cut)

    cfg = plain_cfg(**sizes)
    t, eps = len(tokens), cfg["eps"]
    x = host["model.embed_tokens.weight"][torch.tensor(tokens)]
    h = plain.rms_norm(x, host[p + "input_layernorm.weight"], eps)
    q = (h @ host[p + "self_attn.q_proj.weight"].T + host[p + "self_attn.q_proj.bias"]).view(t, 4, head_dim)
    k = (h @ host[p + "self_attn.k_proj.weight"].T + host[p + "self_attn.k_proj.bias"]).view(t, 2, head_dim)
    v = (h @ host[p + "self_attn.v_proj.weight"].T + host[p + "self_attn.v_proj.bias"]).view(t, 2, head_dim)
    if qk_norm:
        q = plain.rms_norm(q, host[p + "self_attn.q_norm.weight"], eps)
        k = plain.rms_norm(k, host[p + "self_attn.k_norm.weight"], eps)
    cos, sin = plain.rope_angles(torch.arange(t), head_dim, 777.0, torch.float32)
    attended = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v)
    x = x + attended.reshape(t, -1) @ host[p + "self_attn.o_proj.weight"].T
    x = x + plain.swiglu_mlp(plain.rms_norm(x, host[p + "post_attention_layernorm.weight"], eps), host, p + "mlp.")
    want = plain.rms_norm(x, host["model.norm.weight"], eps) @ host["lm_head.weight"].T
    assert torch.allclose(whole, want, atol=3e-5, rtol=1e-4)
    assert float(host[p + "self_attn.v_proj.bias"].abs().max()) > 0.01  # the biases are not negligible


def test_feed_forward_alone():
    model, runner, manager, host = make_runner(one_layer_spec(**SIZES))
    ctx = context_for(runner, manager, [9])
    torch.manual_seed(2)
    h = torch.randn(9, 48, device="cuda")
    out = model.blocks[0].feed_forward.forward(h, ctx).sum(0).cpu()
    want = plain.swiglu_mlp(h.cpu(), host, "model.layers.0.mlp.")
    assert torch.allclose(out, want, atol=2e-5, rtol=1e-4)


def test_block_alone():
    from mini_engine_b200.parts.base import Residual

    model, runner, manager, host = make_runner(one_layer_spec(**SIZES))
    ctx = context_for(runner, manager, [11])
    torch.manual_seed(3)
    x = torch.randn(11, 48, device="cuda")
    state = Residual(x.clone())
    model.blocks[0].forward(state, ctx, runner.layout.views[0])
    got = (state.x + state.pending.sum(0)).cpu()
    want = plain.decoder_layer(x.cpu(), host, 0, plain_cfg(**SIZES), torch.arange(11))
    assert torch.allclose(got, want, atol=3e-5, rtol=1e-4)


# ------------------------------------------------- order as data: repeats, shared caches


def run_whole_and_cut(runner, manager, tokens):
    """Logits of a request run whole and run in portions of 5, 1, 1, 4, ... tokens."""
    from mini_engine_b200.engine.runner import StepEntry

    cache = manager.new_request()
    assert manager.try_allocate(cache, len(tokens))
    whole = runner.execute([StepEntry(cache, 0, tokens, tuple(range(len(tokens))))]).cpu().clone()
    manager.free(cache)
    cache = manager.new_request()
    rows, done = [], 0
    for size in [5, 1, 1, 4, 2, 100]:
        chunk = tokens[done : done + size]
        if not chunk:
            break
        assert manager.try_allocate(cache, done + len(chunk))
        rows.append(runner.execute([StepEntry(cache, done, chunk, tuple(range(len(chunk))))]).cpu().clone())
        done += len(chunk)
        manager.release_behind_window(cache, done)
    manager.free(cache)
    return whole, torch.cat(rows)


def test_a_layer_twice_and_a_layer_reading_anothers_cache():
    """order = [0, 1, 0 (reading entry 0's cache), 1]: weights of a layer are shared by its two
    executions; the third entry attends over the keys that the first one wrote."""
    from mini_engine_b200.config.model_spec import LayerSpec, OrderEntry, PartSpec

    base = one_layer_spec(**SIZES, layers=2)
    order = (OrderEntry(0), OrderEntry(1), OrderEntry(0, cache_of=0), OrderEntry(1))
    spec = type(base)(**{**base.__dict__, "order": order})
    model, runner, manager, host = make_runner(spec)
    assert len(runner.layout.views) == 4 and runner.layout.views[2].k.data_ptr() == runner.layout.views[0].k.data_ptr()
    assert runner.layout.views[3].k.data_ptr() != runner.layout.views[1].k.data_ptr()
    tokens = [3, 14, 15, 9, 2, 6, 5, 35, 8, 9, 7, 9, 3]
    whole, cut = run_whole_and_cut(runner, manager, tokens)
    assert torch.equal(whole, cut)  # float32: cutting changes nothing

    # plain restatement of the same order
    cfg = plain_cfg(**SIZES, layers=2)
    w = host
    ids, pos = torch.tensor(tokens), torch.arange(len(tokens))
    x = w["model.embed_tokens.weight"][ids]

    def attention(x_in, layer, keys_from=None):
        p = f"model.layers.{layer}.self_attn."
        t, d = x_in.shape[0], cfg["head_dim"]
        source = x_in if keys_from is None else keys_from
        q = plain.rms_norm((x_in @ w[p + "q_proj.weight"].T).view(t, cfg["heads"], d), w[p + "q_norm.weight"], cfg["eps"])
        k = plain.rms_norm((source @ w[p + "k_proj.weight"].T).view(t, cfg["kv_heads"], d), w[p + "k_norm.weight"], cfg["eps"])
        v = (source @ w[p + "v_proj.weight"].T).view(t, cfg["kv_heads"], d)
        cos, sin = plain.rope_angles(pos, d, cfg["theta"], torch.float32)
        out = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v)
        return out.reshape(t, -1) @ w[p + "o_proj.weight"].T

    normed_first = None
    for position, entry in enumerate(order):
        p = f"model.layers.{entry.layer}."
        normed = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        if position == 0:
            normed_first = normed
        # the entry that reads entry 0's cache sees the keys and values entry 0 computed
        x = x + attention(normed, entry.layer, normed_first if entry.cache_of == 0 else None)
        x = x + plain.swiglu_mlp(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"]), w, p + "mlp.")
    want = plain.rms_norm(x, w["model.norm.weight"], cfg["eps"]) @ w["lm_head.weight"].T
    assert torch.allclose(whole, want, atol=1e-4, rtol=1e-4)


def test_layers_with_and_without_a_window_get_groups_of_their_own():
    from mini_engine_b200.config.model_spec import PartSpec

    base = one_layer_spec(**SIZES, layers=2)
    windowed = base.layers[1]
    mixer = PartSpec(windowed.mixer.kind, {**windowed.mixer.params, "window": 6})
    layers = (base.layers[0], type(windowed)(**{**windowed.__dict__, "mixer": mixer}))
    spec = type(base)(**{**base.__dict__, "layers": layers})
    model, runner, manager, host = make_runner(spec, page=4)
    assert len(runner.layout.groups) == 2 and [g.window for g in runner.layout.groups] == [None, 6]
    tokens = list(range(1, 30))
    whole, cut = run_whole_and_cut(runner, manager, tokens)
    assert torch.equal(whole, cut)
    manager.check_invariants([])
    # plain: layer 0 full, layer 1 with the window
    cfg0, cfg1 = plain_cfg(**SIZES, layers=2), plain_cfg(**SIZES, layers=2, window=6)
    x = host["model.embed_tokens.weight"][torch.tensor(tokens)]
    x = plain.decoder_layer(x, host, 0, cfg0, torch.arange(len(tokens)))
    x = plain.decoder_layer(x, host, 1, cfg1, torch.arange(len(tokens)))
    want = plain.rms_norm(x, host["model.norm.weight"], cfg0["eps"]) @ host["lm_head.weight"].T
    assert torch.allclose(whole, want, atol=1e-4, rtol=1e-4)


def test_prefix_hits_with_a_windowed_layer_through_the_engine():
    """A model whose second layer reads only the last 6 keys, through the scheduler with prefix
    reuse on: requests that share a prompt prefix skip it (the window group supplies the pages its
    window reaches, its table starts with pages that were never taken), the window group's own pool
    is far smaller than the other's, and the tokens equal those of an engine without prefix reuse
    and the plain implementation's."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.config.model_spec import PartSpec
    from mini_engine_b200.parts.model import DecoderModel
    from mini_engine_b200.weights.loader import place_tensors
    from mini_engine_b200.weights.random_init import random_tensors

    base = one_layer_spec(**SIZES, layers=2)
    windowed = base.layers[1]
    mixer = PartSpec(windowed.mixer.kind, {**windowed.mixer.params, "window": 6})
    spec = type(base)(**{**base.__dict__, "layers": (base.layers[0], type(windowed)(**{**windowed.__dict__, "mixer": mixer}))})
    model = DecoderModel(spec)
    host = random_tensors(model.weight_specs(), 3, torch.float32, scale=5.0)
    model.load(place_tensors(dict(host), model.weight_specs(), torch.float32, "cuda"))
    shared = [7, 3, 9, 1, 4, 4, 8, 2, 6, 5, 11, 13, 12, 10, 15, 14, 17, 19, 21, 23]  # five pages of four
    prompts = [shared + tail for tail in ([30, 31], [32], [33, 34, 35, 36, 37], [38, 39, 40])]
    options = dict(block_size=4, num_blocks=48, max_model_len=64, max_num_seqs=2, max_num_batched_tokens=16)
    runs = {}
    for reuse in (False, True):
        engine = LLMEngine(model, EngineConfig(enable_prefix_caching=reuse, **options), [])
        groups = engine.runner.layout.groups
        assert [g.window for g in groups] == [None, 6]
        # window 6 + a step of 16 tokens: 6 pages and two for the edges, for each of two requests
        assert groups[0].num_blocks == 48 and groups[1].num_blocks == 2 * (-(-(6 + 16) // 4) + 2)
        runs[reuse] = [engine.generate([p], SamplingParams(max_tokens=6))[0] for p in prompts]
        engine.block_manager.check_invariants([])
        assert [pool.num_free for pool in engine.block_manager.pools] == [g.num_blocks for g in groups]
        if reuse:
            assert engine.scheduler.num_cached_tokens == 3 * 20  # every later request found the five shared pages
        else:
            assert engine.scheduler.num_cached_tokens == 0
    assert runs[True] == runs[False]
    cfg0, cfg1 = plain_cfg(**SIZES, layers=2), plain_cfg(**SIZES, layers=2, window=6)
    for prompt, out in zip(prompts, runs[True]):
        ids = list(prompt)
        for token in out:
            x = host["model.embed_tokens.weight"][torch.tensor(ids)]
            x = plain.decoder_layer(x, host, 0, cfg0, torch.arange(len(ids)))
            x = plain.decoder_layer(x, host, 1, cfg1, torch.arange(len(ids)))
            logits = plain.rms_norm(x[-1:], host["model.norm.weight"], cfg0["eps"]) @ host["lm_head.weight"].T
            top = torch.topk(logits[0], 2).values
            assert int(logits[0].argmax()) == token or float(top[0] - logits[0][token]) < 1e-3
            ids.append(token)


# --------------------------------------------------- a toy mixer with state of its own


def register_toy():
    """A mixer that keeps a decaying sum of its inputs per request: s_t = a * s_{t-1} + h_t,
    y_t = s_t W^T.  It owns no pages, only a state slot.  Everything is defined here."""
    from mini_engine_b200.config import Architecture, register_architecture
    from mini_engine_b200.config.model_spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
    from mini_engine_b200.parts.base import MIXERS, Mixer, StateSpec, register
    from mini_engine_b200.weights.loader import WeightSpec

    if "toy_decay" not in MIXERS:

        @register("mixer", "toy_decay")
        class ToyDecay(Mixer):
            def __init__(self, prefix, hidden_size, *, decay):
                self.name, self.hidden, self.decay = prefix + "toy.weight", hidden_size, decay
                self.weight = None

            def state(self):
                return StateSpec((self.hidden,), torch.float32)

            def weight_specs(self):
                return [WeightSpec(self.name, (self.hidden, self.hidden))]

            def load(self, tensors):
                self.weight = tensors[self.name].float()

            def forward(self, h, ctx, cache):
                if ctx.all_decode:
                    # One token per entry: everything stays on the device (slots and fresh flags are
                    # read there), so that a captured decode graph replays it for other requests.
                    slots = ctx.state_slots.long()
                    state = cache.state[slots] * (1.0 - ctx.fresh.float())[:, None]
                    state = state * self.decay + h.float()
                    cache.state.index_copy_(0, slots, state)
                    return (state @ self.weight.T).unsqueeze(0)
                out = torch.empty(1, h.shape[0], self.hidden, device=h.device)
                row = 0
                for count, start, slot in zip(ctx.host["counts"], ctx.host["starts"], ctx.host["state_slots"]):
                    state = cache.state[slot]
                    if start == 0:
                        state.zero_()
                    for _ in range(count):
                        state.mul_(self.decay).add_(h[row].float())
                        out[0, row] = state @ self.weight.T
                        row += 1
                return out

    @dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        hidden_size: int
        intermediate_size: int
        decay: float
        eps: float
        architecture = "ToyDecayLM"

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                    "intermediate_size": self.intermediate_size, "decay": self.decay, "eps": self.eps}  # fmt: skip

        @classmethod
        def from_folder(cls, folder):
            raw = json.loads((Path(folder) / "config.json").read_text())
            return cls(raw["vocab_size"], raw["hidden_size"], raw["intermediate_size"], raw["decay"], raw["eps"])

    def spec(cfg):
        layer = LayerSpec(
            prefix="layers.0.", block="prenorm", mixer=PartSpec("toy_decay", {"decay": cfg.decay}),
            feed_forward=PartSpec("gated_mlp", {"intermediate_size": cfg.intermediate_size}),
            mixer_norm=PartSpec("rmsnorm", {"name": "norm1.weight", "eps": cfg.eps}),
            feed_forward_norm=PartSpec("rmsnorm", {"name": "norm2.weight", "eps": cfg.eps}),
        )  # fmt: skip
        return ModelSpec(
            vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
            embedding=PartSpec("token_embedding", {"weight": "embed.weight"}), layers=(layer,),
            order=(OrderEntry(0), OrderEntry(0)),  # the same layer twice: two states
            final_norm=PartSpec("rmsnorm", {"name": "final.weight", "eps": cfg.eps}),
            head=PartSpec("linear_head", {"weight": "head.weight", "tied_to": "embed.weight"}),
        )  # fmt: skip

    register_architecture(Architecture("ToyDecayLM", ToyConfig.from_folder, spec, ToyConfig), replace=True)
    return ToyConfig


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from safetensors.torch import load_file

    from mini_engine_b200.engine.replay import Replayer
    from mini_engine_b200.weights import write_random_model

    ToyConfig = register_toy()
    cfg = ToyConfig(vocab_size=40, hidden_size=24, intermediate_size=32, decay=0.7, eps=1e-5)
    folder = write_random_model(tmp_path / "toy", cfg, seed=5, dtype=torch.float32, scale=8.0)
    replayer = Replayer(folder, torch.float32, max_tokens=128, block_size=16)
    assert replayer.runner.layout.has_state and replayer.runner.layout.groups == []
    assert not replayer.manager.enable_prefix_caching  # state cannot be shared through page hashes

    a, b = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5], [8, 9, 7, 9, 3, 2]
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:4], "want": [0, 1, 2, 3]}]},
        {"step": 1, "entries": [{"id": "a", "tokens": a[4:5], "want": [0]}, {"id": "b", "tokens": b[:3], "want": [0, 1, 2]}]},
        {"step": 2, "entries": [{"id": "b", "tokens": b[3:], "want": [0, 1, 2]}, {"id": "a", "tokens": a[5:], "want": list(range(6))}], "end": ["a", "b"]},
        {"step": 3, "entries": [{"id": "c", "tokens": b, "want": list(range(6))}], "end": ["c"]},  # reuses a slot
    ]  # fmt: skip
    got = {s["step"]: replayer.step(s) for s in steps}
    replayer.manager.check_invariants([])

    w = load_file(str(folder / "model.safetensors"))

    def plain_toy(tokens):
        x = w["embed.weight"][torch.tensor(tokens)]
        for _ in range(2):
            normed = plain.rms_norm(x, w["layers.0.norm1.weight"], cfg.eps)
            state, rows = torch.zeros(cfg.hidden_size), []
            for t in range(len(tokens)):
                state = cfg.decay * state + normed[t]
                rows.append(state @ w["layers.0.toy.weight"].T)
            x = x + torch.stack(rows)
            x = x + plain.swiglu_mlp(plain.rms_norm(x, w["layers.0.norm2.weight"], cfg.eps), w, "layers.0.")
        return plain.rms_norm(x, w["final.weight"], cfg.eps) @ w["embed.weight"].T

    want_a, want_b = plain_toy(a), plain_toy(b)
    assert torch.allclose(got[0], want_a[:4], atol=1e-4, rtol=1e-4)
    assert torch.allclose(got[1], torch.cat([want_a[4:5], want_b[:3]]), atol=1e-4, rtol=1e-4)
    assert torch.allclose(got[2], torch.cat([want_b[3:], want_a[5:]]), atol=1e-4, rtol=1e-4)
    assert torch.allclose(got[3], want_b, atol=1e-4, rtol=1e-4)


# ------------------------------ a toy position encoding and a toy routed feed-forward


def test_toy_mixer_with_state_runs_through_the_engine_without_steps_launched_ahead(tmp_path):
    """A step that was launched ahead and then dropped is run again, which would advance a mixer's
    own state twice; so for a model with such a mixer the scheduler plans no step ahead.  Requests
    that end early on an end-of-sequence token (the case that drops steps) give the same tokens
    with `overlap_steps` on and off, equal to the whole-sequence restatement of the toy model."""
    from safetensors.torch import load_file

    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.weights import write_random_model

    ToyConfig = register_toy()
    cfg = ToyConfig(vocab_size=40, hidden_size=24, intermediate_size=32, decay=0.7, eps=1e-5)
    folder = write_random_model(tmp_path / "toy", cfg, seed=6, dtype=torch.float32, scale=8.0)
    w = load_file(str(folder / "model.safetensors"))

    def plain_next(tokens):
        x = w["embed.weight"][torch.tensor(tokens)]
        for _ in range(2):
            normed = plain.rms_norm(x, w["layers.0.norm1.weight"], cfg.eps)
            state, rows = torch.zeros(cfg.hidden_size), []
            for row in normed:
                state = state * cfg.decay + row
                rows.append(state @ w["layers.0.toy.weight"].T)
            x = x + torch.stack(rows)
            x = x + plain.swiglu_mlp(plain.rms_norm(x, w["layers.0.norm2.weight"], cfg.eps), w, "layers.0.")
        logits = plain.rms_norm(x, w["final.weight"], cfg.eps) @ w["embed.weight"].T
        return int(logits[-1].argmax())

    prompts = [[3, 1, 4, 1, 5], [9, 2, 6], [5, 3, 5, 8, 9, 7, 9]]
    options = dict(block_size=16, num_blocks=16, max_model_len=64, max_num_seqs=4)
    free_run = LLMEngine.from_pretrained(folder, EngineConfig(**options)).generate(prompts, SamplingParams(max_tokens=10))
    for prompt, out in zip(prompts, free_run):
        ids = list(prompt)
        for token in out:
            assert plain_next(ids) == token
            ids.append(token)
    eos = {free_run[0][3], free_run[2][6]}
    runs = {}
    for overlap in (False, True):
        engine = LLMEngine.from_pretrained(folder, EngineConfig(overlap_steps=overlap, **options))
        engine.scheduler.eos_token_ids = set(eos)
        runs[overlap] = engine.generate(prompts, SamplingParams(max_tokens=10))
        assert engine.stats.graph_steps > 0  # decode steps replay graphs, with the state slots in them
        assert engine.stats.prepacked_steps == 0 and engine.stats.dropped_steps == 0
        engine.block_manager.check_invariants([])
    assert runs[True] == runs[False]
    assert any(len(out) < 10 for out in runs[True])
    for out, free in zip(runs[True], free_run):
        assert out == free[: len(out)]


def test_toy_position_encoding_is_registered_and_applied():
    """A position encoding that is no rotation (queries grow and keys shrink with the position, so
    their product falls with the distance), defined here: the attention mixer then runs its
    norm, the encoding's own `apply` and the cache write as three steps."""
    from mini_engine_b200.config.model_spec import PartSpec
    from mini_engine_b200.parts.base import POSITION_ENCODINGS, PositionEncoding, register

    if "toy_distance_decay" not in POSITION_ENCODINGS:

        @register("position_encoding", "toy_distance_decay")
        class ToyDistanceDecay(PositionEncoding):
            def __init__(self, prefix, hidden_size, *, head_dim, rate):
                self.rates = rate * torch.arange(1, head_dim + 1, dtype=torch.float32, device="cuda") / head_dim

            def apply(self, q, k, positions):
                grow = torch.exp(positions.float()[:, None, None] * self.rates)
                q.copy_((q.float() * grow).to(q.dtype))
                k.copy_((k.float() / grow).to(k.dtype))

    base = one_layer_spec(**SIZES)
    layer = base.layers[0]
    params = {**layer.mixer.params, "position_encoding": PartSpec("toy_distance_decay", {"head_dim": 16, "rate": 0.05})}
    spec = type(base)(**{**base.__dict__, "layers": (type(layer)(**{**layer.__dict__, "mixer": PartSpec(layer.mixer.kind, params)}),)})
    model, runner, manager, host = make_runner(spec)
    tokens = [7, 3, 9, 1, 4, 4, 8, 2, 6, 5, 10, 12, 11, 3]
    whole, cut = run_whole_and_cut(runner, manager, tokens)
    assert torch.equal(whole, cut)

    cfg, w, p = plain_cfg(**SIZES), host, "model.layers.0."
    t, d, pos = len(tokens), cfg["head_dim"], torch.arange(len(tokens), dtype=torch.float32)
    x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    normed = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
    q = plain.rms_norm((normed @ w[p + "self_attn.q_proj.weight"].T).view(t, cfg["heads"], d), w[p + "self_attn.q_norm.weight"], cfg["eps"])
    k = plain.rms_norm((normed @ w[p + "self_attn.k_proj.weight"].T).view(t, cfg["kv_heads"], d), w[p + "self_attn.k_norm.weight"], cfg["eps"])
    v = (normed @ w[p + "self_attn.v_proj.weight"].T).view(t, cfg["kv_heads"], d)
    grow = torch.exp(pos[:, None, None] * (0.05 * torch.arange(1, d + 1, dtype=torch.float32) / d))
    x = x + plain.causal_attention(q * grow, k / grow, v).reshape(t, -1) @ w[p + "self_attn.o_proj.weight"].T
    x = x + plain.swiglu_mlp(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"]), w, p + "mlp.")
    want = plain.rms_norm(x, w["model.norm.weight"], cfg["eps"]) @ w["lm_head.weight"].T
    assert torch.allclose(whole, want, atol=1e-4, rtol=1e-4)


def test_toy_routed_feed_forward_is_registered_and_stepped():
    """A feed-forward with routing, defined here: each token goes to the one of three small
    experts whose router logit (32-bit, per token) is largest."""
    from mini_engine_b200.config.model_spec import PartSpec
    from mini_engine_b200.parts.base import FEED_FORWARDS, FeedForward, register
    from mini_engine_b200.weights.loader import WeightSpec

    if "toy_top1_experts" not in FEED_FORWARDS:

        @register("feed_forward", "toy_top1_experts")
        class ToyTop1Experts(FeedForward):
            def __init__(self, prefix, hidden_size, *, experts, width):
                self.prefix, self.hidden, self.experts, self.width = prefix + "moe.", hidden_size, experts, width

            def weight_specs(self):
                specs = [WeightSpec(self.prefix + "router.weight", (self.experts, self.hidden))]
                for e in range(self.experts):
                    specs.append(WeightSpec(f"{self.prefix}{e}.in.weight", (self.width, self.hidden)))
                    specs.append(WeightSpec(f"{self.prefix}{e}.out.weight", (self.hidden, self.width)))
                return specs

            def load(self, tensors):
                self.w = {spec.name: tensors[spec.name].float() for spec in self.weight_specs()}

            def forward(self, h, ctx):
                # token by token, so that a token's result cannot depend on what else is in the
                # batch (a library product over all rows may add in another order for another
                # number of rows)
                x = h.float()
                out = torch.zeros(1, x.shape[0], self.hidden, device=x.device)
                for i in range(x.shape[0]):
                    e = int((self.w[self.prefix + "router.weight"] @ x[i]).argmax())
                    hidden = torch.relu(self.w[f"{self.prefix}{e}.in.weight"] @ x[i])
                    out[0, i] = self.w[f"{self.prefix}{e}.out.weight"] @ hidden
                return out

    base = one_layer_spec(**SIZES, layers=2)
    routed = PartSpec("toy_top1_experts", {"experts": 3, "width": 20})
    second = base.layers[1]
    layers = (base.layers[0], type(second)(**{**second.__dict__, "feed_forward": routed}))  # dense, then routed
    spec = type(base)(**{**base.__dict__, "layers": layers})
    model, runner, manager, host = make_runner(spec)
    tokens = [5, 40, 13, 2, 2, 31, 8, 19, 44, 6, 27, 3, 9, 9, 1]
    whole, cut = run_whole_and_cut(runner, manager, tokens)
    assert torch.equal(whole, cut)

    cfg, w = plain_cfg(**SIZES, layers=2), host
    x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    x = plain.decoder_layer(x, w, 0, cfg, torch.arange(len(tokens)))
    p = "model.layers.1."
    normed = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
    x = x + plain.attention_block(normed, w, p + "self_attn.", cfg, torch.arange(len(tokens)))
    normed = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
    choice = (normed @ w[p + "moe.router.weight"].T).argmax(-1)
    assert len(set(choice.tolist())) > 1, "the test wants tokens on different experts"
    routed_out = torch.stack([
        torch.relu(normed[i] @ w[f"{p}moe.{int(e)}.in.weight"].T) @ w[f"{p}moe.{int(e)}.out.weight"].T
        for i, e in enumerate(choice)
    ])  # fmt: skip
    x = x + routed_out
    want = plain.rms_norm(x, w["model.norm.weight"], cfg["eps"]) @ w["lm_head.weight"].T
    assert torch.allclose(whole, want, atol=1e-4, rtol=1e-4)


# ------------------------------------------- the model's two ends and blocks with more norms


def test_embedding_multiplier_and_a_head_with_bias_scale_and_cap():
    """An embedding multiplier, a head bias, a logit scale and a soft cap are options of the two
    end parts: a spec switches them on, nothing else changes.  Whole == cut, and equal to the plain
    model with the same four changes restated here."""
    from mini_engine_b200.config.model_spec import PartSpec

    base = one_layer_spec(**SIZES, layers=2)
    spec = type(base)(**{
        **base.__dict__,
        "embedding": PartSpec("token_embedding", {"weight": "model.embed_tokens.weight", "multiplier": 48**0.5}),
        "head": PartSpec("linear_head", {"weight": "lm_head.weight", "tied_to": "model.embed_tokens.weight",
                                         "bias": "lm_head.bias", "logit_scale": 1.5, "soft_cap": 3.0}),
    })  # fmt: skip
    model, runner, manager, host = make_runner(spec, scale=2.0)
    assert "lm_head.bias" in host and "lm_head.weight" not in host  # tied: one tensor; the bias is the head's own
    tokens = [3, 14, 15, 9, 2, 6, 5, 35, 8, 9, 7, 9, 3]
    whole, cut = run_whole_and_cut(runner, manager, tokens)
    assert torch.equal(whole, cut)
    cfg = plain_cfg(**SIZES, layers=2)
    x = host["model.embed_tokens.weight"][torch.tensor(tokens)] * 48**0.5
    for index in range(2):
        x = plain.decoder_layer(x, host, index, cfg, torch.arange(len(tokens)))
    x = plain.rms_norm(x, host["model.norm.weight"], cfg["eps"])
    logits = (x @ host["model.embed_tokens.weight"].T) * 1.5 + host["lm_head.bias"]
    want = 3.0 * torch.tanh(logits / 3.0)
    assert float(logits.abs().max()) > 2.5 and float((logits - want).abs().max()) > 0.3  # the cap bends the largest logits
    assert torch.allclose(whole, want, atol=3e-5, rtol=1e-4)


def test_a_block_with_four_norms_is_registered_from_here():
    """A post-norm arrangement (a norm in front of and behind both the mixer and the feed-forward,
    four per layer) is a block class that names its norms; the layer's spec gives them by name.
    Nothing of the framework changes.  The block adds the normed outputs into the stream itself."""
    from mini_engine_b200.config.model_spec import LayerSpec, PartSpec
    from mini_engine_b200.parts.base import BLOCKS, Block, Residual, register

    if "toy_sandwich" not in BLOCKS:

        @register("block", "toy_sandwich")
        class SandwichBlock(Block):
            """``h = x + post_m(mixer(pre_m(x)))``, ``y = h + post_f(ff(pre_f(h)))``."""

            NORMS = ("mixer", "after_mixer", "feed_forward", "after_feed_forward")

            def _after(self, name, out, state, ctx):
                # normalise the part's output on its own (an all-zero stream plus the pending slices), then
                # hand the normed rows to the residual stream as its next pending addend
                normed = self.norms[name].forward(Residual(torch.zeros_like(state.x), out), ctx, torch.float32)
                state.add(normed.clone())

            def forward(self, state, ctx, cache):
                h = self.norms["mixer"].forward(state, ctx, ctx.dtype)
                self._after("after_mixer", self.mixer.forward(h, ctx, cache), state, ctx)
                h = self.norms["feed_forward"].forward(state, ctx, ctx.dtype)
                self._after("after_feed_forward", self.feed_forward.forward(h, ctx), state, ctx)

    base = one_layer_spec(**SIZES, layers=2)
    eps = 2e-5
    layers = tuple(
        LayerSpec(
            prefix=layer.prefix, block="toy_sandwich", mixer=layer.mixer, feed_forward=layer.feed_forward,
            norms={
                "mixer": layer.mixer_norm,
                "after_mixer": PartSpec("rmsnorm", {"name": "post_mixer_norm.weight", "eps": eps}),
                "feed_forward": layer.feed_forward_norm,
                "after_feed_forward": PartSpec("rmsnorm", {"name": "post_ff_norm.weight", "eps": eps}),
            },
        )
        for layer in base.layers
    )  # fmt: skip
    spec = type(base)(**{**base.__dict__, "layers": layers})
    model, runner, manager, host = make_runner(spec, scale=3.0)
    assert "model.layers.1.post_ff_norm.weight" in host and len(model.blocks[0].norms) == 4
    tokens = [3, 14, 15, 9, 2, 6, 5, 35, 8, 9, 7, 9, 3]
    whole, cut = run_whole_and_cut(runner, manager, tokens)
    assert torch.equal(whole, cut)
    cfg = plain_cfg(**SIZES, layers=2)
    positions = torch.arange(len(tokens))
    x = host["model.embed_tokens.weight"][torch.tensor(tokens)]
    for index in range(2):
        p = f"model.layers.{index}."
        a = plain.attention_block(plain.rms_norm(x, host[p + "input_layernorm.weight"], eps), host, p + "self_attn.", cfg, positions)
        x = x + plain.rms_norm(a, host[p + "post_mixer_norm.weight"], eps)
        f = plain.swiglu_mlp(plain.rms_norm(x, host[p + "post_attention_layernorm.weight"], eps), host, p + "mlp.")
        x = x + plain.rms_norm(f, host[p + "post_ff_norm.weight"], eps)
    want = plain.rms_norm(x, host["model.norm.weight"], eps) @ host["lm_head.weight"].T
    assert torch.allclose(whole, want, atol=3e-5, rtol=1e-4)
    # a layer that names the wrong norms is refused when the model is built
    wrong = type(base)(**{**base.__dict__, "layers": tuple(
        LayerSpec(prefix=l.prefix, block="toy_sandwich", mixer=l.mixer, feed_forward=l.feed_forward,
                  mixer_norm=l.mixer_norm, feed_forward_norm=l.feed_forward_norm) for l in base.layers)})  # fmt: skip
    from mini_engine_b200.parts.model import DecoderModel

    with pytest.raises(ValueError, match="wants the norms"):
        DecoderModel(wrong)
