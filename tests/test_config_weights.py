"""Configuration, registry and weight loading (no GPU)."""

from __future__ import annotations

import json

import pytest
import torch

from tiny_configs import CONFIGS, write_config


def test_qwen3_config_reads_its_own_keys(tmp_path):
    from mini_engine_b200.config import Qwen3Config, load_model_config

    write_config(tmp_path, CONFIGS["B"])
    arch, cfg = load_model_config(tmp_path)
    assert arch.name == "Qwen3ForCausalLM" and isinstance(cfg, Qwen3Config)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 8, 2)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (32, 160, 384)
    assert cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5 and not cfg.tie_word_embeddings
    assert Qwen3Config.from_dict(cfg.to_dict()) == cfg


def test_config_defaults_and_eos(tmp_path):
    from mini_engine_b200.config import Qwen3Config

    raw = dict(CONFIGS["A"], eos_token_id=[7, 9])
    del raw["head_dim"], raw["rope_theta"]
    write_config(tmp_path, raw)
    cfg = Qwen3Config.from_folder(tmp_path)
    assert cfg.head_dim == 16 and cfg.rope_theta == 10000.0 and cfg.eos_token_ids == (7, 9)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 3}))
    assert Qwen3Config.from_folder(tmp_path).eos_token_ids == (3,)


@pytest.mark.parametrize(
    "change,word",
    [
        ({"model_type": "llama"}, "model_type"),
        ({"rope_parameters": {"rope_type": "yarn", "rope_theta": 1e4}}, "RoPE"),
        ({"use_sliding_window": True}, "sliding"),
        ({"attention_bias": True}, "attention_bias"),
        ({"hidden_act": "gelu"}, "hidden_act"),
        ({"num_key_value_heads": 3}, "multiple"),
        ({"rms_norm_eps": None}, "rms_norm_eps"),
        ({"head_dim": 15}, "even"),
    ],
)
def test_config_rejections(change, word):
    from mini_engine_b200.config import Qwen3Config
    from mini_engine_b200.config.qwen3 import ConfigError

    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(dict(CONFIGS["A"], **change))


def test_registry_names_what_is_registered(tmp_path):
    from mini_engine_b200.config import load_model_config, registered_architectures

    assert "Qwen3ForCausalLM" in registered_architectures()
    write_config(tmp_path, dict(CONFIGS["A"], architectures=["NoSuchModel"]))
    with pytest.raises(KeyError, match="Qwen3ForCausalLM"):
        load_model_config(tmp_path)


def test_spec_is_data_and_sizes_come_from_the_config():
    from mini_engine_b200.config import Qwen3Config, architecture_for
    from mini_engine_b200.parts.model import declared_weights

    for name in ("A", "B"):
        cfg = Qwen3Config.from_dict(CONFIGS[name])
        spec = architecture_for("Qwen3ForCausalLM").build_spec(cfg)
        assert len(spec.layers) == cfg.num_hidden_layers and [e.layer for e in spec.order] == list(range(len(spec.layers)))
        shapes = {w.name: w.shape for w in declared_weights(spec)}
        d = cfg.head_dim
        assert shapes["model.layers.0.self_attn.q_proj.weight"] == (cfg.num_attention_heads * d, cfg.hidden_size)
        assert shapes["model.layers.0.self_attn.k_proj.weight"] == (cfg.num_key_value_heads * d, cfg.hidden_size)
        assert shapes["model.layers.0.mlp.down_proj.weight"] == (cfg.hidden_size, cfg.intermediate_size)
        assert shapes["model.layers.0.self_attn.q_norm.weight"] == (d,)
        assert len(shapes) == 11 * cfg.num_hidden_layers + 3


def test_order_validation():
    from mini_engine_b200.config import Qwen3Config, architecture_for
    from mini_engine_b200.config.model_spec import ModelSpec, OrderEntry

    spec = architecture_for("Qwen3ForCausalLM").build_spec(Qwen3Config.from_dict(CONFIGS["A"]))
    fields = {k: getattr(spec, k) for k in ("vocab_size", "hidden_size", "embedding", "layers", "final_norm", "head")}
    ModelSpec(order=(OrderEntry(0), OrderEntry(1), OrderEntry(1), OrderEntry(0, cache_of=0)), **fields)
    with pytest.raises(ValueError, match="does not exist"):
        ModelSpec(order=(OrderEntry(5),), **fields)
    with pytest.raises(ValueError, match="earlier"):
        ModelSpec(order=(OrderEntry(0, cache_of=1), OrderEntry(1)), **fields)


def test_safetensors_round_trip(tmp_path):
    from safetensors.torch import load_file, save_file

    from mini_engine_b200.weights import SafetensorsFile, write_safetensors

    tensors = {
        "a": torch.randn(3, 5),
        "b": torch.randn(7).to(torch.bfloat16),
        "c": torch.arange(6, dtype=torch.int32).view(2, 3),
        "empty": torch.zeros(0, 4),
    }
    write_safetensors(tmp_path / "ours.safetensors", tensors)
    theirs = load_file(str(tmp_path / "ours.safetensors"))  # the library reads what we write
    save_file(tensors, str(tmp_path / "theirs.safetensors"))
    ours = SafetensorsFile(tmp_path / "theirs.safetensors")  # and we read what it writes
    for name, t in tensors.items():
        assert torch.equal(theirs[name], t) and torch.equal(ours.tensor(name), t)


def test_random_weights_depend_on_name_and_seed_only(tmp_path):
    from mini_engine_b200.config import Qwen3Config
    from mini_engine_b200.weights import read_folder_index, write_random_model

    cfg = Qwen3Config.from_dict(CONFIGS["A"])
    one = read_folder_index(write_random_model(tmp_path / "one", cfg, 3, torch.float32))
    two = read_folder_index(write_random_model(tmp_path / "two", cfg, 3, torch.float32))
    other = read_folder_index(write_random_model(tmp_path / "other", cfg, 4, torch.float32))
    assert "lm_head.weight" not in one  # tied: one tensor
    name = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(one[name].tensor(name), two[name].tensor(name))
    assert not torch.equal(one[name].tensor(name), other[name].tensor(name))
    w = one[name].tensor(name)
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    norm = one["model.norm.weight"].tensor("model.norm.weight")
    assert abs(float(norm.mean()) - 1.0) < 0.05
    assert (tmp_path / "one" / "config.json").is_file()


def test_weight_errors_are_listed_in_one_message(tmp_path):
    from safetensors.torch import load_file, save_file

    from mini_engine_b200.config import Qwen3Config, architecture_for
    from mini_engine_b200.parts.model import declared_weights
    from mini_engine_b200.weights import WeightError, load_weights, write_random_model

    cfg = Qwen3Config.from_dict(CONFIGS["B"])
    folder = write_random_model(tmp_path / "m", cfg, 0, torch.float32)
    specs = declared_weights(architecture_for(cfg.architecture).build_spec(cfg))
    assert len(load_weights(folder, specs, torch.float32, "cpu")) == len(specs)
    state = load_file(str(folder / "model.safetensors"))
    del state["model.layers.2.mlp.up_proj.weight"], state["model.norm.weight"]
    state["model.layers.9.extra.weight"] = torch.zeros(2)
    state["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(5, 5)
    state["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)  # derived buffer: ignored
    save_file(state, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as raised:
        load_weights(folder, specs, torch.float32, "cpu")
    error = raised.value
    assert error.missing == ["model.layers.2.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["model.layers.9.extra.weight"]
    assert len(error.wrong_shape) == 1 and "q_proj" in error.wrong_shape[0] and "[5, 5]" in error.wrong_shape[0]
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)"):
        assert needle in str(error)


def test_weight_dtypes_by_role(tmp_path):
    from mini_engine_b200.config import Qwen3Config, architecture_for
    from mini_engine_b200.parts.model import declared_weights
    from mini_engine_b200.weights import load_weights, write_random_model

    cfg = Qwen3Config.from_dict(CONFIGS["A"])
    folder = write_random_model(tmp_path / "m", cfg, 0, torch.float32)
    specs = declared_weights(architecture_for(cfg.architecture).build_spec(cfg))
    loaded = load_weights(folder, specs, torch.bfloat16, "cpu")
    assert loaded["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16  # matrices: compute dtype
    assert loaded["model.norm.weight"].dtype == torch.float32  # stored in 32-bit, stays 32-bit
    assert loaded["lm_head.weight"].data_ptr() == loaded["model.embed_tokens.weight"].data_ptr()  # tied


def _split_into_shards(folder, parts: int) -> dict[str, str]:
    """Rewrites ``model.safetensors`` of a folder as ``parts`` shard files with the usual names;
    returns tensor name -> file name."""
    from safetensors.torch import load_file, save_file

    state = {name: tensor.clone() for name, tensor in load_file(str(folder / "model.safetensors")).items()}
    (folder / "model.safetensors").unlink()
    names = sorted(state)
    weight_map = {}
    for part in range(parts):
        file_name = f"model-{part + 1:05d}-of-{parts:05d}.safetensors"
        mine = names[part::parts]  # interleaved: a layer's tensors lie in different files
        save_file({name: state[name] for name in mine}, str(folder / file_name))
        weight_map.update({name: file_name for name in mine})
    return weight_map


@pytest.mark.parametrize("with_index", [False, True])
def test_a_model_in_several_shards_loads_tensor_by_tensor(tmp_path, with_index):
    """A real checkpoint is several files, with or without ``model.safetensors.index.json``; the
    reference reads every file of the folder in sorted order
    (src/mini_engine/engine.py:126-128 of YuvGev00/mini-engine)."""
    from mini_engine_b200.config import Qwen3Config, architecture_for
    from mini_engine_b200.parts.model import declared_weights
    from mini_engine_b200.weights import load_weights, write_random_model

    cfg = Qwen3Config.from_dict(CONFIGS["B"])
    specs = declared_weights(architecture_for(cfg.architecture).build_spec(cfg))
    whole = load_weights(write_random_model(tmp_path / "whole", cfg, 5, torch.float32), specs, torch.float32, "cpu")
    folder = write_random_model(tmp_path / "sharded", cfg, 5, torch.float32)
    weight_map = _split_into_shards(folder, 3)
    if with_index:
        index = {"metadata": {"total_size": 0}, "weight_map": weight_map}
        (folder / "model.safetensors.index.json").write_text(json.dumps(index))
        # a file that the index does not name is not part of the model
        from safetensors.torch import save_file

        save_file({"model.layers.0.stray.weight": torch.zeros(3)}, str(folder / "stray.safetensors"))
    assert len(list(folder.glob("model-*.safetensors"))) == 3
    sharded = load_weights(folder, specs, torch.float32, "cpu")
    assert sorted(sharded) == sorted(whole)
    for name, tensor in whole.items():
        assert torch.equal(sharded[name], tensor), name


def test_a_shard_that_is_missing_is_reported_by_its_tensors(tmp_path):
    from mini_engine_b200.config import Qwen3Config, architecture_for
    from mini_engine_b200.parts.model import declared_weights
    from mini_engine_b200.weights import WeightError, load_weights, write_random_model

    cfg = Qwen3Config.from_dict(CONFIGS["A"])
    specs = declared_weights(architecture_for(cfg.architecture).build_spec(cfg))
    folder = write_random_model(tmp_path / "m", cfg, 5, torch.float32)
    weight_map = _split_into_shards(folder, 3)
    (folder / "model-00002-of-00003.safetensors").unlink()
    with pytest.raises(WeightError) as raised:
        load_weights(folder, specs, torch.float32, "cpu")
    gone = sorted(name for name, file_name in weight_map.items() if file_name.startswith("model-00002"))
    assert raised.value.missing == gone and not raised.value.unexpected


def test_a_tied_checkpoint_that_also_stores_its_head(tmp_path):
    """With tied embeddings a stored ``lm_head.weight`` is dropped and the head is the embedding's
    own storage (src/mini_engine/model.py:192-194 of YuvGev00/mini-engine)."""
    from safetensors.torch import load_file, save_file

    from mini_engine_b200.config import Qwen3Config, architecture_for
    from mini_engine_b200.parts.model import declared_weights
    from mini_engine_b200.weights import load_weights, write_random_model

    cfg = Qwen3Config.from_dict(CONFIGS["A"])
    assert cfg.tie_word_embeddings
    specs = declared_weights(architecture_for(cfg.architecture).build_spec(cfg))
    folder = write_random_model(tmp_path / "m", cfg, 6, torch.float32)
    state = {name: tensor.clone() for name, tensor in load_file(str(folder / "model.safetensors")).items()}
    state["lm_head.weight"] = torch.full_like(state["model.embed_tokens.weight"], 9.0)  # a stale copy
    save_file(state, str(folder / "model.safetensors"))
    loaded = load_weights(folder, specs, torch.float32, "cpu")
    assert loaded["lm_head.weight"].data_ptr() == loaded["model.embed_tokens.weight"].data_ptr()
    assert torch.equal(loaded["lm_head.weight"], state["model.embed_tokens.weight"])


def test_random_values_are_a_function_of_seed_name_and_index():
    """The generator is counter-based: any element can be made alone, in any chunking, and a
    matrix made in pieces equals the matrix made at once."""
    from mini_engine_b200.weights import random_init

    key = random_init._seed_for(3, "some.weight")
    whole = random_init.standard_normal(5000, key)
    assert torch.equal(random_init.standard_normal(100, key, first=4100), whole[4100:4200])
    old = random_init._CHUNK
    try:
        random_init._CHUNK = 777  # chunk edges must not show
        assert torch.equal(random_init.standard_normal(5000, key), whole)
    finally:
        random_init._CHUNK = old
    assert abs(float(whole.mean())) < 0.05 and abs(float(whole.std()) - 1.0) < 0.05
    assert not torch.equal(random_init.standard_normal(5000, random_init._seed_for(3, "other.weight")), whole)


def test_engine_config_validation():
    from mini_engine_b200 import EngineConfig, SamplingParams

    with pytest.raises(ValueError):
        EngineConfig(dtype=torch.float16)
    with pytest.raises(ValueError):
        EngineConfig(block_size=0)
    with pytest.raises(ValueError):
        SamplingParams(max_tokens=0)
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1.0)
