"""Configuration, registry, the loader's one error, and the random-weights mode."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import helpers
from paged_attention_engine_b200.config import ConfigError, Qwen2Config, resolve, resolve_folder
from paged_attention_engine_b200.weights import (
    WeightsError, collect_tensor_specs, load_tensors, write_random_model,
)


def test_config_reads_every_key_and_defaults_only_head_dim():
    raw = dict(helpers.TINY_B)
    cfg, spec = resolve(raw)
    assert isinstance(cfg, Qwen2Config)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 3, 1)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (32, 256, 509)
    assert (cfg.rope_theta, cfg.rms_norm_eps, cfg.max_position_embeddings, cfg.tie_word_embeddings) == (1e6, 1e-5, 256, False)
    assert cfg.num_kv_groups == 3 and cfg.attention_scale == 32 ** -0.5
    del raw["head_dim"]
    assert resolve(raw)[0].head_dim == 32          # hidden // heads, the reference's fallback
    nested = dict(raw)
    del nested["rope_theta"]
    nested["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert resolve(nested)[0].rope_theta == 12345.0
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.layers[1].mixer.params["num_kv_heads"] == 1


@pytest.mark.parametrize(
    "change,word",
    [
        ({"hidden_size": None}, "hidden_size"),
        ({"num_key_value_heads": 2}, "num_key_value_heads"),
        ({"head_dim": 15}, "head_dim"),
        ({"hidden_act": "gelu"}, "hidden_act"),
        ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_type"),
        ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
        ({"vocab_size": 0}, "vocab_size"),
        ({"architectures": ["LlamaForCausalLM"]}, "LlamaForCausalLM"),
        ({"use_sliding_window": True}, "sliding_window"),
        ({"max_position_embeddings": None}, "max_position_embeddings"),
    ],
)
def test_config_errors_name_the_key(change, word):
    raw = dict(helpers.TINY_B)
    raw.update(change)
    raw = {k: v for k, v in raw.items() if v is not None}
    with pytest.raises(ConfigError) as err:
        resolve(raw)
    assert word in str(err.value)


def test_unknown_architecture_lists_the_known_ones():
    with pytest.raises(ConfigError) as err:
        resolve({"architectures": ["Nope"]})
    assert "Qwen2ForCausalLM" in str(err.value)


def test_window_layers_follow_the_config():
    cfg, spec = resolve(helpers.TINY_C)
    assert [cfg.layer_window(i) for i in range(4)] == [0, 0, 24, 24]
    assert [layer.mixer.params["window"] for layer in spec.layers] == [0, 0, 24, 24]


def test_random_model_folder_round_trips(tmp_path):
    folder = write_random_model(tmp_path / "m", helpers.TINY_A, seed=7, dtype=torch.bfloat16)
    cfg, spec = resolve_folder(folder)
    assert cfg.tie_word_embeddings and cfg.vocab_size == 256
    stored = load_file(str(folder / "model.safetensors"))
    assert set(stored) == set(collect_tensor_specs(spec))
    assert "lm_head.weight" not in stored
    assert all(t.dtype == torch.bfloat16 for t in stored.values())
    norm = stored["model.layers.0.input_layernorm.weight"].float()
    assert 0.9 < norm.mean() < 1.1 and stored["model.layers.0.self_attn.q_proj.bias"].float().abs().max() < 0.2
    again = write_random_model(tmp_path / "n", helpers.TINY_A, seed=7, dtype=torch.bfloat16)
    assert all(torch.equal(stored[k], v) for k, v in load_file(str(again / "model.safetensors")).items())
    other = load_file(str(write_random_model(tmp_path / "o", helpers.TINY_A, seed=8, dtype=torch.bfloat16) / "model.safetensors"))
    assert not torch.equal(other["model.norm.weight"], stored["model.norm.weight"])


def test_loader_storage_classes(tmp_path):
    folder = write_random_model(tmp_path / "m", helpers.TINY_B, seed=1, dtype=torch.bfloat16)
    _, spec = resolve_folder(folder)
    tensors = load_tensors(folder, spec, torch.bfloat16, "cpu")
    assert tensors["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert tensors["model.layers.0.self_attn.k_proj.bias"].dtype == torch.float32
    assert tensors["model.norm.weight"].dtype == torch.float32
    wide = load_tensors(folder, spec, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in wide.values())
    # A matrix that the file stores in 32-bit stays in 32-bit in a bfloat16 engine.
    path = str(folder / "model.safetensors")
    stored = load_file(path)
    stored["lm_head.weight"] = stored["lm_head.weight"].float()
    save_file(stored, path)
    assert load_tensors(folder, spec, torch.bfloat16, "cpu")["lm_head.weight"].dtype == torch.float32


def test_loader_raises_one_error_with_everything_in_it(tmp_path):
    folder = write_random_model(tmp_path / "m", helpers.TINY_B, seed=1, dtype=torch.float32)
    _, spec = resolve_folder(folder)
    path = str(folder / "model.safetensors")
    stored = load_file(path)
    del stored["model.layers.1.mlp.up_proj.weight"]
    del stored["model.norm.weight"]
    stored["model.layers.9.extra.weight"] = torch.zeros(3)
    stored["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(96, 95)
    save_file(stored, path)
    with pytest.raises(WeightsError) as err:
        load_tensors(folder, spec, torch.float32, "cpu")
    text = str(err.value)
    for fragment in (
        "missing (2)", "model.layers.1.mlp.up_proj.weight", "model.norm.weight",
        "unexpected (1)", "model.layers.9.extra.weight",
        "wrong shape (1)", "model.layers.0.self_attn.q_proj.weight", "(96, 95)", "(96, 96)",
    ):
        assert fragment in text, fragment


def test_tied_head_must_not_be_in_the_file(tmp_path):
    folder = write_random_model(tmp_path / "m", helpers.TINY_A, seed=1, dtype=torch.float32)
    _, spec = resolve_folder(folder)
    path = str(folder / "model.safetensors")
    stored = load_file(path)
    stored["lm_head.weight"] = torch.zeros(256, 64)
    save_file(stored, path)
    with pytest.raises(WeightsError) as err:
        load_tensors(folder, spec, torch.float32, "cpu")
    assert "unexpected (1): lm_head.weight" in str(err.value)
    raw = json.loads((folder / "config.json").read_text())
    raw["tie_word_embeddings"] = False
    (folder / "config.json").write_text(json.dumps(raw))
    _, untied = resolve_folder(folder)
    load_tensors(folder, untied, torch.float32, "cpu")


def test_missing_files_are_named(tmp_path):
    with pytest.raises(ConfigError):
        resolve_folder(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(helpers.TINY_A))
    _, spec = resolve_folder(tmp_path)
    with pytest.raises(WeightsError) as err:
        load_tensors(tmp_path, spec, torch.float32, "cpu")
    assert "model.safetensors" in str(err.value)


def _split_into_shards(folder):
    """Rewrites a one-file checkpoint as two shards and an index, as larger checkpoints come."""
    path = folder / "model.safetensors"
    stored = load_file(str(path))
    names = sorted(stored)
    first, second = names[: len(names) // 2], names[len(names) // 2 :]
    save_file({n: stored[n] for n in first}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({n: stored[n] for n in second}, str(folder / "model-00002-of-00002.safetensors"))
    weight_map = {n: "model-00001-of-00002.safetensors" for n in first}
    weight_map.update({n: "model-00002-of-00002.safetensors" for n in second})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    path.unlink()
    return stored


def test_loader_reads_shards_through_the_index(tmp_path):
    folder = write_random_model(tmp_path / "m", helpers.TINY_B, seed=4, dtype=torch.float32)
    _, spec = resolve_folder(folder)
    whole = load_tensors(folder, spec, torch.float32, "cpu")
    stored = _split_into_shards(folder)
    sharded = load_tensors(folder, spec, torch.float32, "cpu")
    assert set(sharded) == set(whole) == set(stored)
    for name in whole:
        assert torch.equal(sharded[name], whole[name]), name


def test_a_shard_that_the_index_names_but_is_not_there(tmp_path):
    folder = write_random_model(tmp_path / "m", helpers.TINY_B, seed=4, dtype=torch.float32)
    _, spec = resolve_folder(folder)
    _split_into_shards(folder)
    (folder / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(WeightsError) as err:
        load_tensors(folder, spec, torch.float32, "cpu")
    assert "model-00002-of-00002.safetensors" in str(err.value) and "not there" in str(err.value)


def test_a_shard_without_a_tensor_lists_it_as_missing(tmp_path):
    folder = write_random_model(tmp_path / "m", helpers.TINY_B, seed=4, dtype=torch.float32)
    _, spec = resolve_folder(folder)
    _split_into_shards(folder)
    shard = str(folder / "model-00001-of-00002.safetensors")
    stored = load_file(shard)
    gone = sorted(stored)[0]
    del stored[gone]
    save_file(stored, shard)
    with pytest.raises(WeightsError) as err:
        load_tensors(folder, spec, torch.float32, "cpu")
    assert "missing (1)" in str(err.value) and gone in str(err.value)


def test_engine_options_size_the_pool_by_pages_or_by_bytes():
    from paged_attention_engine_b200.cache import plan_cache
    from paged_attention_engine_b200.config import EngineConfig

    assert EngineConfig().pool_blocks(1000) == 3584                       # the reference's pool
    assert EngineConfig(num_blocks=77).pool_blocks(1000) == 77
    _, spec = resolve(dict(helpers.TINY_B))
    plan = plan_cache(spec)
    # tiny B: 3 layers x 1 kv head x 32 x (keys + values) x 16 tokens x 4 bytes
    per_block = plan.bytes_per_block(16, 4)
    assert per_block == 3 * 1 * 32 * 2 * 16 * 4
    assert EngineConfig(kv_bytes=10 * per_block + per_block - 1).pool_blocks(per_block) == 10
    # tiny C has two page groups (windowed and not), each with a pool of its own
    _, spec_c = resolve(dict(helpers.TINY_C))
    assert plan_cache(spec_c).bytes_per_block(8, 2) == 4 * 5 * 48 * 2 * 8 * 2
    for bad in (dict(num_blocks=4, kv_bytes=4096), dict(block_size=0), dict(kv_bytes=0), dict(max_num_seqs=0),
                dict(dtype="float16"), dict(admission_margin_blocks=-1)):
        with pytest.raises(ConfigError):
            EngineConfig(**bad)
    with pytest.raises(ConfigError, match="does not pay for one page"):
        EngineConfig(kv_bytes=per_block - 1).pool_blocks(per_block)
    with pytest.raises(ConfigError, match="unknown engine option"):
        EngineConfig.from_options({"num_block": 3})
