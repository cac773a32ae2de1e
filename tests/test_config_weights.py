"""Configuration hydration, the architecture registry, and the strict weight loader."""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny_configs
from mlx_omnia_b200.architectures.muse_glimmer import MuseGlimmerConfig, model_spec, parse
from mlx_omnia_b200.config import ConfigError
from mlx_omnia_b200.parts.base import Runtime
from mlx_omnia_b200.parts.model import DecoderModel
from mlx_omnia_b200.registry import resolve_architecture
from mlx_omnia_b200.weights import WeightError, load_tensors, write_random_model

CPU = Runtime(torch.bfloat16, torch.device("cpu"))


def test_nested_and_flat_configs_hydrate_alike():
    raw = tiny_configs.config("B")
    nested = parse(raw)
    flat = parse({**raw["text_config"], "model_type": "muse_glimmer", "unknown_key": 3})
    assert isinstance(nested, MuseGlimmerConfig) and nested == flat
    c = nested.text_config
    assert c.layer_types == ("sliding_attention", "full_attention", "sliding_attention")
    assert c.layer_rope_theta == (1000000.0, 0.0, 1000000.0) and c.eos == (1, 2)
    assert c.rope_parameters.rope_theta == 1000000.0 and parse(tiny_configs.config("A")).text_config.eos == (0,)


def test_config_errors_name_the_problem():
    raw = tiny_configs.config("A")
    del raw["text_config"]["post_norm_eps"]
    with pytest.raises(ConfigError, match="post_norm_eps"):
        parse(raw)
    for key, value, message in [("layer_types", ["full_attention", "banana"], "unknown layer types"),
                                ("layer_rope_theta", [1.0], "disagree"),
                                ("num_key_value_heads", 3, "do not divide"), ("head_dim", 15, "even")]:
        raw = tiny_configs.config("A")
        raw["text_config"][key] = value
        with pytest.raises(ConfigError, match=message):
            parse(raw)
    with pytest.raises(ConfigError, match="model_type"):
        parse({**tiny_configs.config("A"), "model_type": "qwen3"})


def test_registry_resolves_by_architecture_then_model_type():
    assert resolve_architecture({"architectures": ["MuseGlimmerForConditionalGeneration"]}).name == "muse_glimmer"
    assert resolve_architecture({"architectures": ["Unknown"], "model_type": "muse_glimmer"}).name == "muse_glimmer"
    with pytest.raises(ValueError, match="unsupported architecture"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})


def test_model_spec_is_chosen_layer_by_layer():
    spec = model_spec(parse(tiny_configs.config("B")))
    mixers = [layer.block.params["mixer"].params for layer in spec.layers]
    assert [m["window"] for m in mixers] == [16, None, 16]
    assert [m["position"].kind for m in mixers] == ["rotary", "none", "rotary"]
    assert mixers[0]["scale"] == pytest.approx(1.25 * 24 ** -0.5) and spec.head.params["softcap"] == 20.0
    model = DecoderModel(spec)
    names = model.tensors()
    assert names["model.layers.1.self_attn.gate_proj.weight"].shape == (192, 96)
    assert names["model.layers.2.input_layernorm.weight"].kind == "vector"
    assert "lm_head.weight" in names
    assert "lm_head.weight" not in DecoderModel(model_spec(parse(tiny_configs.config("A")))).tensors()
    needs = model.cache_needs()
    assert [n.kv.window for n in needs] == [16, None, 16] and all(n.state is None for n in needs)


def test_random_folder_loads_and_keeps_dtypes(tmp_path):
    raw = tiny_configs.config("A")
    folder = write_random_model(tmp_path / "m", raw, seed=3)
    assert json.loads((folder / "config.json").read_text()) == raw
    stored = load_file(str(folder / "model.safetensors"))
    assert stored["model.language_model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert stored["model.language_model.norm.weight"].dtype == torch.float32
    again = load_file(str(write_random_model(tmp_path / "n", raw, seed=3) / "model.safetensors"))
    assert all(torch.equal(stored[k], again[k]) for k in stored)
    architecture = resolve_architecture(raw)
    config = architecture.parse(raw)
    model = DecoderModel(architecture.model_spec(config))
    for runtime, matrix in [(CPU, torch.bfloat16), (Runtime(torch.float32, torch.device("cpu")), torch.float32)]:
        tensors = load_tensors(folder, architecture, config, model.tensors(), runtime)
        assert set(tensors) == set(model.tensors())
        assert tensors["model.layers.1.self_attn.q_proj.weight"].dtype == matrix
        assert tensors["model.layers.1.input_layernorm.weight"].dtype == torch.float32
        assert torch.equal(tensors["model.embed_tokens.weight"].float(),
                           stored["model.language_model.embed_tokens.weight"].float())


def test_weight_errors_list_everything_at_once(tmp_path):
    raw = tiny_configs.config("B")
    folder = write_random_model(tmp_path / "m", raw, seed=1)
    stored = load_file(str(folder / "model.safetensors"))
    del stored["model.language_model.layers.2.mlp.down_proj.weight"]
    del stored["lm_head.weight"]
    stored["model.language_model.layers.0.extra.weight"] = torch.zeros(3)
    stored["model.vision_tower.patch.weight"] = torch.zeros(3)  # ignored on purpose
    stored["model.language_model.layers.1.self_attn.k_proj.weight"] = torch.zeros(24, 95, dtype=torch.bfloat16)
    save_file(stored, str(folder / "model.safetensors"))
    architecture = resolve_architecture(raw)
    config = architecture.parse(raw)
    model = DecoderModel(architecture.model_spec(config))
    with pytest.raises(WeightError) as caught:
        load_tensors(folder, architecture, config, model.tensors(), CPU)
    error = caught.value
    assert error.missing == ["lm_head.weight", "model.layers.2.mlp.down_proj.weight"]
    assert error.unexpected == ["model.language_model.layers.0.extra.weight"]
    assert len(error.wrong) == 1 and "k_proj" in error.wrong[0] and "[24, 95]" in error.wrong[0]
    text = str(error)
    assert "missing (2)" in text and "unexpected (1)" in text and "wrong shape" in text


def test_tied_head_drops_a_stored_lm_head(tmp_path):
    raw = tiny_configs.config("A")
    folder = write_random_model(tmp_path / "m", raw, seed=1)
    stored = load_file(str(folder / "model.safetensors"))
    stored["lm_head.weight"] = torch.zeros(512, 64, dtype=torch.bfloat16)
    save_file(stored, str(folder / "model.safetensors"))
    architecture = resolve_architecture(raw)
    config = architecture.parse(raw)
    model = DecoderModel(architecture.model_spec(config))
    assert "lm_head.weight" not in load_tensors(folder, architecture, config, model.tensors(), CPU)
