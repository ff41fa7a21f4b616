"""Configuration parsing and the architecture registry."""

import json

import pytest

from helpers import TINY_A, TINY_B
from torchllms_b200.config import ConfigError, get_architecture, load_config
from torchllms_b200.models.llama_config import LlamaConfig, RopeScaling


def write(tmp_path, raw, name="config.json"):
    (tmp_path / name).write_text(json.dumps(raw))
    return tmp_path


def test_reads_every_size_from_config_json(tmp_path):
    arch, cfg = load_config(write(tmp_path, TINY_B))
    assert arch.name == "LlamaForCausalLM"
    assert (cfg.n_layers, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim) == (3, 96, 3, 1, 32)
    assert (cfg.ffn_hidden, cfg.vocab_size, cfg.norm_eps, cfg.rope_theta) == (256, 1000, 1e-6, 500000.0)
    assert cfg.tie_word_embeddings and cfg.max_seq_len == 256
    assert cfg.rope_scaling == RopeScaling("llama3", 8.0, 1.0, 4.0, 64)


def test_defaults_follow_the_reference(tmp_path):
    raw = dict(TINY_A)
    del raw["num_key_value_heads"], raw["head_dim"], raw["tie_word_embeddings"]
    _, cfg = load_config(write(tmp_path, raw))
    assert cfg.n_kv_heads == cfg.n_heads == 4          # torchllms/models/networks.py:153-154
    assert cfg.head_dim == 64 // 4                      # :150-151
    assert cfg.tie_word_embeddings is False
    assert cfg.rope_scaling.rope_type == "default"


def test_round_trip_through_to_hf(tmp_path):
    for raw in (TINY_A, TINY_B):
        cfg = LlamaConfig.from_hf(raw)
        assert LlamaConfig.from_hf(cfg.to_hf()) == cfg


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                                 "vocab_size", "rms_norm_eps", "rope_theta", "architectures"])
def test_missing_key_is_named(tmp_path, key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        load_config(write(tmp_path, raw))


def test_bad_values_are_named(tmp_path):
    for key, value in (("num_key_value_heads", 3), ("head_dim", 15), ("rms_norm_eps", 0), ("vocab_size", "big"),
                       ("num_hidden_layers", 0)):
        raw = dict(TINY_A, **{key: value})
        with pytest.raises(ConfigError):
            LlamaConfig.from_hf(raw)
    with pytest.raises(ConfigError, match="rope_type"):
        LlamaConfig.from_hf(dict(TINY_B, rope_scaling={"rope_type": "yarn", "factor": 2.0}))
    with pytest.raises(ConfigError, match="attention_bias"):
        LlamaConfig.from_hf(dict(TINY_A, attention_bias=True))


def test_old_rope_type_key_is_accepted():
    raw = dict(TINY_B, rope_scaling={"type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64})
    assert LlamaConfig.from_hf(raw).rope_scaling.rope_type == "llama3"


def test_unknown_architecture_lists_the_known_ones(tmp_path):
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        load_config(write(tmp_path, dict(TINY_A, architectures=["MambaForCausalLM"])))
    with pytest.raises(ConfigError):
        get_architecture("nope")


def test_params_json_of_the_reference(tmp_path):
    raw = {"dim": 96, "n_layers": 3, "n_heads": 3, "n_kv_heads": 1, "vocab_size": 1000, "multiple_of": 256,
           "ffn_dim_multiplier": 256 / 96, "norm_eps": 1e-6, "rope_theta": 500000.0, "tie_word_embeddings": True,
           "rope_scaling": TINY_B["rope_scaling"], "max_seq_len": 256}
    arch, cfg = load_config(write(tmp_path, raw, "params.json"))
    assert cfg.ffn_hidden == 256 and cfg.head_dim == 32           # torchllms/models/networks.py:595-598, :150-151
    assert cfg == LlamaConfig.from_hf(TINY_B)
    with pytest.raises(ConfigError, match="olmo2_arch"):
        LlamaConfig.from_params_json(dict(raw, olmo2_arch=True))


def test_overrides_like_model_kwargs(tmp_path):
    _, cfg = load_config(write(tmp_path, TINY_A), {"max_seq_len": 64})
    assert cfg.max_seq_len == 64
    with pytest.raises(ConfigError, match="unknown"):
        cfg.with_overrides({"n_experts": 8})


def test_another_activation_is_refused():
    assert LlamaConfig.from_hf(dict(TINY_A, hidden_act="silu")) == LlamaConfig.from_hf(TINY_A)
    with pytest.raises(ConfigError, match="hidden_act"):
        LlamaConfig.from_hf(dict(TINY_A, hidden_act="gelu"))


def test_spec_is_data_and_takes_its_numbers_from_the_config():
    arch = get_architecture("LlamaForCausalLM")
    cfg = LlamaConfig.from_hf(TINY_B)
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 3 and [r.layer for r in spec.run_order] == [0, 1, 2]
    mixer = spec.layers[0].block["mixer"]
    assert (mixer.kind, mixer["n_heads"], mixer["n_kv_heads"], mixer["head_dim"]) == ("attention", 3, 1, 32)
    assert mixer["scale"] == 32 ** -0.5 and mixer["position"]["theta"] == 500000.0
    assert spec.layers[1].block["feed_forward"]["hidden"] == 256 and spec.layers[2].block["ffn_norm"]["eps"] == 1e-6
    assert spec.tie_head
