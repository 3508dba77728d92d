import json

import pytest

import helpers as H
from batchspec_b200.config import (ConfigError, LlamaConfig, config_from_json_dict, get_config, load_config,
                                   register_config, save_config)


def test_llama_config_reads_its_own_keys():
    cfg = config_from_json_dict(H.TINY_B)
    assert isinstance(cfg, LlamaConfig)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (96, 3, 3, 1)
    assert cfg.head_dim == 32 and cfg.intermediate_size == 256 and cfg.vocab_size == 1000
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 500000.0 and cfg.tie_word_embeddings
    rs = cfg.rope_scaling
    assert (rs.rope_type, rs.factor, rs.low_freq_factor, rs.high_freq_factor, rs.original_max_position_embeddings) == \
        ("llama3", 8.0, 1.0, 4.0, 64)


def test_defaults_derived_not_assumed():
    d = dict(H.TINY_A)
    del d["num_key_value_heads"], d["head_dim"]
    cfg = config_from_json_dict(d)
    assert cfg.num_key_value_heads == cfg.num_attention_heads == 4 and cfg.head_dim == 64 // 4
    for key in ("rms_norm_eps", "rope_theta", "intermediate_size", "vocab_size", "max_position_embeddings"):
        bad = dict(H.TINY_A)
        del bad[key]
        with pytest.raises(ConfigError, match=key):
            config_from_json_dict(bad)


@pytest.mark.parametrize("patch, word", [
    (dict(architectures=["MambaForCausalLM"]), "not registered"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "yarn"),
    (dict(hidden_act="gelu"), "gelu"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(hidden_size="64"), "integer"),
    (dict(head_dim=15), "even"),
    (dict(model_type="mistral"), "model_type"),
    (dict(sliding_window=4096), "sliding_window"),
    (dict(attention_dropout=0.1), "attention_dropout"),
    (dict(partial_rotary_factor=0.5), "partial_rotary_factor"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                            original_max_position_embeddings=64, attention_factor=1.3)), "attention_factor"),
    (dict(rope_scaling=dict(rope_type="linear", factor=2.0, low_freq_factor=1.0)), "low_freq_factor"),
])
def test_rejects_what_it_cannot_run(patch, word):
    with pytest.raises(ConfigError, match=word):
        config_from_json_dict({**H.TINY_A, **patch})


def test_keys_nothing_reads_are_listed_and_neutral_values_pass():
    cfg = config_from_json_dict({**H.TINY_A, "sliding_window": None, "attention_dropout": 0.0, "use_cache": True,
                                 "pretraining_tp": 1, "some_new_option": 3, "another": "x"})
    assert cfg.unread_keys == ("another", "some_new_option")
    assert config_from_json_dict(H.TINY_A).unread_keys == ()
    assert "unread_keys" not in cfg.to_json_dict()


def test_round_trip_through_a_folder(tmp_path):
    for d in (H.TINY_A, H.TINY_B, H.TINY_C):
        cfg = config_from_json_dict(d)
        save_config(cfg, tmp_path)
        assert load_config(tmp_path) == cfg
        assert json.loads((tmp_path / "config.json").read_text())["architectures"] == ["LlamaForCausalLM"]


def test_eos_may_be_a_list():
    assert config_from_json_dict({**H.TINY_A, "eos_token_id": [7, 9]}).eos_token_ids == (7, 9)
    assert config_from_json_dict({**H.TINY_A, "eos_token_id": 7}).eos_token_ids == (7,)


def test_by_name_table_lookup_rule():
    cfg = get_config("llama-3-8b")
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size) == (32, 4096, 14336, 128256)
    assert get_config("meta-llama/Llama-3.1-8B-Instruct").rope_scaling.factor == 8.0     # longest substring wins
    with pytest.raises(ValueError, match="No configuration"):
        get_config("gpt-2")
    register_config("zz-tiny1", H.TINY_A)
    register_config("zz-tiny2", H.TINY_B)
    with pytest.raises(ValueError, match="Ambiguous"):
        get_config("zz-tiny1-zz-tiny2")
