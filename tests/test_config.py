"""Configuration and registries (no GPU)."""
import copy

import pytest

from helpers import TINY_A, TINY_B, TINY_C
from pulsar_b200.config import (ARCHITECTURES, ConfigError, EngineConfig, architecture_name,
                                config_from_dict)
from pulsar_b200.models.qwen3 import Qwen3Config


def test_reads_the_architectures_own_keys():
    cfg = config_from_dict(TINY_B)
    assert isinstance(cfg, Qwen3Config)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (512, 96, 320, 3)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (8, 2, 32)
    assert cfg.num_attention_heads * cfg.head_dim != cfg.hidden_size
    assert cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5 and cfg.tie_word_embeddings is False
    assert cfg.eos_token_id == 11


def test_head_dim_defaults_to_hidden_over_heads():
    raw = dict(TINY_A)
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == 64 // 4
    raw["head_dim"] = None
    assert config_from_dict(raw).head_dim == 16


def test_eos_list_takes_first_and_missing_is_none():
    assert config_from_dict(dict(TINY_A, eos_token_id=[9, 3])).eos_token_id == 9
    raw = dict(TINY_A)
    del raw["eos_token_id"]
    assert config_from_dict(raw).eos_token_id == -1


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "rope_theta", "rms_norm_eps"])
def test_required_keys(key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(raw)


@pytest.mark.parametrize("change,match", [
    (dict(num_key_value_heads=3), "multiple"), (dict(head_dim=15), "even"), (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "attention_bias"), (dict(rope_scaling={"type": "yarn", "factor": 4}), "rope_scaling"),
    (dict(use_sliding_window=True, sliding_window=None), "sliding_window"), (dict(vocab_size=0), "positive"),
    (dict(vocab_size="256"), "integer"), (dict(rms_norm_eps=0.0), "positive")])
def test_rejects_what_the_engine_does_not_implement(change, match):
    with pytest.raises(ConfigError, match=match):
        config_from_dict(dict(TINY_A, **change))


def test_unknown_architecture_lists_known_names():
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict(dict(TINY_A, architectures=["NopeForCausalLM"]))
    raw = dict(TINY_A)
    del raw["architectures"]
    assert architecture_name(raw) == "qwen3" and isinstance(config_from_dict(raw), Qwen3Config)
    del raw["model_type"]
    with pytest.raises(ConfigError, match="neither"):
        config_from_dict(raw)
    assert "Qwen3ForCausalLM" in ARCHITECTURES.names()


def test_window_per_layer_and_model_spec():
    cfg = config_from_dict(TINY_C)
    assert [cfg.layer_window(i) for i in range(4)] == [None, None, 12, 12]
    spec = cfg.model_spec()
    assert [b.mixer.window for b in spec.blocks] == [None, None, 12, 12]
    assert [(c.block, c.cache) for c in spec.run_order] == [(i, i) for i in range(4)]
    m = spec.blocks[0].mixer
    assert (m.n_heads, m.n_kv_heads, m.head_dim, m.qk_norm_eps) == (6, 3, 48, 3e-6)
    assert abs(m.scale - 48 ** -0.5) < 1e-15 and m.position.theta == 500000.0 and m.position.rotary_dim == 48
    assert spec.blocks[2].feed_forward.intermediate == 176 and spec.final_norm.eps == 3e-6
    assert config_from_dict(TINY_A).model_spec().blocks[1].mixer.window is None


def test_layer_types_decide_where_they_are_listed():
    kinds = ["sliding_attention", "full_attention", "full_attention", "sliding_attention"]
    cfg = config_from_dict(dict(TINY_C, layer_types=kinds))                  # TINY_C alone: layers 2 and 3 slide
    assert [cfg.layer_window(i) for i in range(4)] == [12, None, None, 12]
    assert [b.mixer.window for b in cfg.model_spec().blocks] == [12, None, None, 12]
    assert config_from_dict(cfg.to_dict()) == cfg
    with pytest.raises(ConfigError, match="names 3 layers"):
        config_from_dict(dict(TINY_C, layer_types=kinds[:3]))
    with pytest.raises(ConfigError, match="chunked_attention"):
        config_from_dict(dict(TINY_C, layer_types=kinds[:3] + ["chunked_attention"]))
    with pytest.raises(ConfigError, match="sliding_window"):
        config_from_dict(dict(TINY_A, layer_types=["full_attention", "sliding_attention"]))


def test_rotary_settings_as_one_dictionary():
    raw = {k: v for k, v in TINY_B.items() if k != "rope_theta"}
    cfg = config_from_dict(dict(raw, rope_parameters={"rope_theta": 250000.0, "rope_type": "default"}))
    assert cfg.rope_theta == 250000.0 and cfg.model_spec().blocks[0].mixer.position.theta == 250000.0
    with pytest.raises(ConfigError, match="rope_scaling"):
        config_from_dict(dict(raw, rope_parameters={"rope_theta": 1e6, "rope_type": "yarn", "factor": 4.0}))
    with pytest.raises(ConfigError, match="rope_theta"):
        config_from_dict(dict(raw, rope_parameters={"rope_type": "default"}))


def test_to_dict_round_trip():
    for raw in (TINY_A, TINY_B, TINY_C):
        cfg = config_from_dict(raw)
        assert config_from_dict(cfg.to_dict()) == cfg


def test_engine_config_rejects_unknown_keys_and_checks_invariants():
    with pytest.raises(ConfigError, match=r"\['bogus', 'zzz'\]"):
        EngineConfig.from_dict({"zzz": 1, "bogus": 2, "page_size": 16})
    cfg = EngineConfig.from_dict({"max_sessions": 2, "active_buffer_size": 64, "page_size": 16, "dtype": "fp32"})
    assert cfg.num_pages == 8 and cfg.dtype == "float32"       # max_sessions * active_buffer_size / page_size
    with pytest.raises(ConfigError, match="multiple"):
        EngineConfig.from_dict({"active_buffer_size": 50, "page_size": 16})
    with pytest.raises(ConfigError, match="dtype"):
        EngineConfig.from_dict({"dtype": "int4"})
    with pytest.raises(ConfigError, match="page_size"):
        EngineConfig.from_dict({"page_size": 0})
    with pytest.raises(ConfigError, match="top_p"):
        EngineConfig.from_dict({"top_p": 0.0})
    assert EngineConfig.from_dict({}).temperature == 0.0 and EngineConfig.from_dict({}).seed == -1


def test_decode_splits_choice():
    """The number of key splits of the decode attention: fills the SMs once while everything fits, stays within
    one split per 256 tokens of the block table, and takes more than one split where a single one would leave a
    thin last round of blocks (the measured cases: batch 48 with 8 kv heads, not batch 64)."""
    from pulsar_b200 import ops
    assert ops.decode_splits(8, 8, 4096 + 64) == 4
    assert ops.decode_splits(1, 8, 4096 + 64) == 16
    assert ops.decode_splits(1, 8, 32768) == 32
    assert ops.decode_splits(64, 8, 4096 + 64) == 1
    assert ops.decode_splits(48, 8, 4096 + 64) in (2, 3)
    for batch in range(1, 300, 7):
        for heads in (1, 2, 8):
            for tokens in (16, 300, 4096, 100000):
                k = ops.decode_splits(batch, heads, tokens)
                assert 1 <= k <= 32 and k <= max(1, tokens // 256)
                assert k == ops.decode_splits(batch, heads, tokens)
