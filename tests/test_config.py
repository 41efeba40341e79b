"""Configuration from config.json keys, and the registry from architecture name to model."""
import json

import pytest

from tiny_configs import TINY_A, TINY_B, TINY_C

from llm_infrence_engine_b200.config import ConfigError, EngineConfig, Qwen2Config, read_config_json
from llm_infrence_engine_b200.models import build_model_spec, known_architectures, register_architecture
from llm_infrence_engine_b200.cache import PagedKVSpec


def test_reads_every_key():
    c = Qwen2Config.from_dict(TINY_B)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (320, 96, 200, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 1, 32)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and c.tie_word_embeddings is False and c.attention_bias is True
    c = Qwen2Config.from_dict(TINY_C)
    assert c.head_dim == 48 and c.attention_bias is False
    assert [c.layer_window(i) for i in range(4)] == [None, None, 24, 24]


def test_defaults_follow_the_reference():
    d = {k: v for k, v in TINY_A.items() if k not in ("rope_theta", "tie_word_embeddings")}
    c = Qwen2Config.from_dict(d)
    assert c.rope_theta == 10000.0 and c.tie_word_embeddings is False  # src/miniserve/model.py:45-47,57
    d["rope_parameters"] = {"rope_theta": 5e5}
    assert Qwen2Config.from_dict(d).rope_theta == 5e5


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"head_dim": 15}, "even"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768}}, "rope_scaling"),
    ({"rope_parameters": {"rope_theta": 1e6, "rope_type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"partial_rotary_factor": 0.5}, "partial_rotary_factor"),
    ({"attention_dropout": 0.1}, "attention_dropout"),
    ({"mlp_bias": True}, "mlp_bias"),
])
def test_rejects_what_makes_no_sense(change, match):
    with pytest.raises(ConfigError, match=match):
        Qwen2Config.from_dict(dict(TINY_A, **change))


def test_neutral_values_of_unread_keys_pass():
    """Absent, null or neutral: nothing to refuse (real Qwen2 checkpoints carry ``attention_dropout: 0.0``)."""
    c = Qwen2Config.from_dict(dict(TINY_A, rope_scaling=None, attention_dropout=0.0, partial_rotary_factor=1.0, mlp_bias=False,
                                   rope_parameters={"rope_theta": 1e4, "rope_type": "default"}))
    assert c.rope_theta == TINY_A["rope_theta"]


def test_missing_key_is_named():
    d = dict(TINY_A)
    del d["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        Qwen2Config.from_dict(d)


def test_registry_chooses_by_name(tmp_path):
    assert "Qwen2ForCausalLM" in known_architectures()
    spec = build_model_spec(TINY_C)
    assert len(spec.layers) == 4 and len(spec.schedule) == 4
    assert spec.cache_specs() == [PagedKVSpec(3, 48, None)] * 2 + [PagedKVSpec(3, 48, 24)] * 2
    assert spec.head.tied_to is spec.embedding
    assert build_model_spec(TINY_B).head.tied_to is None
    with pytest.raises(ConfigError, match="LlamaForCausalLM.*known.*Qwen2ForCausalLM"):
        build_model_spec(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        build_model_spec({k: v for k, v in TINY_A.items() if k != "architectures"})
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("Qwen2ForCausalLM", Qwen2Config, lambda c: None)
    (tmp_path / "config.json").write_text("{ not json")
    with pytest.raises(ConfigError, match="not JSON"):
        read_config_json(tmp_path)


def test_no_size_is_written_in_the_parts():
    """The same code builds models that differ in every size: sizes come from the configuration alone."""
    for cfg in (TINY_A, TINY_B, TINY_C):
        spec = build_model_spec(cfg)
        m = spec.layers[0].mixer
        assert m.w_qkv is None  # no weights yet
        shapes = {k: p.shape for k, p in m.params().items()}
        c = Qwen2Config.from_dict(cfg)
        assert shapes["w_qkv"] == ((c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim, c.hidden_size)
        assert ("b_qkv" in shapes) == c.attention_bias
        assert spec.layers[0].ff.params()["w_gate_up"].shape == (2 * c.intermediate_size, c.hidden_size)


def test_engine_config():
    e = EngineConfig(max_seqs=4, max_len=100, block_size=16)
    assert e.pool_blocks() == 4 * 7 + 1
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16").validate()
    with pytest.raises(ValueError):
        EngineConfig(num_blocks=1).validate()
