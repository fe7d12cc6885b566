"""Configuration: reading, defaults, the feed-forward width rule, every validation error, and
the registry from architecture name to model."""
import copy

import pytest

import helpers
from zinfer_b200.config import (ConfigError, Lfm2Config, build_model, config_from_dict, register_architecture,
                                registered_architectures, unregister_architecture)

A = helpers.TINY["tiny_a"]["config"]
B = helpers.TINY["tiny_b"]["config"]
C = helpers.TINY["tiny_c"]["config"]


def test_typed_fields_come_from_config_json():
    cfg = config_from_dict(B)
    assert isinstance(cfg, Lfm2Config)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers) == (512, 96, 6)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (3, 1, 32)
    assert cfg.layer_types[0] == "full_attention" and cfg.layer_types[1] == "conv"
    assert cfg.conv_L_cache == 4 and cfg.conv_bias is True
    assert cfg.rope_theta == 1e6 and cfg.norm_eps == 1e-6
    assert cfg.tie_word_embeddings is False and cfg.eos_token_ids == (3, 5)
    assert config_from_dict(A).eos_token_ids == (7,)


def test_feed_forward_width_rule():
    assert config_from_dict(A).ffn_dim == 128                      # auto-adjust off
    assert config_from_dict(B).ffn_dim == 192                      # 288 -> 192, multiple of 64
    big = dict(B, block_ff_dim=12288, block_multiple_of=256)
    assert config_from_dict(big).ffn_dim == 8192
    assert config_from_dict(dict(big, block_ff_dim=16128)).ffn_dim == 10752
    assert config_from_dict(dict(big, block_ff_dim=6912)).ffn_dim == 4608
    assert config_from_dict(C).ffn_dim == 136                      # int(400/3)=133 -> 136
    d = dict(A)
    d.pop("block_ff_dim")
    d["intermediate_size"] = 100
    assert config_from_dict(d).ffn_dim == 100


def test_defaults_and_aliases():
    d = {k: v for k, v in A.items() if k not in ("norm_eps", "rope_theta", "conv_L_cache", "conv_bias", "tie_word_embeddings")}
    cfg = config_from_dict(d)
    assert (cfg.norm_eps, cfg.rope_theta, cfg.conv_L_cache, cfg.conv_bias, cfg.tie_word_embeddings) == (1e-5, 10000.0, 3, False, True)
    assert config_from_dict(dict(d, rope_parameters={"rope_theta": 5.0, "rope_type": "default"})).rope_theta == 5.0
    assert config_from_dict(dict(d, tie_embedding=False)).tie_word_embeddings is False
    d2 = dict(d)
    d2.pop("layer_types")
    d2["full_attn_idxs"] = [1, 3]
    assert config_from_dict(d2).layer_types == tuple(A["layer_types"])
    assert config_from_dict(A).head_dim == 16 and config_from_dict(C).head_dim == 48


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "max_position_embeddings", "block_ff_dim", "layer_types"])
def test_missing_key_is_named(key):
    d = dict(A)
    d.pop(key)
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("change,match", [
    (dict(layer_types=["conv", "full_attention"]), "layer_types has 2 entries"),
    (dict(layer_types=["conv", "mamba", "conv", "full_attention"]), "mamba"),
    (dict(num_key_value_heads=3), "not a multiple"),
    (dict(conv_L_cache=1), "conv_L_cache"),
    (dict(conv_L_cache=65), "64 taps"),
    (dict(norm_eps=0.0), "norm_eps"),
    (dict(rope_theta=-1.0), "rope_theta"),
    (dict(vocab_size=0), "vocab_size"),
    (dict(vocab_size="many"), "vocab_size"),
    (dict(hidden_size=66), "head_dim"),
    (dict(head_dim=15), "even"),
    (dict(layer_types=["conv", "sliding_attention", "conv", "full_attention"]), "sliding_window"),
    (dict(full_attn_idxs=[9], layer_types=None), "full_attn_idxs"),
])
def test_validation_errors(change, match):
    with pytest.raises(ConfigError, match=match):
        config_from_dict(dict(A, **change))


def test_registry_knows_the_architecture_and_names_the_unknown():
    assert "Lfm2ForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError, match="NoSuchModel.*Lfm2ForCausalLM"):
        config_from_dict(dict(A, architectures=["NoSuchModel"]))
    d = dict(A)
    d.pop("architectures")
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict(d)


def test_another_architecture_can_be_registered():
    made = {}

    class Cfg(Lfm2Config):
        pass

    def build(cfg):
        made["cfg"] = cfg
        return "model"

    register_architecture("ToyForCausalLM", Cfg, build)
    try:
        cfg = config_from_dict(dict(A, architectures=["ToyForCausalLM"]))
        assert type(cfg) is Cfg and build_model(cfg) == "model" and made["cfg"] is cfg
        with pytest.raises(KeyError):
            register_architecture("ToyForCausalLM", Cfg, build)
    finally:
        unregister_architecture("ToyForCausalLM")


def test_round_trip_through_config_json():
    for spec in helpers.TINY.values():
        cfg = config_from_dict(spec["config"])
        again = config_from_dict(cfg.to_json_dict())
        assert again.to_json_dict() == cfg.to_json_dict() and again.ffn_dim == cfg.ffn_dim


def test_model_is_assembled_layer_by_layer():
    from zinfer_b200.parts import GqaAttention, ShortConv
    m = build_model(config_from_dict(C))
    kinds = [type(l.mixer) for l in m.layers]
    assert kinds == [GqaAttention, ShortConv, GqaAttention, GqaAttention, ShortConv]
    assert [l.mixer.window for l in m.layers if isinstance(l.mixer, GqaAttention)] == [24, 0, 24]
    specs = m.cache_specs()
    assert specs[0].kv.window == 24 and specs[2].kv.window == 0 and specs[1].state.shape == (1, 80)
