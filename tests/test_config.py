"""Configuration and registry (no device needed)."""
import json

from dataclasses import replace

import pytest

from tiny import CONFIGS, TINY_A, TINY_B
from torchless_rs_b200.config import (ConfigError, LayerSpec, MistralConfig, ModelSpec, PartSpec,
                                      UnknownArchitectureError, architecture_names,
                                      config_from_dict, load_config, register_architecture)


def test_reads_every_key():
    c = config_from_dict(TINY_A)
    assert isinstance(c, MistralConfig)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (64, 176, 2)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (4, 2, 16)
    assert (c.vocab_size, c.rope_theta, c.sliding_window, c.rms_norm_eps) == (256, 1e4, 16, 1e-5)
    b = config_from_dict(TINY_B)
    assert b.sliding_window is None and b.head_dim == 32 and b.rms_norm_eps == 1e-6


def test_defaults_follow_the_reference():
    d = {"model_type": "mistral", "hidden_size": 64, "intermediate_size": 128,
         "num_hidden_layers": 1, "num_attention_heads": 4, "vocab_size": 100}
    c = config_from_dict(d)
    assert c.num_key_value_heads == 4          # defaults to the number of heads
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5
    assert c.max_position_embeddings == 4096 and c.sliding_window is None
    d["layer_norm_eps"] = 1e-3
    assert config_from_dict(d).rms_norm_eps == 1e-3


def test_head_dim_may_differ_from_hidden_over_heads():
    c = config_from_dict(CONFIGS["C"])
    assert c.head_dim == 48 and c.hidden_size // c.num_attention_heads != 48
    spec = c.model_spec()
    assert spec.layers[0].mixer.params["head_dim"] == 48


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "vocab_size"])
def test_missing_required_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 24}, "head_dim"),
    ({"head_dim": 512}, "head_dim"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"tie_word_embeddings": True}, "tie_word_embeddings"),
    ({"hidden_size": "64"}, "integer"), ({"rope_theta": -1}, "rope_theta"),
    ({"vocab_size": 0}, "vocab_size"), ({"eos_token_id": 999}, "vocabulary"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"hidden_size": 66}, "head_dim"),
])
def test_bad_values_are_refused(patch, word):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_registry_hit_miss_and_aliases():
    assert "mistralforcausallm" in architecture_names()
    for name in ({"architectures": ["MistralForCausalLM"]}, {"model_type": "mistral"},
                 {"model_type": "mistralai"}):
        d = {k: v for k, v in TINY_A.items() if k not in ("architectures", "model_type")}
        d.update(name)
        assert isinstance(config_from_dict(d), MistralConfig)
    d = dict(TINY_A, architectures=["NoSuchModel"])
    with pytest.raises(UnknownArchitectureError, match="NoSuchModel.*known:.*mistral"):
        config_from_dict(d)
    d = {k: v for k, v in TINY_A.items() if k not in ("architectures", "model_type")}
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict(d)


def test_another_architecture_can_be_registered():
    @register_architecture("ToyForCausalLM")
    class ToyConfig(MistralConfig):
        pass
    d = dict(TINY_A, architectures=["ToyForCausalLM"])
    assert type(config_from_dict(d)).__name__ == "ToyConfig"


def test_round_trip_through_config_json(tmp_path):
    c = config_from_dict(CONFIGS["C"])
    with open(tmp_path / "config.json", "w") as f:
        json.dump(c.to_dict(), f)
    assert load_config(str(tmp_path)) == c
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path / "nowhere"))
    (tmp_path / "bad").mkdir()
    (tmp_path / "bad" / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path / "bad"))


def test_layers_are_chosen_one_by_one():
    d = dict(TINY_A, layer_types=["sliding_attention", "full_attention"])
    spec = config_from_dict(d).model_spec()
    assert spec.layers[0].mixer.params["window"] == 16
    assert spec.layers[1].mixer.params["window"] is None
    assert list(spec.order) == [0, 1]


def test_spec_validation_of_order_and_shared_caches():
    c = config_from_dict(TINY_A)
    base = c.model_spec()
    L = list(base.layers)

    def with_(layers=None, order=None):
        return ModelSpec(base.hidden_size, base.vocab_size, base.embedding_name, base.head_name,
                         False, base.final_norm, base.final_norm_prefix,
                         tuple(layers or L), tuple(order or base.order))
    with_(order=[0, 1, 0]).validate()                      # a layer may run twice
    with pytest.raises(ConfigError, match="order"):
        with_(order=[0, 2]).validate()
    shared = replace(L[1], cache_from=0)
    with_(layers=[L[0], shared]).validate()
    with pytest.raises(ConfigError, match="before"):
        with_(layers=[L[0], shared], order=[1, 0]).validate()
    bad = replace(L[1], cache_from=5)
    with pytest.raises(ConfigError, match="does not exist"):
        with_(layers=[L[0], bad]).validate()
    # a reader may not look further back than the owner of the cache keeps keys
    wide = replace(L[1], cache_from=0, mixer=PartSpec("attention", {**L[1].mixer.params, "window": None}))
    with pytest.raises(ConfigError, match="window"):
        with_(layers=[L[0], wide]).validate()
    narrow = replace(L[1], cache_from=0, mixer=PartSpec("attention", {**L[1].mixer.params, "window": 8}))
    with_(layers=[L[0], narrow]).validate()


def test_tensor_names_and_norm_roles_are_data():
    from torchless_rs_b200.engine.model import expected_tensors
    base = config_from_dict(TINY_A).model_spec()
    L = list(base.layers)
    assert L[0].tensor_prefix("mixer") == "model.layers.0.self_attn"
    assert L[1].tensor_prefix("feed_forward_norm") == "model.layers.1.post_attention_layernorm"
    renamed = [replace(l, prefix=f"h.{i}", names={"mixer_norm": "ln_1", "mixer": "attn",
                                                   "feed_forward_norm": "ln_2", "feed_forward": "ffn"})
               for i, l in enumerate(L)]
    spec = replace(base, layers=tuple(renamed), embedding_name="wte.weight", head_name="out.weight",
                   final_norm_prefix="ln_f")
    names = expected_tensors(spec)
    assert "h.1.attn.q_proj.weight" in names and "h.0.ln_2.weight" in names and "h.0.ffn.down_proj.weight" in names
    assert "wte.weight" in names and "ln_f.weight" in names and not any(n.startswith("model.") for n in names)
    # a layer that does not name one of its parts, or gives norms its block does not take
    with pytest.raises(ConfigError, match="no tensor name"):
        replace(base, layers=(replace(L[0], names={"mixer": "a", "feed_forward": "m"}), L[1])).validate()
    with pytest.raises(ConfigError, match="takes the norms"):
        expected_tensors(replace(base, layers=(replace(L[0], norms={"mixer_norm": L[0].norms["mixer_norm"]}), L[1])))
    # the hooks before the first layer and after the head
    with pytest.raises(ConfigError, match="max_positions"):
        replace(base, position_table_name="wpe.weight").validate()
    with pytest.raises(ConfigError, match="logit_softcap"):
        replace(base, logit_softcap=0.0).validate()
    table = replace(base, position_table_name="wpe.weight", max_positions=128)
    assert expected_tensors(table)["wpe.weight"].shape == (128, base.hidden_size)
