"""Configuration and registry (no GPU)."""
import copy

import pytest

import helpers
from llama_rs_metal_b200.config import LlamaConfig
from llama_rs_metal_b200.errors import InvalidError, UnsupportedError
from llama_rs_metal_b200.registry import find_architecture, register_architecture


def cfg(**changes):
    out = copy.deepcopy(helpers.TINY["B"]["config"])
    out.update(changes)
    return out


def test_reads_every_key_of_config_b():
    c = LlamaConfig.from_dict(cfg())
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (96, 256, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 1, 32)
    assert (c.vocab_size, c.max_position_embeddings) == (512, 256)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0 and not c.tie_word_embeddings
    s = c.rope_scaling
    assert (s.kind, s.factor, s.low_freq_factor, s.high_freq_factor,
            s.original_max_position_embeddings) == ("llama3", 8.0, 1.0, 4.0, 64)
    assert c.rotary_dim == 32


def test_defaults_follow_the_reference():
    d = cfg()
    for key in ("head_dim", "num_key_value_heads", "rms_norm_eps", "rope_theta", "rope_scaling",
                "tie_word_embeddings", "max_position_embeddings"):
        d.pop(key)
    c = LlamaConfig.from_dict(d)
    assert c.head_dim == 96 // 3 and c.num_key_value_heads == 3
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0
    assert c.rope_scaling.kind == "default" and c.tie_word_embeddings is False
    assert c.max_position_embeddings == 8192


def test_round_trip_through_to_dict():
    for name in helpers.TINY:
        c = LlamaConfig.from_dict(helpers.TINY[name]["config"])
        assert LlamaConfig.from_dict(c.to_dict()) == c


def test_text_config_nesting_and_rope_parameters():
    inner = cfg()
    inner["rope_parameters"] = dict(inner.pop("rope_scaling"), rope_theta=1234.0)
    c = LlamaConfig.from_dict({"model_type": "llama", "text_config": inner})
    assert c.rope_theta == 1234.0 and c.rope_scaling.kind == "llama3"


@pytest.mark.parametrize("key", ["hidden_size", "num_attention_heads", "num_hidden_layers",
                                 "vocab_size", "intermediate_size"])
def test_missing_required_key_names_it(key):
    d = cfg()
    d.pop(key)
    with pytest.raises(InvalidError, match=f"missing config.{key}"):
        LlamaConfig.from_dict(d)


@pytest.mark.parametrize("changes", [
    dict(num_key_value_heads=2),            # 3 heads are no multiple of 2
    dict(num_hidden_layers=0), dict(num_hidden_layers=2000), dict(head_dim=1024),
    dict(rms_norm_eps=0.0), dict(rope_theta=-1.0), dict(vocab_size=0),
    dict(partial_rotary_factor=0.55),       # odd rotary width
    dict(hidden_size=2_000_000),
    dict(rope_scaling=dict(rope_type="llama3", factor=8.0)),  # original_max missing
    dict(rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=4.0, high_freq_factor=1.0,
                           original_max_position_embeddings=64)),
    dict(rope_scaling=dict(rope_type="linear", factor=0.0)),
    dict(max_position_embeddings=0),
])
def test_invalid_values_are_rejected(changes):
    with pytest.raises(InvalidError):
        LlamaConfig.from_dict(cfg(**changes))


@pytest.mark.parametrize("changes", [
    dict(attention_bias=True), dict(mlp_bias=True), dict(sliding_window=128),
    dict(hidden_act="gelu"), dict(rope_scaling=dict(rope_type="yarn", factor=2.0)),
    dict(layer_types=["full_attention", "linear_attention", "full_attention"]),
])
def test_unsupported_options_are_rejected(changes):
    with pytest.raises(UnsupportedError):
        LlamaConfig.from_dict(cfg(**changes))


def test_rotary_pairing_follows_rope_traditional():
    assert LlamaConfig.from_dict(cfg()).rope_adjacent_pairs is False
    adjacent = LlamaConfig.from_dict(cfg(rope_traditional=True))
    assert adjacent.rope_adjacent_pairs is True and adjacent.to_dict()["rope_traditional"] is True
    assert LlamaConfig.from_dict(adjacent.to_dict()) == adjacent
    from llama_rs_metal_b200.parts.rope import RotaryEmbedding
    assert RotaryEmbedding(12, 8, 10000.0, adjacent_pairs=True).head_permutation() == \
        [0, 2, 4, 6, 1, 3, 5, 7, 8, 9, 10, 11]
    assert RotaryEmbedding(12, 8, 10000.0).head_permutation() is None


def test_eos_ids_int_or_list():
    assert LlamaConfig.from_dict(cfg(eos_token_id=7)).eos_token_ids == (7,)
    assert LlamaConfig.from_dict(cfg(eos_token_id=[7, 9])).eos_token_ids == (7, 9)
    assert LlamaConfig.from_dict(cfg()).eos_token_ids == ()


def test_registry_finds_llama_by_architecture_or_model_type():
    assert find_architecture(cfg()).name == "LlamaForCausalLM"
    d = cfg()
    d.pop("architectures")
    assert find_architecture(d).name == "LlamaForCausalLM"
    with pytest.raises(UnsupportedError, match="registered: .*LlamaForCausalLM"):
        find_architecture({"architectures": ["MambaForCausalLM"], "model_type": "mamba"})
    with pytest.raises(InvalidError):
        find_architecture({})


def test_plan_takes_every_size_from_the_configuration():
    arch = find_architecture(cfg())
    for name in helpers.TINY:
        c = arch.config_class.from_dict(helpers.TINY[name]["config"])
        plan = arch.plan(c)
        assert len(plan.layers) == c.num_hidden_layers == len(plan.schedule)
        mixer = plan.layers[0].mixer
        assert mixer.kind == "attention" and mixer.params["num_kv_heads"] == c.num_key_value_heads
        assert mixer.params["position"].params["theta"] == c.rope_theta
        assert plan.layers[0].feed_forward.params["intermediate_size"] == c.intermediate_size
        assert plan.final_norm.params["eps"] == c.rms_norm_eps
        assert (plan.head_name is None) == c.tie_word_embeddings


def test_another_architecture_can_be_registered():
    calls = []

    class OtherConfig:
        @classmethod
        def from_dict(cls, d):
            calls.append(d)
            return cls()

    register_architecture("OtherForCausalLM", OtherConfig, lambda c: None, model_types=("other",))
    assert find_architecture({"architectures": ["OtherForCausalLM"]}).config_class is OtherConfig
    assert find_architecture({"model_type": "other"}).name == "OtherForCausalLM"
