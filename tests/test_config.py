"""Typed configuration, the architecture registry and the model description (CPU)."""

import json

import pytest

import tiny
from mini_infer_b200.config import (ConfigError, Qwen2MoeConfig, UnknownArchitecture, UnknownPart,
                                    build_model_spec, known_architectures, part_class, read_config_json)
from mini_infer_b200.config.spec import ScheduleEntry
import dataclasses


def test_round_trip_and_defaults(tmp_path):
    c = Qwen2MoeConfig.from_json_dict(tiny.CONFIG_B)
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (96, 4, 1, 24)
    assert c.mlp_only_layers == (0,) and c.decoder_sparse_step == 2 and c.tie_word_embeddings
    c.save(str(tmp_path))
    again = Qwen2MoeConfig.from_json_dict(read_config_json(str(tmp_path)))
    assert again == c
    # defaults of the reference's parser (src/model/model_config.cpp:68-112)
    d = Qwen2MoeConfig.from_json_dict({"architectures": ["Qwen2MoeForCausalLM"], "hidden_size": 32,
                                       "num_hidden_layers": 1, "num_attention_heads": 2, "vocab_size": 10,
                                       "intermediate_size": 8})
    assert d.num_key_value_heads == 2 and d.rms_norm_eps == 1e-6 and d.rope_theta == 10000.0
    assert d.max_position_embeddings == 32768 and not d.tie_word_embeddings and d.num_experts == 0


def test_tolerant_number_forms():
    j = dict(tiny.CONFIG_A, hidden_size="64", rms_norm_eps="1e-6", num_hidden_layers=2.0)
    c = Qwen2MoeConfig.from_json_dict(j)
    assert c.hidden_size == 64 and c.num_hidden_layers == 2 and c.rms_norm_eps == 1e-6


def test_number_of_experts_under_its_other_names():
    """The reference takes the first of num_experts, num_local_experts, n_routed_experts that is not zero
    (src/model/model_config.cpp:95-105)."""
    j = {k: v for k, v in tiny.CONFIG_B.items() if k != "num_experts"}
    n = tiny.CONFIG_B["num_experts"]
    assert Qwen2MoeConfig.from_json_dict(dict(j, num_local_experts=n)).num_experts == n
    assert Qwen2MoeConfig.from_json_dict(dict(j, n_routed_experts=n)).num_experts == n
    assert Qwen2MoeConfig.from_json_dict(dict(j, num_experts=n, num_local_experts=n + 1)).num_experts == n


def test_sparse_and_window_rules():
    b = Qwen2MoeConfig.from_json_dict(tiny.CONFIG_B)
    assert [b.layer_is_sparse(i) for i in range(3)] == [False, True, False]
    a = Qwen2MoeConfig.from_json_dict(tiny.CONFIG_A)
    assert all(a.layer_is_sparse(i) for i in range(2)) and a.layer_window(1) == 0
    c = Qwen2MoeConfig.from_json_dict(tiny.CONFIG_C)
    assert [c.layer_window(i) for i in range(4)] == [0, 0, 24, 24]
    assert [c.layer_is_sparse(i) for i in range(4)] == [True, True, False, True]


@pytest.mark.parametrize("patch,needle", [
    ({"hidden_size": 0}, "missing required"),
    ({"vocab_size": None}, "missing required"),
    ({"num_attention_heads": 5}, "not divisible by num_attention_heads"),
    ({"num_key_value_heads": 3}, "not divisible by num_key_value_heads"),
    ({"num_experts_per_tok": 9}, "num_experts_per_tok"),
    ({"decoder_sparse_step": 0}, "decoder_sparse_step"),
    ({"mlp_only_layers": [7]}, "mlp_only_layers"),
    ({"moe_intermediate_size": 0, "intermediate_size": 0}, "moe_intermediate_size"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"head_dim": 15}, "even"),
    ({"use_sliding_window": True, "sliding_window": 0}, "sliding_window"),
    ({"hidden_size": "many"}, "must be an integer"),
    ({"tie_word_embeddings": "perhaps"}, "must be a boolean"),
])
def test_validation_errors(patch, needle):
    j = dict(tiny.CONFIG_A)
    j.update(patch)
    with pytest.raises(ConfigError, match=needle):
        Qwen2MoeConfig.from_json_dict(j)


def test_dense_layers_need_intermediate_size():
    j = dict(tiny.CONFIG_B, intermediate_size=0)
    with pytest.raises(ConfigError, match="dense layers need"):
        Qwen2MoeConfig.from_json_dict(j)


def test_cannot_open(tmp_path):
    with pytest.raises(ConfigError, match="cannot open"):
        read_config_json(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))


def test_registry():
    assert "Qwen2MoeForCausalLM" in known_architectures()
    with pytest.raises(UnknownArchitecture, match="LlamaForCausalLM.*Qwen2MoeForCausalLM"):
        build_model_spec(dict(tiny.CONFIG_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        build_model_spec({k: v for k, v in tiny.CONFIG_A.items() if k != "architectures"})
    with pytest.raises(UnknownPart, match="no mixer part of kind 'convolution'"):
        part_class("mixer", "convolution")


def test_spec_is_chosen_layer_by_layer():
    spec = build_model_spec(tiny.CONFIG_B)
    assert [l.feed_forward.kind for l in spec.layers] == ["swiglu_mlp", "sparse_moe", "swiglu_mlp"]
    assert spec.lm_head.get("tied_to") == "model.embed_tokens.weight"
    assert spec.layers[1].feed_forward.get("top_k") == 3 and not spec.layers[1].feed_forward.get("norm_topk_prob")
    spec_c = build_model_spec(tiny.CONFIG_C)
    assert [l.mixer.get("window") for l in spec_c.layers] == [0, 0, 24, 24]
    assert spec_c.layers[0].mixer.get("position").get("theta") == 50000.0
    assert not spec_c.layers[0].mixer.get("bias")


def test_schedule_validation():
    spec = build_model_spec(tiny.CONFIG_A)
    twice = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                                                ScheduleEntry(1, cache_from=1)))
    twice.validate()
    with pytest.raises(ValueError, match="earlier schedule position"):
        dataclasses.replace(spec, schedule=(ScheduleEntry(0, cache_from=0),)).validate()
    with pytest.raises(ValueError, match="names layer 5"):
        dataclasses.replace(spec, schedule=(ScheduleEntry(5),)).validate()


def test_schedule_plans_caches():
    """A layer named twice gets a cache per run; an entry with cache_from shares its source's."""
    from mini_infer_b200.engine.model import Model
    spec = build_model_spec(tiny.CONFIG_C)
    m = Model(spec)
    assert len(m.kv_groups) == 2                       # full-history layers and windowed layers
    assert {g.window for g in m.kv_groups} == {0, 24}
    twice = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                                                ScheduleEntry(1, cache_from=1)))
    m2 = Model(twice)
    assert [b["mixer"].layer_slot for b in m2.bindings] == [0, 1, 2, 1]
    assert [b["mixer"].writes for b in m2.bindings] == [True, True, True, False]
    assert m2.kv_groups[0].num_layers == 3


@pytest.mark.parametrize("name", sorted(tiny.CONFIGS))
def test_agrees_with_the_reference_parser_on_the_keys_it_reads(name):
    """tests/golden/reference_config_<name>.json is what the reference's own parser
    (src/model/model_config.cpp:61-178, compiled on the host by tests/golden/make_config_golden.py)
    reads from the same config.json.  It never reads norm_topk_prob, decoder_sparse_step,
    mlp_only_layers or use_sliding_window, and it keeps sliding_window whatever
    use_sliding_window says (src/model/model_config.cpp:153); those are ours alone."""
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "golden", f"reference_config_{name}.json")) as f:
        ref = json.load(f)
    cfg = Qwen2MoeConfig.from_json_dict(tiny.CONFIGS[name])
    for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "vocab_size", "max_position_embeddings", "tie_word_embeddings",
                "hidden_act", "num_experts", "num_experts_per_tok", "moe_intermediate_size",
                "shared_expert_intermediate_size", "sliding_window"):
        assert getattr(cfg, key) == ref[key], key
    raw = tiny.CONFIGS[name]
    # the reference takes head_dim = hidden_size / heads for this family (it reads the key for Gemma only,
    # src/model/model_config.cpp:117) and decides the bias by the architecture's name (:146-151); a
    # config.json that states either gets its way here
    if "head_dim" not in raw:
        assert cfg.head_dim == ref["head_dim"]
    else:
        assert ref["head_dim"] == raw["hidden_size"] // raw["num_attention_heads"]
    if "qkv_bias" not in raw:
        assert cfg.qkv_bias == ref["has_qkv_bias"]
    assert abs(cfg.rms_norm_eps - ref["rms_norm_eps"]) <= 1e-7 * ref["rms_norm_eps"] + 1e-12   # float in the reference
    assert abs(cfg.rope_theta - ref["rope_theta"]) <= 1e-6 * ref["rope_theta"]
    assert ref["is_moe"] == (cfg.num_experts > 0 and cfg.num_experts_per_tok > 0)
