"""Typed configuration and the architecture registry."""
import json

import pytest

import helpers as H
from spite_b200.config import (ConfigError, Llama4Config, ModelPlan, config_from_dict,
                               known_architectures, load_config, register_architecture)


def test_config_a_and_b_differ_in_every_size_and_option():
    a, b = Llama4Config.from_dict(H.CONFIG_A), Llama4Config.from_dict(H.CONFIG_B)
    for f in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
              "head_dim", "intermediate_size", "intermediate_size_mlp", "num_local_experts", "moe_layers",
              "no_rope_layers", "rope_theta", "rope_scaling", "attention_chunk_size", "use_qk_norm",
              "attn_temperature_tuning", "rms_norm_eps", "tie_word_embeddings"):
        assert getattr(a, f) != getattr(b, f), f


def test_layer_schedule_follows_the_intervals():
    a, b = Llama4Config.from_dict(H.CONFIG_A), Llama4Config.from_dict(H.CONFIG_B)
    assert a.moe_layers == (0, 1, 2, 3) and a.no_rope_layers == (1, 1, 1, 0)
    assert b.moe_layers == (1, 3, 5) and b.no_rope_layers == (1, 1, 0, 1, 1, 0)
    explicit = dict(H.CONFIG_B, moe_layers=[0, 5], no_rope_layers=[0, 1, 1, 1, 1, 1])
    c = Llama4Config.from_dict(explicit)
    assert c.moe_layers == (0, 5) and not c.uses_rope(0) and c.uses_rope(1)


def test_plan_chooses_parts_layer_by_layer():
    b = Llama4Config.from_dict(H.CONFIG_B)
    plan = b.plan()
    assert isinstance(plan, ModelPlan) and len(plan.blocks) == 6
    assert [blk.ffn.kind for blk in plan.blocks] == ["dense_swiglu", "moe_sigmoid_prescaled"] * 3
    windows = [blk.mixer.params["window"] for blk in plan.blocks]
    assert windows == [("chunk", 16), ("chunk", 16), ("full", 0)] * 2
    assert plan.blocks[0].mixer.params["position"].kind == "rotary_interleaved"
    assert plan.blocks[2].mixer.params["position"].kind == "no_position"
    assert plan.blocks[0].mixer.params["qk_norm_eps"] is None            # use_qk_norm off in B
    a = Llama4Config.from_dict(H.CONFIG_A).plan()
    assert a.blocks[0].mixer.params["qk_norm_eps"] == 1e-5
    assert a.blocks[3].mixer.params["temperature_tuning"] == (16.0, 0.1)
    assert a.blocks[0].mixer.params["temperature_tuning"] is None
    assert [(c.layer, c.cache, c.write_cache) for c in a.order] == [(i, i, True) for i in range(4)]
    assert plan.tie_word_embeddings and not a.tie_word_embeddings


def test_defaults_and_nesting():
    d = {k: v for k, v in H.CONFIG_A.items() if k not in ("head_dim", "rms_norm_eps", "rope_theta", "use_qk_norm")}
    c = Llama4Config.from_dict(d)
    assert c.head_dim == 16 and c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0 and c.use_qk_norm
    nested = {"architectures": ["Llama4ForConditionalGeneration"], "text_config": d, "vision_config": {"x": 1}}
    n = config_from_dict(nested)
    assert n.hidden_size == 64 and n.architecture == "Llama4ForConditionalGeneration"


def test_round_trip_through_config_json(tmp_path):
    for raw in (H.CONFIG_A, H.CONFIG_B):
        c = Llama4Config.from_dict(raw)
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        assert load_config(tmp_path) == c


@pytest.mark.parametrize("change,needle", [
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"hidden_size": 0}, "positive"),
    ({"num_experts_per_tok": 9}, "num_experts_per_tok"), ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "llama3"),
    ({"no_rope_layers": [1, 0]}, "no_rope_layers"), ({"attention_chunk_size": -1}, "attention_chunk_size"),
    ({"moe_layers": [7]}, "moe_layers"), ({"num_local_experts": 0}, "num_local_experts")])
def test_validation_errors(change, needle):
    with pytest.raises(ConfigError, match=needle):
        Llama4Config.from_dict(dict(H.CONFIG_A, **change))


def test_missing_key_and_unknown_architecture(tmp_path):
    d = dict(H.CONFIG_A)
    del d["vocab_size"]
    with pytest.raises(ConfigError, match="vocab_size"):
        Llama4Config.from_dict(d)
    with pytest.raises(ConfigError, match="Llama4ForCausalLM"):
        config_from_dict(dict(H.CONFIG_A, architectures=["NoSuchModel"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"hidden_size": 4})
    with pytest.raises(ConfigError, match="not found"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(tmp_path)


def test_registry_accepts_another_architecture():
    @register_architecture("ToyForTests")
    class Toy:
        @classmethod
        def from_dict(cls, d):
            return ("toy", d["n"])
    assert "ToyForTests" in known_architectures()
    assert config_from_dict({"architectures": ["ToyForTests"], "n": 3}) == ("toy", 3)


def test_model_type_stands_in_for_a_missing_architectures_list():
    d = {k: v for k, v in H.CONFIG_A.items() if k != "architectures"}
    assert config_from_dict(dict(d, model_type="llama4_text")) == Llama4Config.from_dict(H.CONFIG_A)
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict(dict(d, model_type="something_else"))


def test_plan_validation_of_the_run_order():
    from dataclasses import replace
    from spite_b200.config import LayerCall
    plan = Llama4Config.from_dict(H.CONFIG_A).plan()
    shared = replace(plan, order=(LayerCall(0, 0), LayerCall(1, 0, write_cache=False), LayerCall(0, 1)))
    shared.validate()                       # a layer twice, a layer reading another layer's cache
    with pytest.raises(ConfigError, match="written by two"):
        replace(plan, order=(LayerCall(0, 0), LayerCall(1, 0))).validate()
    with pytest.raises(ConfigError, match="read before"):
        replace(plan, order=(LayerCall(1, 0, write_cache=False), LayerCall(0, 0))).validate()
    with pytest.raises(ConfigError, match="names layer"):
        replace(plan, order=(LayerCall(9, 0),)).validate()
