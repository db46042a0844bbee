import json

import pytest

import citlali_b200 as cb
from helpers import TINY


def test_reads_every_size_from_config_json(tmp_path):
    for name, d in TINY.items():
        c = cb.config_from_dict(dict(d))
        assert c.vocab_size == d["vocab_size"] and c.hidden_size == d["hidden_size"]
        assert c.num_hidden_layers == d["num_hidden_layers"] and c.intermediate_size == d["intermediate_size"]
        assert c.num_attention_heads == d["num_attention_heads"] and c.num_key_value_heads == d["num_key_value_heads"]
        assert c.head_dim == d["head_dim"] and c.rms_norm_eps == d["rms_norm_eps"] and c.rope_theta == d["rope_theta"]
        assert c.max_position_embeddings == d["max_position_embeddings"]
        assert c.tie_word_embeddings == d["tie_word_embeddings"]
        # round trip through config.json
        (tmp_path / name).mkdir()
        (tmp_path / name / "config.json").write_text(json.dumps(c.to_dict()))
        assert cb.config_from_model_dir(str(tmp_path / name)) == c


def test_fallbacks_follow_the_reference():
    d = dict(TINY["A"])
    del d["head_dim"], d["num_key_value_heads"]
    c = cb.config_from_dict(d)
    assert c.head_dim == d["hidden_size"] // d["num_attention_heads"]
    assert c.num_key_value_heads == d["num_attention_heads"]
    d = dict(TINY["A"]); del d["tie_word_embeddings"]
    assert cb.config_from_dict(d).tie_word_embeddings is None


def test_eos_ids():
    assert cb.config_from_dict(dict(TINY["C"])).eos_token_ids == (5, 9)
    d = dict(TINY["A"], eos_token_id=7)
    assert cb.config_from_dict(d).eos_token_ids == (7,)
    assert cb.config_from_dict(dict(TINY["A"])).eos_token_ids == ()
    with pytest.raises(cb.CitlaliError, match="outside the vocabulary"):
        cb.config_from_dict(dict(TINY["A"], eos_token_id=512))


@pytest.mark.parametrize("change, message", [
    (dict(attention_bias=True), "attention_bias"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"type": "yarn", "factor": 4.0}), "rope_scaling"),
    (dict(use_sliding_window=True, sliding_window=64), "sliding_window"),
    (dict(num_key_value_heads=3), "not a multiple"),
    (dict(head_dim=15), "even"),
    (dict(vocab_size=0), "vocab_size"),
    (dict(hidden_size=-4), "hidden_size"),
    (dict(rms_norm_eps=0), "rms_norm_eps"),
    (dict(num_hidden_layers=2.5), "num_hidden_layers"),
])
def test_rejections_name_the_key(change, message):
    with pytest.raises(cb.CitlaliError, match=message):
        cb.config_from_dict(dict(TINY["A"], **change))


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers", "intermediate_size",
                                 "num_attention_heads", "rms_norm_eps", "rope_theta", "max_position_embeddings"])
def test_required_keys(key):
    d = dict(TINY["B"]); del d[key]
    with pytest.raises(cb.CitlaliError, match=key):
        cb.config_from_dict(d)


def test_registry_names_one_architecture_and_lists_it_on_a_miss():
    assert cb.registered_architectures() == ["Qwen3ForCausalLM"]
    with pytest.raises(cb.CitlaliError, match="unknown architecture 'LlamaForCausalLM'.*Qwen3ForCausalLM"):
        cb.config_from_dict(dict(TINY["A"], architectures=["LlamaForCausalLM"]))
    with pytest.raises(cb.CitlaliError, match="architectures"):
        cb.config_from_dict({k: v for k, v in TINY["A"].items() if k != "architectures"})


def test_model_spec_is_data():
    spec = cb.config_from_dict(dict(TINY["B"])).to_model_spec()
    assert len(spec.layers) == 3 and [s.layer for s in spec.schedule] == [0, 1, 2]
    layer = spec.layers[1]
    assert layer.block == "pre_norm_residual"
    assert list(layer.parts) == ["mixer_norm", "mixer", "feed_forward_norm", "feed_forward"]
    mixer, ff = layer.part("mixer"), layer.part("feed_forward")
    assert mixer.kind == "gqa_attention" and mixer.params["head_dim"] == 32 and mixer.params["qk_norm_eps"] == 1e-5
    assert mixer.params["position"] == {"kind": "rotary_half_split", "theta": 1e4, "rotary_dim": 32}
    assert ff.kind == "gated_silu" and ff.params["intermediate_size"] == 160
    assert mixer.prefix == "model.layers.1.self_attn" and layer.part("mixer_norm").params["eps"] == 1e-5
    assert spec.embedding_scale is None and spec.logit_scale is None
    with pytest.raises(cb.CitlaliError, match="needs a part named 'gate'.*mixer_norm, mixer"):
        layer.part("gate")


def test_schedule_validation():
    spec = cb.config_from_dict(dict(TINY["A"])).to_model_spec()
    import dataclasses
    bad = dataclasses.replace(spec, schedule=(cb.ScheduleStep(0), cb.ScheduleStep(5)))
    with pytest.raises(cb.CitlaliError, match="names layer 5"):
        bad.validate()
    bad = dataclasses.replace(spec, schedule=(cb.ScheduleStep(0, cache_of=0),))
    with pytest.raises(cb.CitlaliError, match="does not run before"):
        bad.validate()
    twice = dataclasses.replace(spec, schedule=(cb.ScheduleStep(0), cb.ScheduleStep(1), cb.ScheduleStep(0),
                                                cb.ScheduleStep(1, cache_of=1)))
    twice.validate()


def test_rope_theta_inside_rope_parameters():
    """Newer writers of config.json put the rotary base inside a rope_parameters object."""
    import helpers
    d = dict(helpers.TINY["B"])
    theta = d.pop("rope_theta")
    d["rope_parameters"] = {"rope_type": "default", "rope_theta": theta}
    assert cb.config_from_dict(d).rope_theta == theta
    d["rope_parameters"] = {"rope_type": "yarn", "rope_theta": theta, "factor": 4.0}
    with pytest.raises(cb.CitlaliError, match="rope_type 'yarn'"):
        cb.config_from_dict(d)
    d["rope_parameters"] = {"rope_type": "default"}
    with pytest.raises(cb.CitlaliError, match="rope_theta"):
        cb.config_from_dict(d)
