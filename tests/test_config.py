"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

import helpers as H
from dinfer_b200.config.engine_config import EngineConfig
from dinfer_b200.config.model_config import ConfigError, Qwen3Config
from dinfer_b200.config.registry import (register_architecture, registered_architectures,
                                         resolve_architecture, unregister_architecture)
from dinfer_b200.models.qwen3 import qwen3_spec


def test_reads_every_key():
    for cfg in (H.TINY_A, H.TINY_B, H.TINY_C):
        c = Qwen3Config.from_dict(cfg)
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "max_position_embeddings"):
            assert getattr(c, k) == cfg[k]
        assert c.q_size == cfg["num_attention_heads"] * cfg["head_dim"]
        assert c.group_size == cfg["num_attention_heads"] // cfg["num_key_value_heads"]
    assert Qwen3Config.from_dict(H.TINY_A).eos_token_ids == (7,)
    assert Qwen3Config.from_dict(H.TINY_B).eos_token_ids == (3, 5)
    assert Qwen3Config.from_dict(H.TINY_C).eos_token_ids == ()
    assert Qwen3Config.from_dict(H.TINY_A).tie_word_embeddings is True
    assert Qwen3Config.from_dict(H.TINY_C).tie_word_embeddings is False      # default


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "head_dim", "rms_norm_eps",
                                 "rope_theta", "max_position_embeddings"])
def test_no_default_for_sizes(key):
    d = copy.deepcopy(H.TINY_B)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
    ({"use_sliding_window": True}, "sliding window"), ({"num_key_value_heads": 4}, "divisible"),
    ({"head_dim": 31}, "even"), ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"vocab_size": "many"}, "integer"), ({"num_hidden_layers": 0}, "positive"),
])
def test_refusals(patch, word):
    d = copy.deepcopy(H.TINY_B)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(d)


def test_round_trip_through_json():
    c = Qwen3Config.from_dict(H.TINY_B)
    assert Qwen3Config.from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_registry_resolves_by_name():
    arch = resolve_architecture(H.TINY_A)
    assert arch.name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError, match="not registered.*Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["NoSuchModel"]})
    with pytest.raises(ConfigError, match="architectures"):
        resolve_architecture({})
    register_architecture("ToyForTest", Qwen3Config.from_dict, qwen3_spec)
    try:
        assert "ToyForTest" in registered_architectures()
        d = dict(H.TINY_A, architectures=["ToyForTest"])
        assert resolve_architecture(d).name == "ToyForTest"
        with pytest.raises(ValueError):
            register_architecture("ToyForTest", Qwen3Config.from_dict, qwen3_spec)
    finally:
        unregister_architecture("ToyForTest")


def test_spec_follows_config():
    for cfg in (H.TINY_A, H.TINY_B):
        c = Qwen3Config.from_dict(cfg)
        s = qwen3_spec(c)
        assert len(s.layers) == c.num_hidden_layers and [e.layer for e in s.schedule] == list(range(len(s.layers)))
        m = s.layers[-1].mixer.params
        assert (m["num_heads"], m["num_kv_heads"], m["head_dim"], m["eps"]) == (
            c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.rms_norm_eps)
        assert m["position"].params["theta"] == c.rope_theta
        assert s.layers[0].feed_forward.params["intermediate_size"] == c.intermediate_size
        assert s.tie_word_embeddings == c.tie_word_embeddings and s.vocab_size == c.vocab_size


def test_engine_config_checks():
    EngineConfig().check()
    for bad in (dict(dtype="float16"), dict(block_size=0), dict(max_num_seqs=0), dict(gpu_memory_utilization=1.5),
                dict(max_model_len=1), dict(num_blocks=0)):
        with pytest.raises(ValueError):
            EngineConfig(**bad).check()


def test_generation_config_adds_eos_ids(tmp_path):
    import json
    from dinfer_b200.config.model_config import Qwen3Config, read_config_json
    import helpers as H
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(dict(H.TINY_A)))                     # eos_token_id 7
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": [7, 11], "temperature": 0.6}))
    cfg = Qwen3Config.from_dict(read_config_json(str(d)))
    assert list(cfg.eos_token_ids) == [7, 11]
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": "x"}))
    with pytest.raises(Exception):
        read_config_json(str(d))


def test_sampling_defaults_of_a_model_folder(tmp_path):
    """temperature, top_p and top_k of generation_config.json stand in for the built-in defaults
    (models/qwen3/src/service.rs:477-493); other keys, a broken file or no file change nothing."""
    import json
    from dinfer_b200.sampling.params import SamplingParams, generation_defaults
    assert generation_defaults(None) == SamplingParams()
    assert generation_defaults(str(tmp_path)) == SamplingParams()
    (tmp_path / "generation_config.json").write_text(json.dumps(
        {"temperature": 0.6, "top_p": 0.95, "top_k": 20, "do_sample": True, "eos_token_id": [1, 2], "max_new_tokens": 9}))
    sp = generation_defaults(str(tmp_path))
    assert (sp.temperature, sp.top_p, sp.top_k) == (0.6, 0.95, 20) and sp.max_tokens == SamplingParams().max_tokens
    sp.validate()
    (tmp_path / "generation_config.json").write_text(json.dumps({"top_k": 0, "temperature": True}))
    sp = generation_defaults(str(tmp_path))
    assert sp.top_k == -1 and sp.temperature == SamplingParams().temperature
    (tmp_path / "generation_config.json").write_text("{ not json")
    assert generation_defaults(str(tmp_path)) == SamplingParams()
