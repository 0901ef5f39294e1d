"""Configuration and registry (no GPU)."""
import json

import numpy as np
import pytest

import helpers
from hymt2sharp_b200.config import (ConfigError, HunyuanDenseConfig, get_architecture, known_architectures,
                                    load_config)


def test_reads_every_key_and_defaults():
    cfg = HunyuanDenseConfig.from_dict(helpers.CONFIGS["B"]["config"])
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 6, 1)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (32, 224, 509)
    assert cfg.q_size == 192 and cfg.kv_size == 32 and cfg.rope_dim == 32
    assert cfg.rms_norm_eps == 1e-6 and not cfg.use_qk_norm and not cfg.tie_word_embeddings
    minimal = dict(architectures=[helpers.ARCH], num_hidden_layers=1, hidden_size=32, num_attention_heads=2,
                   intermediate_size=48, vocab_size=10)
    d = HunyuanDenseConfig.from_dict(minimal)
    # defaults of src/HyMT2Sharp/ModelConfig.cs:26-49
    assert d.num_key_value_heads == 2 and d.head_dim == 16 and d.rope_theta == 10000.0 and d.rope_alpha == 0.0
    assert d.rms_norm_eps == 1e-5 and d.max_position_embeddings == 4096 and d.use_qk_norm and d.tie_word_embeddings
    assert HunyuanDenseConfig.from_dict({**minimal, "attention_head_dim": 24}).head_dim == 24


def test_ntk_base_in_float32():
    cfg = HunyuanDenseConfig.from_dict(helpers.CONFIGS["B"]["config"])
    # base = theta * alpha^(d/(d-2)), src/HyMT2Sharp/ModelConfig.cs:31-34
    want = np.float32(1e6) * np.float32(np.float32(1000.0) ** (np.float32(32) / np.float32(30)))
    assert cfg.rope_base == pytest.approx(float(want), rel=1e-6)
    assert HunyuanDenseConfig.from_dict(helpers.CONFIGS["A"]["config"]).rope_base == 10000.0  # alpha 1 changes nothing
    off = dict(helpers.CONFIGS["B"]["config"]); off.pop("rope_scaling")
    assert HunyuanDenseConfig.from_dict(off).rope_base == 1e6


@pytest.mark.parametrize("change, word", [
    (dict(num_hidden_layers=None), "num_hidden_layers"),
    (dict(hidden_size="64"), "hidden_size"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(rope_dim=15), "rope_dim"),
    (dict(rms_norm_eps=0), "rms_norm_eps"),
    (dict(vocab_size=0), "vocab_size"),
    (dict(use_qk_norm=1), "use_qk_norm"),
    (dict(rope_scaling={"type": "yarn", "alpha": 2.0}), "rope_scaling"),
    (dict(architectures=[]), "architectures"),
])
def test_bad_configs_name_the_key(change, word, tmp_path):
    data = {**helpers.CONFIGS["A"]["config"], **change}
    data = {k: v for k, v in data.items() if v is not None}
    (tmp_path / "config.json").write_text(json.dumps(data))
    with pytest.raises(ConfigError) as e:
        load_config(str(tmp_path))
    assert word in str(e.value)


def test_registry():
    assert helpers.ARCH in known_architectures()
    assert get_architecture(helpers.ARCH).config_class is HunyuanDenseConfig
    with pytest.raises(ConfigError) as e:
        get_architecture("NoSuchForCausalLM")
    assert helpers.ARCH in str(e.value)


def test_round_trip_through_config_json(tmp_path):
    for name in helpers.CONFIGS:
        cfg = HunyuanDenseConfig.from_dict(helpers.CONFIGS[name]["config"])
        (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
        arch, again = load_config(str(tmp_path))
        assert again == cfg and arch.name == helpers.ARCH


def test_spec_is_data(tmp_path):
    """The layers and their order are data: one part spec per layer, one order entry per run."""
    from hymt2sharp_b200.engine.spec import ModelSpec, Run
    arch = get_architecture(helpers.ARCH)
    cfg = HunyuanDenseConfig.from_dict(helpers.CONFIGS["B"]["config"])
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 3 and [r.layer for r in spec.order] == [0, 1, 2]
    assert spec.layers[1].params["mixer"].params["kv_heads"] == 1
    with pytest.raises(ValueError):
        ModelSpec(spec.vocab, spec.hidden, spec.embedding, spec.layers, spec.final_norm, spec.head,
                  order=[Run(0), Run(1, cache_from=1)])
    with pytest.raises(ValueError):
        ModelSpec(spec.vocab, spec.hidden, spec.embedding, spec.layers, spec.final_norm, spec.head, order=[Run(3)])
