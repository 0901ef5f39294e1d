"""Weights by name: stored types, the one error with everything that is wrong, random mode (no GPU)."""
import json
import os

import numpy as np
import pytest
import torch

import helpers
from hymt2sharp_b200.config import load_config
from hymt2sharp_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_checkpoint,
                                     write_random_model, write_safetensors)


def _expected(folder):
    arch, cfg = load_config(folder)
    return arch.tensor_shapes(cfg)


def test_random_folder_loads_and_keeps_types(model_dirs):
    for name, gain_dtype in (("A", torch.bfloat16), ("B", torch.float32)):
        folder = model_dirs(name)
        w = load_checkpoint(folder, _expected(folder))
        assert w["model.embed_tokens.weight"].dtype == torch.bfloat16
        assert w["model.layers.0.input_layernorm.weight"].dtype == gain_dtype  # a 32-bit tensor stays 32-bit
        assert ("lm_head.weight" in w) == (name == "B")
        assert ("model.layers.0.self_attn.query_layernorm.weight" in w) == (name == "A")
        # the library `safetensors` reads the same bytes
        from safetensors.torch import load_file
        other = load_file(os.path.join(folder, "model.safetensors"))
        assert set(other) == set(w)
        for k in w:
            assert torch.equal(other[k], w[k])


def test_random_mode_is_seeded(tmp_path):
    from hymt2sharp_b200.config import HunyuanDenseConfig
    cfg = HunyuanDenseConfig.from_dict(helpers.CONFIGS["A"]["config"])
    a = write_random_model(str(tmp_path / "a"), cfg, 7, 0.02)
    b = write_random_model(str(tmp_path / "b"), cfg, 7, 0.02)
    c = write_random_model(str(tmp_path / "c"), cfg, 8, 0.02)
    wa, wb, wc = (load_checkpoint(d, _expected(d)) for d in (a, b, c))
    assert all(torch.equal(wa[k], wb[k]) for k in wa)
    assert not torch.equal(wa["model.embed_tokens.weight"], wc["model.embed_tokens.weight"])
    emb = wa["model.embed_tokens.weight"].float()
    assert abs(emb.std().item() - 0.02) < 0.002 and abs(emb.mean().item()) < 0.001
    gain = wa["model.norm.weight"].float()
    assert abs(gain.mean().item() - 1.0) < 0.02


def test_one_error_lists_everything(model_dirs, tmp_path):
    folder = model_dirs("A")
    src = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 65, dtype=torch.bfloat16)
    tensors["model.layers.9.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 160, dtype=torch.int32)
    out = tmp_path / "bad"
    out.mkdir()
    (out / "config.json").write_text(open(os.path.join(folder, "config.json")).read())
    write_safetensors(str(out / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        load_checkpoint(str(out), _expected(str(out)))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    assert [w[0] for w in err.wrong_type] == ["model.layers.0.mlp.down_proj.weight"]
    text = str(err)
    for word in ("up_proj", "model.norm.weight", "extra", "[64, 65]", "[64, 64]", "down_proj"):
        assert word in text


def test_stored_types(tmp_path):
    from hymt2sharp_b200.weights.loader import TensorSpec
    t = {"a": torch.randn(4, 4).to(torch.float16), "b": torch.randn(3, dtype=torch.float64),
         "c": torch.arange(5, dtype=torch.int64), "d": torch.randn(2, 2)}
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    w = load_checkpoint(str(tmp_path), {"a": TensorSpec((4, 4)), "b": TensorSpec((3,)),
                                        "c": TensorSpec((5,), kind="int"), "d": TensorSpec((2, 2))})
    assert w["a"].dtype == torch.bfloat16 and w["b"].dtype == torch.float32
    assert w["c"].dtype == torch.int32 and w["d"].dtype == torch.float32  # integer tables are int32
    assert torch.equal(w["c"], torch.arange(5, dtype=torch.int32))


def test_broken_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    write_safetensors(str(p), {"x": torch.zeros(1000, dtype=torch.float32)})
    data = p.read_bytes()
    p.write_bytes(data[: len(data) - 100])  # truncated
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFile(str(p))
    assert "truncated" in str(e.value)
    with pytest.raises(SafetensorsError):
        load_checkpoint(str(tmp_path / "nowhere"), {})


def test_sharded_checkpoint(model_dirs, tmp_path):
    folder = model_dirs("A")
    src = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    names = src.names()
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for fn, ns in shards.items():
        write_safetensors(str(tmp_path / fn), {n: src.tensor(n) for n in ns})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {n: fn for fn, ns in shards.items() for n in ns}}))
    (tmp_path / "config.json").write_text(open(os.path.join(folder, "config.json")).read())
    w = load_checkpoint(str(tmp_path), _expected(str(tmp_path)))
    assert all(torch.equal(w[n], src.tensor(n)) for n in names)


def test_harmless_extra_tensors_are_reported_not_refused(model_dirs, tmp_path):
    """A folder that the reference would run (it looks its tensors up by name) may hold a recomputed rotary buffer
    and, with a tied head, the head once more under its own name: both are left unread with a warning.  A head copy
    with OTHER values, and any other extra tensor, stay errors."""
    from hymt2sharp_b200.engine.hunyuan_dense import build_spec
    folder = model_dirs("A")   # tie_word_embeddings is set
    arch, cfg = load_config(folder)
    src = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    (tmp_path / "config.json").write_text(open(os.path.join(folder, "config.json")).read())
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    ignorable = build_spec(cfg).ignorable_tensors
    with pytest.warns(RuntimeWarning, match="not read") as rec:
        w = load_checkpoint(str(tmp_path), _expected(str(tmp_path)), ignorable)
    assert "inv_freq" in str(rec[0].message) and "lm_head.weight (a copy of model.embed_tokens.weight)" in str(rec[0].message)
    assert "lm_head.weight" not in w and set(w) == set(src.names())
    with pytest.raises(WeightError) as e:     # without the architecture's say-so the buffer is unexpected
        load_checkpoint(str(tmp_path), _expected(str(tmp_path)))
    assert e.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    tensors["lm_head.weight"][3, 5] += 1.0
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightError, match="holds other values"):
        load_checkpoint(str(tmp_path), _expected(str(tmp_path)), ignorable)


def test_index_that_names_the_wrong_shard(model_dirs, tmp_path):
    folder = model_dirs("A")
    src = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    names = src.names()
    shards = {"a.safetensors": names[:5], "b.safetensors": names[5:]}
    for fn, ns in shards.items():
        write_safetensors(str(tmp_path / fn), {n: src.tensor(n) for n in ns})
    weight_map = {n: fn for fn, ns in shards.items() for n in ns}
    weight_map[names[0]] = "b.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    (tmp_path / "config.json").write_text(open(os.path.join(folder, "config.json")).read())
    with pytest.raises(WeightError, match="which does not hold it"):
        load_checkpoint(str(tmp_path), _expected(str(tmp_path)))
