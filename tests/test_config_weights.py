"""Configuration, registry and weights on the CPU.  Where tamnd/fastmlx ships JSON fixtures
of its own parsers (compute/testdata/*.json) they are read in place, as data, when that
checkout is present; nothing of them is copied here."""
import json
import os
import struct

import pytest
import torch

import tiny
from fastmlx_b200 import registry
from fastmlx_b200.config import ConfigError, LlamaConfig
from fastmlx_b200.weights import WeightError, load_checkpoint, shard_files, write_random_model
from fastmlx_b200.weights import safetensors_io as st

REF = tiny.reference_dir()
needs_ref = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "compute", "testdata")),
                               reason="the reference checkout is not present")


def test_defaults_follow_the_reference_parser():
    c = LlamaConfig.from_dict({"model_type": "llama", "hidden_size": 64, "num_hidden_layers": 2,
                               "intermediate_size": 128, "num_attention_heads": 4, "vocab_size": 100})
    assert (c.head_dim, c.num_key_value_heads, c.rope_theta, c.tie_word_embeddings) == (16, 4, 10000.0, True)
    assert c.rope_scaling is None and not c.attention_bias and not c.mlp_bias and c.eos_token_id == -1
    assert c.scale == 0.25 and c.q_proj_out == 64 and c.kv_proj_out == 64 and c.gqa_repeat == 1


@pytest.mark.parametrize("patch,word", [
    ({"num_attention_heads": 0}, "num_attention_heads"), ({"hidden_size": 0}, "hidden_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"), ({"vocab_size": 0}, "vocab_size"),
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"intermediate_size": 0}, "intermediate"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2}}, "rope_scaling"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8}}, "low_freq_factor"),
    ({"quantization": {"group_size": 64, "bits": 4}}, "quantiz"), ({"hidden_size": "big"}, "integer")])
def test_config_errors_name_the_key(patch, word):
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict({**tiny.TINY_A, **patch})


def test_eos_may_be_an_int_or_a_list_and_config_round_trips():
    assert LlamaConfig.from_dict({**tiny.TINY_A, "eos_token_id": 7}).eos_token_id == 7
    c = LlamaConfig.from_dict({**tiny.TINY_B, "eos_token_id": [5, 6]})
    assert c.eos_token_id == 5 and c.eos_token_ids == (5, 6)
    assert LlamaConfig.from_dict(json.loads(c.to_json())) == c


def test_registry_resolves_by_model_type_and_by_architecture():
    assert registry.resolve({"model_type": "llama"}).name == "llama"
    assert registry.resolve({"architectures": ["LlamaForCausalLM"]}).name == "llama"
    assert "llama" in registry.registered_model_types()
    with pytest.raises(ConfigError, match="unsupported model_type 'mamba'"):
        registry.resolve({"model_type": "mamba"})
    with pytest.raises(ConfigError, match="no model_type"):
        registry.resolve({})


@needs_ref
def test_reference_fixture_args():
    with open(os.path.join(REF, "compute", "testdata", "llama_args.json")) as f:
        fx = json.load(f)
    for case in fx["args"]:
        c = LlamaConfig.from_dict(case["config"])
        for key, want in case["expected"].items():
            if key == "rope_scaling":
                continue
            assert getattr(c, key) == want, (case["label"], key)
    for case in fx["weight_names"]:
        _, model = registry.build_model(case["config"])
        assert sorted(s.name for s in model.weight_specs()) == case["names"], case["label"]


@needs_ref
def test_reference_fixture_safetensors_headers():
    import base64
    with open(os.path.join(REF, "compute", "testdata", "safetensors_header.json")) as f:
        fx = json.load(f)
    cases = fx["cases"] if isinstance(fx, dict) else fx
    checked = 0
    for case in cases:
        if "blob_b64" not in case or "truth" not in case:
            continue
        infos, meta, base = st.parse_header(base64.b64decode(case["blob_b64"]))
        truth = case["truth"]
        assert base == truth["data_start"], case["label"]
        assert [(t.name, t.dtype, list(t.shape), t.begin, t.end) for t in infos] == \
            [(w["name"], w["dtype"], list(w["shape"]), w["begin"], w["end"]) for w in truth["tensors"]], case["label"]
        assert (meta or None) == (truth.get("metadata") or None), case["label"]
        checked += 1
    assert checked


def test_random_model_folder_round_trip_and_determinism(tmp_path):
    d1 = write_random_model(str(tmp_path / "a"), tiny.TINY_B, seed=5)
    d2 = write_random_model(str(tmp_path / "b"), tiny.TINY_B, seed=5, max_shard_bytes=300_000)
    d3 = write_random_model(str(tmp_path / "c"), tiny.TINY_B, seed=6)
    assert os.path.exists(os.path.join(d1, "model.safetensors")) and os.path.exists(os.path.join(d1, "config.json"))
    assert len(shard_files(d2)) > 1 and os.path.exists(os.path.join(d2, st.INDEX_NAME))
    c1, w1 = load_checkpoint(d1)
    c2, w2 = load_checkpoint(d2)
    _, w3 = load_checkpoint(d3)
    assert c1 == c2 == tiny.TINY_B and sorted(w1) == sorted(w2)
    for n in w1:
        assert w1[n].dtype == torch.bfloat16 and torch.equal(w1[n], w2[n])          # values do not depend on sharding
    assert not torch.equal(w1["model.norm.weight"], w3["model.norm.weight"])
    assert abs(w1["model.norm.weight"].float().mean().item() - 1.0) < 0.02
    assert abs(w1["model.embed_tokens.weight"].float().std().item() - 0.02) < 0.002
    # the safetensors library reads the same values
    from safetensors.torch import load_file
    lib = load_file(os.path.join(d1, "model.safetensors"))
    assert all(torch.equal(lib[n], w1[n]) for n in w1)
    # tied model: no lm_head tensor; untied: one
    _, wa = load_checkpoint(write_random_model(str(tmp_path / "t"), tiny.TINY_A, seed=1))
    assert "lm_head.weight" not in wa and "lm_head.weight" in w1


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    d = write_random_model(str(tmp_path / "m"), tiny.TINY_A, seed=1)
    _, w = load_checkpoint(d)
    w = dict(w)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.extra.weight"] = torch.zeros(3)
    w["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 64)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)      # dropped, not "unexpected"
    w["lm_head.weight"] = torch.zeros(256, 64)                              # dropped for a tied model
    _, model = registry.build_model(tiny.TINY_A)
    with pytest.raises(WeightError) as ei:
        model.check_weights(w)
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.extra.weight"]
    assert [n for n, _, _ in e.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    text = str(e)
    assert "missing (2)" in text and "unexpected (1)" in text and "has [10, 64], want [64, 64]" in text


def test_bias_tensors_are_required_when_the_flags_are_on():
    _, model = registry.build_model(tiny.TINY_C)
    names = {s.name for s in model.weight_specs()}
    assert "model.layers.0.self_attn.o_proj.bias" in names and "model.layers.0.mlp.down_proj.bias" in names
    assert "lm_head.weight" in names


def test_checkpoint_folder_rules(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    with pytest.raises(ConfigError, match="config.json"):
        load_checkpoint(str(d))
    (d / "config.json").write_text(json.dumps(tiny.TINY_A))
    with pytest.raises(WeightError, match="no .safetensors"):
        load_checkpoint(str(d))
    st.write_file(str(d / "a.safetensors"), {"x": torch.ones(2)})
    st.write_file(str(d / "b.safetensors"), {"x": torch.ones(2)})
    with pytest.raises(WeightError, match="more than one shard"):
        load_checkpoint(str(d))
    # with an index, only the files it names are read
    st.write_index(str(d / st.INDEX_NAME), {"x": "a.safetensors"}, 8)
    _, w = load_checkpoint(str(d))
    assert list(w) == ["x"]
    (d / st.INDEX_NAME).write_text(json.dumps({"weight_map": {}}))
    with pytest.raises(st.SafetensorsError, match="weight_map"):
        load_checkpoint(str(d))


def test_dtype_policy(tmp_path):
    p = str(tmp_path / "x.safetensors")
    st.write_file(p, {"h": torch.ones(2, dtype=torch.float16), "f": torch.ones(2), "b": torch.ones(2, dtype=torch.bfloat16),
                      "i": torch.tensor([1, 2]), "j": torch.tensor([3], dtype=torch.int32)})
    (tmp_path / "config.json").write_text("{}")
    _, w = load_checkpoint(str(tmp_path))
    assert w["h"].dtype == torch.bfloat16 and w["f"].dtype == torch.float32 and w["b"].dtype == torch.bfloat16
    assert w["i"].dtype == torch.int32 and w["j"].dtype == torch.int32


def _blob(header: dict, data: bytes = b"") -> bytes:
    h = json.dumps(header).encode()
    return struct.pack("<Q", len(h)) + h + data


@pytest.mark.parametrize("blob,word", [
    (b"\x01\x02", "shorter"), (struct.pack("<Q", 1 << 40), "too large"), (struct.pack("<Q", 50) + b"{}", "does not fit"),
    (_blob({"x": {"dtype": "F99", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4), "unknown dtype"),
    (_blob({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4), "needs 8 bytes"),
    (_blob({"x": {"dtype": "F32", "shape": [1], "data_offsets": [0, 8]}}, b"\0" * 4), "outside")])
def test_safetensors_header_errors(blob, word):
    with pytest.raises(st.SafetensorsError, match=word):
        st.parse_header(blob)


def test_fp8_tensors_are_refused(tmp_path):
    p = tmp_path / "x.safetensors"
    p.write_bytes(_blob({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 4))
    with pytest.raises(st.SafetensorsError, match="unsupported dtype"):
        st.read_file(str(p))
