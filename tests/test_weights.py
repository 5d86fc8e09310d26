"""Safetensors reading and writing, the one error that lists everything wrong with a model
folder, and the random-weights mode."""
import json
import os
import struct

import pytest
import torch

from camelid_b200 import SafetensorsError, WeightsError
from camelid_b200.engine.model import DecoderModel
from camelid_b200.weights import ModelFiles, SafetensorsFile, random_tensors, write_random_model, write_safetensors
from conftest import TINY_A, TINY_B
import plain_llama as pl


def test_round_trip_and_independent_reader(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b.c": torch.arange(7, dtype=torch.int32),
         "d": torch.randn(2, 2, 2), "e": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"k": "v"})
    f = SafetensorsFile(p)
    assert sorted(f.names()) == sorted(t) and f.metadata == {"k": "v"}
    for n in t:
        assert f.dtype(n) == t[n].dtype and torch.equal(f.tensor(n), t[n])
    other = pl.read_safetensors(p)                       # the oracle's own reader
    for n in t:
        assert torch.equal(other[n], t[n])
    f.close()


def test_reads_what_the_safetensors_package_writes(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"w": torch.randn(4, 6).to(torch.bfloat16), "n": torch.randn(6)}
    p = str(tmp_path / "pkg.safetensors")
    st.save_file(t, p)
    f = SafetensorsFile(p)
    for n in t:
        assert torch.equal(f.tensor(n), t[n])
    p2 = str(tmp_path / "ours.safetensors")
    write_safetensors(p2, t)
    back = st.load_file(p2)
    for n in t:
        assert torch.equal(back[n], t[n])


def _raw(path, header: dict, payload: bytes):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + payload)


@pytest.mark.parametrize("header,payload,word", [
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 16]}}, b"\0" * 8, "outside"),
    ({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8, "needs"),
    ({"a": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8, "unsupported"),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
      "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12, "overlap"),
    ({"a": {"dtype": "F32"}}, b"", "malformed"),
])
def test_malformed_files(tmp_path, header, payload, word):
    p = str(tmp_path / "bad.safetensors")
    _raw(p, header, payload)
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFile(p)
    assert word in str(e.value)


def test_short_and_broken_header(tmp_path):
    p = str(tmp_path / "s.safetensors")
    open(p, "wb").write(b"abc")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 4) + b"{{{{")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError):
        ModelFiles(str(tmp_path / "empty_folder_that_is_missing"))


def test_shards_and_duplicates(tmp_path):
    write_safetensors(str(tmp_path / "m1.safetensors"), {"a": torch.ones(2)})
    write_safetensors(str(tmp_path / "m2.safetensors"), {"b": torch.ones(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "m1.safetensors", "b": "m2.safetensors"}}))
    files = ModelFiles(str(tmp_path))
    assert sorted(files.names()) == ["a", "b"] and files.shape("b") == [3]
    write_safetensors(str(tmp_path / "m2.safetensors"), {"a": torch.ones(2), "b": torch.ones(3)})
    with pytest.raises(SafetensorsError) as e:
        ModelFiles(str(tmp_path))
    assert "both" in str(e.value)


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    model = DecoderModel.from_config(TINY_A, device="cpu")
    tensors = random_tensors(model.tensor_specs(), 0)
    assert len(tensors) == 2 + 2 * 9             # embedding, final norm, nine per layer; tied output
    model.load_tensors  # exists
    bad = dict(tensors)
    del bad["model.layers.1.mlp.up_proj.weight"]
    del bad["model.norm.weight"]
    bad["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16)
    bad["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    bad["model.embed_tokens.weight"] = torch.zeros(256, 64, dtype=torch.int32)
    with pytest.raises(WeightsError) as e:
        model.load_tensors(bad)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (16, 64))]
    assert any("model.embed_tokens.weight" in m for m in err.other)
    for word in ("missing", "unexpected", "wrong shape", "q_norm", "up_proj"):
        assert word in str(err)


def test_untied_model_needs_lm_head_and_tied_model_tolerates_one():
    untied = DecoderModel.from_config(TINY_B, device="cpu")
    t = random_tensors(untied.tensor_specs(), 1)
    assert "lm_head.weight" in t
    del t["lm_head.weight"]
    with pytest.raises(WeightsError) as e:
        untied.load_tensors(t)
    assert e.value.missing == ["lm_head.weight"]
    tied = DecoderModel.from_config(TINY_A, device="cpu")
    specs = tied.tensor_specs()
    assert "lm_head.weight" not in specs
    from camelid_b200.weights.loader import check_tensors
    found = {n: (s.shape, torch.bfloat16) for n, s in specs.items()}
    found["lm_head.weight"] = ((256, 64), torch.bfloat16)
    check_tensors(specs, found, tolerated=("lm_head.weight",))
    with pytest.raises(WeightsError):
        check_tensors(specs, found)


def test_random_model_folder(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_B, seed=1, norm_dtype=torch.float32)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    cfg, w = pl.read_model(d)
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["intermediate_size"] == 512
    assert w["model.layers.2.mlp.down_proj.weight"].shape == (192, 512)
    assert w["model.layers.0.mlp.gate_proj.weight"].dtype == torch.bfloat16
    assert w["model.norm.weight"].dtype == torch.float32
    lin = w["model.embed_tokens.weight"].float()
    assert abs(float(lin.std()) - 0.02) < 0.002 and abs(float(lin.mean())) < 0.002
    nrm = w["model.layers.1.input_layernorm.weight"].float()
    assert abs(float(nrm.mean()) - 1.0) < 0.01 and 0.01 < float(nrm.std()) < 0.03
    d2 = write_random_model(str(tmp_path / "m2"), TINY_B, seed=1, norm_dtype=torch.float32)
    w2 = pl.read_safetensors(os.path.join(d2, "model.safetensors"))
    assert all(torch.equal(w[n], w2[n]) for n in w)
    d3 = write_random_model(str(tmp_path / "m3"), TINY_B, seed=2)
    w3 = pl.read_safetensors(os.path.join(d3, "model.safetensors"))
    assert not torch.equal(w["model.embed_tokens.weight"], w3["model.embed_tokens.weight"])
