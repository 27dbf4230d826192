"""The safetensors container, loading by name and its one error, random weights (no GPU)."""
import json
import struct

import numpy as np
import pytest
import torch

from nncpu_b200.engine.model import parameter_list
from nncpu_b200.errors import BadFormat, UnsupportedModel
from nncpu_b200.weights import (ParamSpec, SafetensorsFile, check_tensors, convert, draw, load_tensors,
                                random_tensors, write_model_folder, write_safetensors)
from plain_qwen3 import read_safetensors
from tiny import make_folder, tiny_config


def test_container_round_trip(tmp_path):
    t = {"a.weight": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "ids": torch.arange(6, dtype=torch.int32),
         "empty": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "x.safetensors", t, {"note": "hi"})
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert set(f.names()) == set(t) and f.metadata["note"] == "hi"
    for k, v in t.items():
        assert f.dtype(k) == {torch.float32: "F32", torch.bfloat16: "BF16", torch.int32: "I32"}[v.dtype]
        assert torch.equal(f.tensor(k), v) and f.shape(k) == tuple(v.shape)
    # an independent reader agrees
    plain = read_safetensors(tmp_path / "x.safetensors")
    assert np.array_equal(plain["a.weight"], t["a.weight"].numpy())
    assert np.array_equal(plain["b"], t["b"].float().numpy())


def test_container_refuses_damage(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(BadFormat, match="too short"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(BadFormat, match="header length"):
        SafetensorsFile(p)
    head = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 8)
    with pytest.raises(BadFormat, match="does not match"):
        SafetensorsFile(p)
    head = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 4)
    with pytest.raises(UnsupportedModel, match="F8_E4M3"):
        SafetensorsFile(p)
    with pytest.raises(BadFormat, match="does not exist"):
        SafetensorsFile(tmp_path / "none.safetensors")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder(tmp_path / "m", "B")
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(4)
    tensors["model.layers.2.self_attn.q_norm.weight"] = torch.zeros(7)
    tensors["lm_head.weight"] = torch.zeros(5, 96)
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(BadFormat) as e:
        load_tensors(folder, parameter_list(tiny_config("B").model_spec()), torch.float32, "cpu")
    msg = str(e.value)
    assert "missing (2): model.layers.1.mlp.up_proj.weight, model.norm.weight" in msg
    assert "unexpected (1): model.layers.0.self_attn.rotary.inv_freq" in msg
    assert "wrong shape (2)" in msg
    assert "lm_head.weight is [5, 96], expected [384, 96]" in msg
    assert "model.layers.2.self_attn.q_norm.weight is [7], expected [32]" in msg


def test_optional_tensor_may_be_absent_or_present(tmp_path):
    params = [ParamSpec("w", (2, 2)), ParamSpec("b", (2,), required=False)]
    check_tensors({"w": (2, 2)}, params, "file")
    check_tensors({"w": (2, 2), "b": (2,)}, params, "file")
    with pytest.raises(BadFormat, match="wrong shape"):
        check_tensors({"w": (2, 2), "b": (3,)}, params, "file")


def test_tied_model_refuses_a_stray_output_matrix(tmp_path):
    folder = make_folder(tmp_path / "m", "A")
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(BadFormat, match=r"unexpected \(1\): lm_head.weight"):
        load_tensors(folder, parameter_list(tiny_config("A").model_spec()), torch.float32, "cpu")


def test_element_types_kept_or_widened():
    bf, f32, f16 = torch.ones(2).bfloat16(), torch.ones(2), torch.ones(2).half()
    i64 = torch.arange(3)
    # bfloat16 run: BF16 stays, 32-bit stays 32-bit, F16 becomes BF16, integer tables become int32
    assert convert(bf, "BF16", torch.bfloat16).dtype == torch.bfloat16
    assert convert(f32, "F32", torch.bfloat16).dtype == torch.float32
    assert convert(f16, "F16", torch.bfloat16).dtype == torch.bfloat16
    assert convert(i64, "I64", torch.bfloat16).dtype == torch.int32
    # float32 run: every floating tensor is widened
    for t, name in ((bf, "BF16"), (f32, "F32"), (f16, "F16")):
        assert convert(t, name, torch.float32).dtype == torch.float32
    assert convert(i64, "I64", torch.float32).dtype == torch.int32


def test_load_keeps_stored_element_types(tmp_path):
    folder = make_folder(tmp_path / "m", "B", store_dtype=torch.bfloat16, vector_dtype=torch.float32)
    params = parameter_list(tiny_config("B").model_spec())
    t = load_tensors(folder, params, torch.bfloat16, "cpu")
    assert t["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert t["model.layers.0.input_layernorm.weight"].dtype == torch.float32
    assert t["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32
    t = load_tensors(folder, params, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t.values())


def test_random_weights_depend_on_seed_and_name_only():
    a = ParamSpec("x.weight", (4, 6))
    b = ParamSpec("y.weight", (4, 6))
    g = ParamSpec("n.weight", (64,), init=("one_plus_normal", 0.1))
    assert torch.equal(draw(a, 3), draw(a, 3))
    assert not torch.equal(draw(a, 3), draw(a, 4))
    assert not torch.equal(draw(a, 3), draw(b, 3))
    one = random_tensors([a, b, g], 5, torch.float32)
    other = random_tensors([g, b], 5, torch.float32)
    assert torch.equal(one["y.weight"], other["y.weight"]) and torch.equal(one["n.weight"], other["n.weight"])
    assert abs(float(one["n.weight"].mean()) - 1.0) < 0.1
    big = draw(ParamSpec("big", (400, 400)), 0)
    assert abs(float(big.std()) - 0.02) < 0.002 and abs(float(big.mean())) < 0.001


def test_written_folder_is_what_the_model_asks_for(tmp_path):
    for name in ("A", "B", "C"):
        cfg = tiny_config(name)
        folder = write_model_folder(tmp_path / name, cfg, seed=1)
        written = json.loads((folder / "config.json").read_text())
        assert written["architectures"] == ["Qwen3ForCausalLM"]
        t = load_tensors(folder, parameter_list(cfg.model_spec()), torch.bfloat16, "cpu")
        assert ("lm_head.weight" in t) == (not cfg.tie_word_embeddings)
        assert ("model.layers.0.self_attn.k_proj.bias" in t) == cfg.attention_bias
        assert t["model.embed_tokens.weight"].shape == (cfg.vocab_size, cfg.hidden_size)


def test_load_can_be_cancelled(tmp_path):
    from nncpu_b200.errors import Cancelled
    folder = make_folder(tmp_path / "m", "A")
    seen = []
    with pytest.raises(Cancelled):
        load_tensors(folder, parameter_list(tiny_config("A").model_spec()), torch.float32, "cpu",
                     progress=lambda done, total: seen.append((done, total)) or len(seen) < 3)
    assert len(seen) == 3


def _split_folder(tmp_path, name):
    """A written model folder cut into two files with an index, the way large checkpoints are published."""
    cfg = tiny_config(name)
    folder = write_model_folder(tmp_path / name, cfg, seed=2)
    params = parameter_list(cfg.model_spec())
    whole = load_tensors(folder, params, torch.bfloat16, "cpu")
    f = SafetensorsFile(folder / "model.safetensors")
    stored = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    (folder / "model.safetensors").unlink()
    names = sorted(stored)
    parts = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
    for file_name, members in parts.items():
        write_safetensors(folder / file_name, {n: stored[n] for n in members})
    index = {"metadata": {}, "weight_map": {n: file_name for file_name, members in parts.items() for n in members}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    return folder, params, whole, index


def test_checkpoint_in_several_files_loads_like_one(tmp_path):
    folder, params, whole, _ = _split_folder(tmp_path, "B")
    t = load_tensors(folder, params, torch.bfloat16, "cpu")
    assert set(t) == set(whole) and all(torch.equal(t[n], whole[n]) for n in whole)


def test_checkpoint_in_several_files_reports_everything_at_once(tmp_path):
    folder, params, _, index = _split_folder(tmp_path, "A")
    # one error over the union of the files: a tensor of another model's shape set
    with pytest.raises(BadFormat) as e:
        load_tensors(folder, parameter_list(tiny_config("B").model_spec()), torch.float32, "cpu")
    assert "index.json" in str(e.value) and "wrong shape" in str(e.value)
    # the index names a tensor that its file does not hold
    broken = dict(index, weight_map=dict(index["weight_map"], **{"model.ghost.weight": "model-00001-of-00002.safetensors"}))
    (folder / "model.safetensors.index.json").write_text(json.dumps(broken))
    with pytest.raises(BadFormat, match="model.ghost.weight"):
        load_tensors(folder, params, torch.float32, "cpu")
    # a file of the index is missing
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    (folder / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(BadFormat, match="model-00002-of-00002.safetensors does not exist"):
        load_tensors(folder, params, torch.float32, "cpu")
    # an index without a weight_map, or one that leaves the folder
    (folder / "model.safetensors.index.json").write_text("{}")
    with pytest.raises(BadFormat, match="weight_map"):
        load_tensors(folder, params, torch.float32, "cpu")
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "../x.safetensors"}}))
    with pytest.raises(BadFormat, match="outside the folder"):
        load_tensors(folder, params, torch.float32, "cpu")
