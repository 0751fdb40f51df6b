"""Weights (no GPU): the safetensors container is read with suspicion, the checkpoint must
hold exactly what the model declares, and one error lists everything that is wrong
(safetensors/safetensors.go:133-272, model/weights.go:158-276)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import tiny
from tgo_b200.engine.model import Model
from tgo_b200.registry import model_spec_from_config
from tgo_b200.weights.binder import WeightError, WeightSpec, check_weights, load_weights
from tgo_b200.weights.random_init import random_weights, write_random_model
from tgo_b200.weights.safetensors import (SafetensorsError, SafetensorsFile, SafetensorsRepo,
                                          write_safetensors)


def raw_file(path, header, data=b""):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + data)
    return str(path)


def test_round_trip_keeps_dtypes(tmp_path):
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
               "d": torch.randn(2, 2).to(torch.float16)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors)
    f = SafetensorsFile(path)
    for name, t in tensors.items():
        got = f.tensor(name)
        assert got.dtype == t.dtype and torch.equal(got, t)
    import plain_qwen3
    plain = plain_qwen3.read_safetensors(path)          # the tests' own reader agrees
    assert np.allclose(plain["a"], tensors["a"].double().numpy())


@pytest.mark.parametrize("header,data,needle", [
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 8, "needs 8 bytes"),
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 16]}}, b"\0" * 8, "outside"),
    ({"x": {"dtype": "Q9", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8, "unknown dtype"),
    ({"x": {"dtype": "F32", "shape": [-2], "data_offsets": [0, 8]}}, b"\0" * 8, "bad shape"),
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [8, 0]}}, b"\0" * 8, "outside"),
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0]}}, b"\0" * 8, "bad data_offsets"),
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
      "y": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12, "overlap"),
])
def test_hostile_headers_are_refused(tmp_path, header, data, needle):
    path = raw_file(tmp_path / "m.safetensors", header, data)
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFile(path)
    assert needle in str(e.value)


def test_truncated_and_oversized_headers(tmp_path):
    p = tmp_path / "m.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 10 ** 12) + b"{}")
    with pytest.raises(SafetensorsError, match="does not fit"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="not JSON"):
        SafetensorsFile(str(p))


def test_sharded_repo_and_bad_shard_names(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.zeros(2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.ones(3)})
    index = tmp_path / "model.safetensors.index.json"
    index.write_text(json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    repo = SafetensorsRepo(str(tmp_path))
    assert repo.names() == ["a", "b"] and torch.equal(repo.tensor("b"), torch.ones(3))
    index.write_text(json.dumps({"weight_map": {"a": "../s1.safetensors"}}))
    with pytest.raises(SafetensorsError, match="plain file name"):
        SafetensorsRepo(str(tmp_path))
    index.write_text(json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s1.safetensors"}}))
    with pytest.raises(SafetensorsError, match="is not in"):
        SafetensorsRepo(str(tmp_path))
    index.write_text(json.dumps({"weight_map": {"a": "s1.safetensors"}}))
    os.rename(tmp_path / "s2.safetensors", tmp_path / "s1b.safetensors")
    SafetensorsRepo(str(tmp_path))        # a shard the index never names is simply not opened
    with pytest.raises(SafetensorsError, match="neither"):
        SafetensorsRepo(str(tmp_path / "nowhere"))


def model_and_dir(tmp_path, cfg, run):
    d = tiny.make_model_dir(tmp_path / "m", cfg, run["seed"], run["sigma"])
    return Model(model_spec_from_config(cfg), torch.float32, "cpu"), d


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    cfg, run = tiny.TINIES["B"]
    model, d = model_and_dir(tmp_path, cfg, run)
    repo = SafetensorsRepo(d)
    tensors = {n: repo.tensor(n).clone() for n in repo.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"], tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192)
    tensors["model.layers.2.self_attn.k_norm.weight"] = torch.zeros(16)
    tensors["model.embed_tokens.weight"] = torch.zeros(383, 96, dtype=torch.bfloat16)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        load_weights(model.weight_specs(), SafetensorsRepo(d), torch.float32, "cpu")
    msg = str(e.value)
    assert "2 missing" in msg and "model.layers.1.mlp.up_proj.weight" in msg
    assert "1 unexpected" in msg and "q_proj.bias" in msg
    assert "2 of the wrong shape" in msg and "k_norm.weight is [16], declared [32]" in msg
    # the embedding's row count is the vocabulary: the message names the config's field
    assert "vocab_size is 384 and model.embed_tokens.weight has 383 rows" in msg


def test_errors_for_rank_empty_and_values_that_do_not_survive(tmp_path):
    """weights/weights.go:756-762 (a weight is a matrix or a gain vector), :605-610 (an empty
    tensor), :450-458 (values the 16-bit storage type cannot hold); and the rounding of
    float16 to bfloat16 is said once."""
    specs = [WeightSpec("m", (2, 3), "matrix"), WeightSpec("g", (3,), "gain")]
    with pytest.raises(WeightError) as e:
        check_weights(specs, {"m": ("BF16", (2, 3, 1)), "g": ("F32", (0,))})
    assert "m has rank 3" in str(e.value) and "g is empty" in str(e.value)
    write_safetensors(str(tmp_path / "model.safetensors"),
                      {"m": torch.tensor([[1.0, 2.0, 0.3337], [4.0, 5.0, 6.0]], dtype=torch.float16),
                       "g": torch.ones(3)})
    logs = []
    got = load_weights(specs, SafetensorsRepo(str(tmp_path)), torch.bfloat16, "cpu", None, logs.append)
    assert got["m"].dtype == torch.bfloat16
    assert len(logs) == 1 and "1 tensors are stored as float16" in logs[0] and "m" in logs[0]
    logs.clear()
    load_weights(specs, SafetensorsRepo(str(tmp_path)), torch.float32, "cpu", None, logs.append)
    assert not logs                                  # widening loses nothing and says nothing
    write_safetensors(str(tmp_path / "model.safetensors"),
                      {"m": torch.tensor([[1.0, float("inf"), 0.0], [4.0, 5.0, 6.0]],
                                         dtype=torch.float16), "g": torch.ones(3)})
    with pytest.raises(WeightError, match="not finite"):
        load_weights(specs, SafetensorsRepo(str(tmp_path)), torch.bfloat16, "cpu", None, logs.append)


def test_declared_names_are_the_checkpoints_own(tmp_path):
    cfg, run = tiny.TINIES["B"]
    model, d = model_and_dir(tmp_path, cfg, run)
    names = {w.name: w for w in model.weight_specs()}
    assert len(names) == 2 + 11 * 3 + 1
    assert names["model.layers.2.self_attn.q_proj.weight"].shape == (192, 96)
    assert names["model.layers.0.self_attn.k_proj.weight"].shape == (64, 96)
    assert names["model.layers.0.self_attn.o_proj.weight"].shape == (96, 192)
    assert names["model.layers.1.mlp.down_proj.weight"].shape == (96, 224)
    assert names["model.layers.1.self_attn.q_norm.weight"].role == "gain"
    assert names["lm_head.weight"].shape == (384, 96)
    assert sorted(names) == SafetensorsRepo(d).names()


def test_tied_head_shipped_anyway(tmp_path):
    cfg, run = tiny.TINIES["A"]
    model, d = model_and_dir(tmp_path, cfg, run)
    assert "lm_head.weight" not in SafetensorsRepo(d).names()
    repo = SafetensorsRepo(d)
    tensors = {n: repo.tensor(n).clone() for n in repo.names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    load_weights(model.weight_specs(), SafetensorsRepo(d), torch.float32, "cpu", model.tied_alias())
    tensors["lm_head.weight"][0, 0] += 1
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightError, match="ties the head"):
        load_weights(model.weight_specs(), SafetensorsRepo(d), torch.float32, "cpu",
                     model.tied_alias())


def test_storage_widths(tmp_path):
    cfg, run = tiny.TINIES["A"]
    model, d = model_and_dir(tmp_path, cfg, run)
    logs = []
    w = load_weights(model.weight_specs(), SafetensorsRepo(d), torch.bfloat16, "cpu",
                     model.tied_alias(), logs.append)
    assert w["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16     # kept as stored
    assert w["model.norm.weight"].dtype == torch.float32                       # gains widen
    assert not logs
    specs = [WeightSpec("m", (2, 2), "matrix"), WeightSpec("t", (3,), "other"),
             WeightSpec("i", (2,), "other")]
    write_safetensors(str(tmp_path / "model.safetensors"),
                      {"m": torch.ones(2, 2), "t": torch.ones(3), "i": torch.tensor([1, 2])})
    got = load_weights(specs, SafetensorsRepo(str(tmp_path)), torch.bfloat16, "cpu", None,
                       logs.append)
    assert got["m"].dtype == torch.bfloat16 and "narrowed" in logs[0]
    assert got["t"].dtype == torch.float32          # stored in 32-bit, stays so
    assert got["i"].dtype == torch.int32            # integer tables as int32
    with pytest.raises(WeightError, match="declared twice"):
        check_weights([WeightSpec("m", (1,)), WeightSpec("m", (1,))], {})


def test_random_weights_are_seeded_per_tensor(tmp_path):
    specs = [WeightSpec("a", (4, 4)), WeightSpec("g", (4,), "gain")]
    w1, w2 = random_weights(specs, 3, dtype=torch.float32), random_weights(specs[::-1], 3,
                                                                          dtype=torch.float32)
    assert torch.equal(w1["a"], w2["a"]) and torch.equal(w1["g"], w2["g"])
    assert not torch.equal(w1["a"], random_weights(specs, 4, dtype=torch.float32)["a"])
    assert abs(float(w1["g"].mean()) - 1) < 0.3
    from tgo_b200.weights.random_init import seeded_normal
    x = seeded_normal(200000, 7)
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1) < 0.01
    assert abs(float((x ** 4).mean()) - 3) < 0.1 and float(x.abs().max()) < 4.4
    assert torch.equal(x[:1000], seeded_normal(1000, 7))       # a stream's start does not depend on its length
    write_random_model(str(tmp_path / "r"), tiny.TINY_A, seed=0)
    assert sorted(os.listdir(tmp_path / "r")) == ["config.json", "model.safetensors"]
    with open(tmp_path / "r" / "config.json") as f:
        assert json.load(f) == tiny.TINY_A
