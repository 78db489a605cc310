"""Safetensors reading and writing, the one weight error, random weights (CPU)."""
import json
import struct

import pytest
import torch

import plain_qwen3 as plain
import tiny
from garlic_inference_b200 import WeightError, write_random_model
from garlic_inference_b200.engine import wanted_tensors
from garlic_inference_b200.weights import (Checkpoint, SafetensorsFile, device_dtype, write_safetensors)


def test_write_then_read_every_dtype(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {
        "a.f32": torch.randn(3, 5, generator=g),
        "b.bf16": torch.randn(7, 2, generator=g).to(torch.bfloat16),
        "c.f16": torch.randn(4, generator=g).to(torch.float16),
        "d.i32": torch.arange(6, dtype=torch.int32).view(2, 3),
        "e.i64": torch.arange(4, dtype=torch.int64),
        "f.scalar": torch.tensor(2.5),
    }
    path = tmp_path / "x.safetensors"
    write_safetensors(path, tensors, metadata={"k": "v"})
    f = SafetensorsFile(path)
    assert set(f.names()) == set(tensors)
    for n, t in tensors.items():
        got = f.tensor(n)
        assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t), n
    # an independent reader (the plain implementation's) sees the same numbers
    other = plain.read_safetensors(path)
    assert torch.equal(other["b.bf16"], tensors["b.bf16"].float())


def test_truncated_and_malformed_files(tmp_path):
    path = tmp_path / "x.safetensors"
    write_safetensors(path, {"w": torch.ones(8, 8)})
    raw = path.read_bytes()
    (tmp_path / "cut.safetensors").write_bytes(raw[:-16])
    with pytest.raises(Exception, match="truncated"):
        SafetensorsFile(tmp_path / "cut.safetensors")
    (tmp_path / "short.safetensors").write_bytes(raw[:4])
    with pytest.raises(Exception, match="shorter"):
        SafetensorsFile(tmp_path / "short.safetensors")
    hdr = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    (tmp_path / "fp8.safetensors").write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(Exception, match="F8_E4M3"):
        SafetensorsFile(tmp_path / "fp8.safetensors")
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    (tmp_path / "size.safetensors").write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(Exception, match="needs 16 bytes"):
        SafetensorsFile(tmp_path / "size.safetensors")


def test_random_model_is_seeded_and_complete(tmp_path):
    cfg = tiny.make_config("B")
    a = write_random_model(tmp_path / "a", cfg, seed=5, std=0.05, norm_std=0.2)
    b = write_random_model(tmp_path / "b", cfg, seed=5, std=0.05, norm_std=0.2)
    c = write_random_model(tmp_path / "c", cfg, seed=6, std=0.05, norm_std=0.2)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    ck = Checkpoint(a)
    ck.check(wanted_tensors(cfg.plan()))
    w = ck.tensor("model.layers.1.mlp.up_proj.weight").float()
    assert w.dtype == torch.float32 and abs(float(w.std()) - 0.05) < 0.005
    n = ck.tensor("model.layers.2.self_attn.q_norm.weight").float()
    assert abs(float(n.mean()) - 1.0) < 0.2 and float(n.std()) > 0.05
    assert ck.stored_dtype("model.norm.weight") == torch.bfloat16
    assert json.loads((a / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = tiny.make_config("A")
    d = write_random_model(tmp_path / "m", cfg, seed=0)
    ck = Checkpoint(d)
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    del tensors["model.layers.1.self_attn.k_norm.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(191, 64, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64, dtype=torch.bfloat16)
    tensors["lm_head.weight"] = torch.zeros(512, 64, dtype=torch.bfloat16)     # tied model: not wanted
    write_safetensors(d / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        Checkpoint(d).check(wanted_tensors(cfg.plan()))
    msg = str(e.value)
    assert "2 missing, 2 unexpected, 1 of wrong shape" in msg
    for needle in ("missing:    model.layers.1.self_attn.k_norm.weight", "missing:    model.norm.weight",
                   "unexpected: model.layers.0.self_attn.q_proj.bias", "unexpected: lm_head.weight",
                   "model.layers.0.mlp.gate_proj.weight  wanted [192, 64], found [191, 64]"):
        assert needle in msg, (needle, msg)


def test_integer_tensor_where_floating_is_wanted(tmp_path):
    cfg = tiny.make_config("A")
    d = write_random_model(tmp_path / "m", cfg, seed=0)
    ck = Checkpoint(d)
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    tensors["model.norm.weight"] = torch.ones(64, dtype=torch.int32)
    write_safetensors(d / "model.safetensors", tensors)
    with pytest.raises(WeightError, match="wrong dtype: model.norm.weight"):
        Checkpoint(d).check(wanted_tensors(cfg.plan()))


def test_sharded_folder_and_missing_files(tmp_path):
    cfg = tiny.make_config("A")
    d = write_random_model(tmp_path / "m", cfg, seed=0)
    ck = Checkpoint(d)
    names = ck.names()
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    s = tmp_path / "sharded"
    s.mkdir()
    weight_map = {}
    for fname, ns in shards.items():
        write_safetensors(s / fname, {n: ck.tensor(n) for n in ns})
        weight_map.update({n: fname for n in ns})
    (s / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    (s / "config.json").write_text((d / "config.json").read_text())
    sh = Checkpoint(s)
    sh.check(wanted_tensors(cfg.plan()))
    for n in names:
        assert torch.equal(sh.tensor(n), ck.tensor(n))
    with pytest.raises(WeightError, match="neither model.safetensors"):
        Checkpoint(tmp_path)
    (s / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(WeightError, match="no such file"):
        Checkpoint(s)


def test_device_dtype_policy():
    bf, f32, f16 = torch.bfloat16, torch.float32, torch.float16
    assert device_dtype(bf, bf) == bf and device_dtype(f16, bf) == bf
    assert device_dtype(f32, bf) == f32                      # stored in 32-bit: stays so
    assert device_dtype(torch.int64, bf) == torch.int32      # integer tables
    assert device_dtype(bf, f32) == f32 and device_dtype(f32, f32) == f32
    with pytest.raises(ValueError):
        device_dtype(bf, f16)
