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


def test_surplus_tensors_are_listed_in_a_warning_not_refused(tmp_path):
    """A tied model whose file also stores lm_head.weight (and a stray buffer) loads; both are named once."""
    from garlic_inference_b200.weights import SurplusTensorWarning
    cfg = tiny.make_config("A")                                      # tied head
    d = write_random_model(tmp_path / "m", cfg, seed=0)
    ck = Checkpoint(d)
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    write_safetensors(d / "model.safetensors", tensors)
    with pytest.warns(SurplusTensorWarning) as rec:
        ck2 = Checkpoint(d)
        ck2.check(wanted_tensors(cfg.plan()))
    assert len(rec) == 1
    msg = str(rec[0].message)
    assert "2 tensors are not used" in msg and "lm_head.weight [512, 64]" in msg and "inv_freq" in msg
    assert ck2.unexpected == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]


def test_packed_tensors_keep_the_widest_stored_type(tmp_path):
    """q in bfloat16, k and v in float32: the packed q/k/v weight is float32 and holds k and v exactly."""
    from garlic_inference_b200.engine.model import DecoderModel
    from garlic_inference_b200.parts import Runtime
    cfg = tiny.make_config("A")
    d = write_random_model(tmp_path / "m", cfg, seed=0)
    ck = Checkpoint(d)
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    g = torch.Generator().manual_seed(1)
    k32 = torch.randn(tensors["model.layers.0.self_attn.k_proj.weight"].shape, generator=g) * 0.02
    tensors["model.layers.0.self_attn.k_proj.weight"] = k32
    tensors["model.layers.0.self_attn.v_proj.weight"] = tensors["model.layers.0.self_attn.v_proj.weight"].float()
    tensors["model.layers.1.mlp.up_proj.weight"] = tensors["model.layers.1.mlp.up_proj.weight"].float() + 1e-4
    write_safetensors(d / "model.safetensors", tensors)
    ck = Checkpoint(d)
    ck.check(wanted_tensors(cfg.plan()))
    model = DecoderModel(cfg.plan(), ck, Runtime(torch.bfloat16, torch.device("cpu")))
    a0, a1 = model.blocks[0].mixer, model.blocks[1].mixer
    assert a0.w_qkv.dtype == torch.float32 and a1.w_qkv.dtype == torch.bfloat16
    q_rows, kv_rows = a0.n_q * a0.d, a0.n_kv * a0.d
    assert torch.equal(a0.w_qkv[q_rows:q_rows + kv_rows], k32)                 # not rounded to bfloat16
    assert torch.equal(a0.w_qkv[:q_rows], tensors["model.layers.0.self_attn.q_proj.weight"].float())
    assert model.blocks[1].feed_forward.w_gate_up.dtype == torch.float32
    assert model.blocks[0].feed_forward.w_gate_up.dtype == torch.bfloat16


def test_random_values_depend_on_seed_name_and_index_only():
    from garlic_inference_b200.weights.random_init import normal_values, tensor_key
    k = tensor_key(3, "model.layers.0.mlp.up_proj.weight")
    assert k == tensor_key(3, "model.layers.0.mlp.up_proj.weight")
    assert k != tensor_key(4, "model.layers.0.mlp.up_proj.weight") and k != tensor_key(3, "model.norm.weight")
    whole = normal_values(k, 10000, 0.0, 1.0)
    assert whole.dtype.name == "float32"
    # any slice of the stream is the same numbers: the generator has no state
    part = normal_values(k, 100, 0.0, 1.0, start=5000)
    assert (part == whole[5000:5100]).all()
    big = normal_values(k, 1 << 20, 0.0, 1.0)
    assert abs(float(big.mean())) < 5e-3 and abs(float(big.std()) - 1.0) < 5e-3
    assert float(abs(big).max()) <= 6.0
    frac = float((abs(big) < 1.0).mean())
    assert abs(frac - 0.6827) < 5e-3                       # a normal variate's one-sigma mass
    shifted = normal_values(k, 1000, 1.0, 0.1)
    assert ((shifted - 1.0) / 0.1 - whole[:1000]).__abs__().max() < 1e-5


def test_the_compiled_generator_agrees_with_the_host_one():
    """The integer part of the weight generator and the two ends of the sampling uniform, through the C ABI."""
    from garlic_inference_b200.ops import ExtensionError, lib
    from garlic_inference_b200.weights.random_init import normal_values
    try:
        l = lib()
    except ExtensionError as e:                              # no nvcc on this machine
        pytest.skip(str(e))
    z = normal_values(987654321, 64, 0.0, 1.0)
    for i in range(64):
        assert (2 * l.gi_random_sum12(987654321, i) - 786420) / 131072 == float(z[i]), i
    lo, hi = l.gi_sample_uniform_from_hash(0), l.gi_sample_uniform_from_hash(2 ** 64 - 1)
    assert 0.0 < lo < 1e-6 and 1.0 - 1e-6 < hi < 1.0        # strictly inside (0, 1): no infinite Gumbel term
    assert l.gi_sample_uniform_from_hash((2 ** 23 - 1) << 41) == hi
