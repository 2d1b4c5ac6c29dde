"""Weights: the safetensors container, binding by name, storage rule, one error for everything that is wrong."""
import json
import os
import struct

import pytest
import torch

import tiny
from zedinfer_b200.config import load_model_config
from zedinfer_b200.engine.model import Model
from zedinfer_b200.weights import (SafetensorsError, SafetensorsFile, TensorSpec, WeightsError, canonical_name,
                                   load_weights, random_tensors, save_file, storage_dtype, write_random_model)


def test_container_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b.c": torch.randn(7).to(torch.bfloat16), "i": torch.arange(6, dtype=torch.int64),
         "h": torch.randn(2, 2).to(torch.float16), "i32": torch.arange(4, dtype=torch.int32)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p, metadata={"format": "pt"})
    f = SafetensorsFile(p)
    assert set(f.entries) == set(t)
    for name, ref in t.items():
        got = f.entries[name].load()
        assert got.dtype == ref.dtype and torch.equal(got, ref)


def _write_raw(path, header: dict, data: bytes):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + data)


def test_container_errors(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    with open(p, "wb") as f:
        f.write(b"abc")
    with pytest.raises(SafetensorsError, match="too small"):
        SafetensorsFile(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    _write_raw(p, {"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 32]}}, b"\0" * 16)
    with pytest.raises(SafetensorsError, match="data_offsets"):
        SafetensorsFile(p)
    _write_raw(p, {"t": {"dtype": "F32", "shape": [5], "data_offsets": [0, 16]}}, b"\0" * 16)
    with pytest.raises(SafetensorsError, match="needs 20 bytes"):
        SafetensorsFile(p)
    _write_raw(p, {"t": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 16)
    with pytest.raises(SafetensorsError, match="unknown dtype"):
        SafetensorsFile(p)


def test_names_and_storage_rule():
    assert canonical_name("model.layers.0.mlp.up_proj.weight") == "layers.0.mlp.up_proj.weight"
    assert canonical_name("model.language_model.norm.weight") == "norm.weight"
    assert canonical_name("lm_head.weight") == "lm_head.weight"
    bf, f32 = torch.bfloat16, torch.float32
    assert storage_dtype(bf, "float", bf) == bf
    assert storage_dtype(f32, "float", bf) == f32          # a tensor stored in 32-bit stays so
    assert storage_dtype(torch.float16, "float", bf) == bf
    assert storage_dtype(bf, "float", f32) == f32
    assert storage_dtype(torch.int64, "int", bf) == torch.int32


def test_random_model_folder_and_load(tmp_path):
    d = tiny.make_model_dir(tmp_path, "B")
    assert os.path.isfile(os.path.join(d, "config.json")) and os.path.isfile(os.path.join(d, "model.safetensors"))
    arch, cfg, spec = load_model_config(d)
    model = Model(spec)
    specs = model.tensor_specs()
    assert "lm_head.weight" in specs and not specs["lm_head.weight"].optional
    w = load_weights(d, specs, torch.bfloat16, "cpu")
    assert set(w) == set(specs)
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    w32 = load_weights(d, specs, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["norm.weight"], w["norm.weight"].float())
    # same seed, same values; another seed, other values; norm weights sit around one
    again = random_tensors(specs, 1, torch.bfloat16, tiny.INIT_SCALE)
    assert torch.equal(again["layers.2.mlp.down_proj.weight"], w["layers.2.mlp.down_proj.weight"])
    other = random_tensors(specs, 2, torch.bfloat16, tiny.INIT_SCALE)
    assert not torch.equal(other["layers.2.mlp.down_proj.weight"], w["layers.2.mlp.down_proj.weight"])
    assert abs(float(w32["norm.weight"].mean()) - 1.0) < 0.01
    assert abs(float(w32["layers.0.self_attn.q_proj.weight"].std()) - 0.02 * tiny.INIT_SCALE) < 0.01


def test_tied_head_is_optional(tmp_path):
    d = tiny.make_model_dir(tmp_path, "A")
    _, _, spec = load_model_config(d)
    specs = Model(spec).tensor_specs()
    assert specs["lm_head.weight"].optional
    w = load_weights(d, specs, torch.float32, "cpu")
    assert "lm_head.weight" not in w


def test_float32_tensors_stay_float32_in_a_bfloat16_run(tmp_path):
    d = tiny.make_model_dir(tmp_path, "A", dtype="float32")
    _, _, spec = load_model_config(d)
    w = load_weights(d, Model(spec).tensor_specs(), torch.bfloat16, "cpu")
    assert all(t.dtype == torch.float32 for t in w.values())


def test_one_error_lists_everything(tmp_path):
    d = tiny.make_model_dir(tmp_path, "B")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: e.load().clone() for n, e in f.entries.items()}
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(10, 96, dtype=torch.bfloat16)
    tensors["model.layers.9.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(96, dtype=torch.int32)
    bad = tmp_path / "bad"
    bad.mkdir()
    save_file(tensors, str(bad / "model.safetensors"))
    with open(os.path.join(d, "config.json")) as src:
        (bad / "config.json").write_text(src.read())
    _, _, spec = load_model_config(str(bad))
    with pytest.raises(WeightsError) as ei:
        load_weights(str(bad), Model(spec).tensor_specs(), torch.bfloat16, "cpu")
    e = ei.value
    assert e.missing == ["layers.1.self_attn.k_proj.bias", "norm.weight"]
    assert e.unexpected == ["layers.9.extra.weight"]
    assert len(e.wrong) == 2
    msg = str(e)
    for word in ("layers.1.self_attn.k_proj.bias", "norm.weight", "layers.9.extra.weight", "[10, 96]", "[256, 96]",
                 "input_layernorm.weight"):
        assert word in msg


def test_folder_errors(tmp_path):
    with pytest.raises(SafetensorsError, match="No .safetensors files"):
        load_weights(str(tmp_path), {}, torch.float32, "cpu")
    with pytest.raises(SafetensorsError, match="does not exist"):
        load_weights(str(tmp_path / "nope"), {}, torch.float32, "cpu")
    a, b = tmp_path / "m1.safetensors", tmp_path / "m2.safetensors"
    save_file({"model.x": torch.zeros(2)}, str(a))
    save_file({"x": torch.zeros(2)}, str(b))
    with pytest.raises(WeightsError, match="more than once"):
        load_weights(str(tmp_path), {"x": TensorSpec((2,))}, torch.float32, "cpu")


def test_one_rule_draws_the_weights_everywhere(tmp_path):
    """(seed, tensor name, element index) decides a value: the folder that ``write_random_model`` writes, the tensors
    ``random_tensors`` draws directly (what the engine does on the device, without a folder), any piece of a tensor
    drawn on its own, and the plain implementation's restatement of the rule all hold the same bits."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from plain import qwen2_plain as P
    from zedinfer_b200.weights.random_init import draw_tensor, unit_normal
    d = tiny.make_model_dir(tmp_path, "B")
    _, _, spec = load_model_config(d)
    specs = Model(spec).tensor_specs()
    stored = load_weights(d, specs, torch.bfloat16, "cpu")
    seed = tiny.CONFIGS["B"][1]
    direct = random_tensors(specs, seed, torch.bfloat16, tiny.INIT_SCALE)
    assert set(direct) == set(stored) and all(torch.equal(direct[k], stored[k]) for k in stored)
    cfg, _ = P.load(d)
    plain = P.random_weights(cfg, seed, tiny.INIT_SCALE, torch.bfloat16)
    assert set(plain) == set(stored) and all(torch.equal(plain[k], stored[k].float()) for k in stored)
    whole = unit_normal(5, "layers.7.mlp.up_proj.weight", 3000, "cpu")
    piece = unit_normal(5, "layers.7.mlp.up_proj.weight", 1000, "cpu", first=1500)
    assert torch.equal(whole[1500:2500], piece)
    assert not torch.equal(whole[:1000], unit_normal(5, "layers.8.mlp.up_proj.weight", 1000, "cpu"))
    big = unit_normal(11, "embed_tokens.weight", 400_000, "cpu")
    assert abs(float(big.mean())) < 5e-3 and abs(float(big.std()) - 1.0) < 5e-3 and float(big.abs().max()) < 6.0
    norm = draw_tensor(2, "norm.weight", specs["norm.weight"], torch.float32, "cpu")
    assert abs(float(norm.mean()) - 1.0) < 5e-3 and 0.005 < float(norm.std()) < 0.015


def test_a_scratch_buffer_that_a_graph_may_hold_is_never_given_back():
    """A captured step has its scratch buffer's address baked in.  When a later call needs more, the old buffer is
    kept alive beside the new one instead of going back to the allocator, and growth at least doubles."""
    from zedinfer_b200 import ops
    key = ("test_scratch", "cpu")
    ops._scratch.pop(key, None)
    first = ops._grown_scratch(key, 100, "cpu")
    assert ops._grown_scratch(key, 80, "cpu") is first
    second = ops._grown_scratch(key, 101, "cpu")
    assert second is not first and second.numel() >= 200
    assert any(t is first for t in ops._retired)
    ops._scratch.pop(key, None)
