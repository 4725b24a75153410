"""Weights: the safetensors reader and writer, binding by name, and the one error that lists
everything wrong with a checkpoint."""

import json
import os
import struct

import pytest
import torch

from tiny_configs import TINY_A, TINY_B

from ninfer_amd_mi50_b200.engine import build_model
from ninfer_amd_mi50_b200.weights import (CheckpointSource, RandomSource, SafetensorsError,
                                          SafetensorsFile, WeightError, check_specs, held_dtype,
                                          load_model, write_random_model, write_safetensors)


def test_safetensors_round_trip_and_foreign_reader(tmp_path):
    p = str(tmp_path / "x.safetensors")
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32),
         "c": torch.randn(2, 2, 2)}
    write_safetensors(p, t.items(), metadata={"k": "v"})
    f = SafetensorsFile(p)
    assert set(f.names()) == set(t) and f.metadata == {"k": "v"}
    for n, v in t.items():
        assert torch.equal(f.read(n), v)
    from safetensors import safe_open          # an independent reader agrees
    with safe_open(p, framework="pt") as g:
        for n, v in t.items():
            assert torch.equal(g.get_tensor(n), v)


def test_safetensors_errors(tmp_path):
    with pytest.raises(SafetensorsError, match="not found"):
        SafetensorsFile(str(tmp_path / "none.safetensors"))
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 2) + b"{]")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)      # 8 of 16 bytes
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr)
    with pytest.raises(SafetensorsError, match="malformed"):
        SafetensorsFile(str(p))


def test_random_model_folder_loads_and_is_seeded(tmp_path):
    a, b, c = (str(tmp_path / n) for n in "abc")
    write_random_model(TINY_A, 0, a)
    write_random_model(TINY_A, 0, b)
    write_random_model(TINY_A, 1, c)
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    name = "model.layers.1.mlp.experts.3.up_proj.weight"
    assert torch.equal(fa.read(name), fb.read(name)) and not torch.equal(fa.read(name), fc.read(name))
    w = fa.read(name).float()
    assert w.shape == (128, 256) and abs(w.std().item() - 0.02) < 0.002
    n = fa.read("model.norm.weight").float()
    assert abs(n.mean().item() - 1.0) < 0.02 and 0.03 < n.std().item() < 0.07
    assert json.load(open(os.path.join(a, "config.json")))["num_experts"] == 8
    _, model = build_model(TINY_A)
    load_model(model, CheckpointSource(a), torch.float32, "cpu")
    assert model.blocks[0].mixer.w_qkv.shape == (4 * 64 + 2 * 2 * 64, 256)
    assert model.blocks[0].feed_forward.w13.shape == (8, 256, 256)
    assert model.blocks[0].feed_forward.w_router.shape == (9, 256)      # router rows + the shared gate
    assert model.head is not model.embedding


def test_tied_head_shares_the_embedding(tmp_path):
    d = str(tmp_path / "b")
    write_random_model(TINY_B, 1, d)
    assert "lm_head.weight" not in SafetensorsFile(os.path.join(d, "model.safetensors")).names()
    _, model = build_model(TINY_B)
    load_model(model, CheckpointSource(d), torch.bfloat16, "cpu")
    assert model.head is model.embedding and model.embedding.dtype == torch.bfloat16
    assert model.final_norm.weight.dtype == torch.float32       # vectors stay 32-bit
    assert model.blocks[0].feed_forward.w_router.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = str(tmp_path / "a")
    write_random_model(TINY_A, 0, d)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.read(n).clone() for n in f.names()}
    f.close()
    del tensors["model.layers.0.self_attn.k_proj.bias"]
    del tensors["model.layers.1.mlp.experts.7.down_proj.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(32)
    tensors["model.embed_tokens.weight"] = torch.zeros(1000, 256, dtype=torch.bfloat16)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    _, model = build_model(TINY_A)
    with pytest.raises(WeightError) as ei:
        load_model(model, CheckpointSource(d), torch.float32, "cpu")
    e = ei.value
    assert e.missing == ["model.layers.0.self_attn.k_proj.bias", "model.layers.1.mlp.experts.7.down_proj.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert e.wrong_shape == [("model.embed_tokens.weight", (1024, 256), (1000, 256))]
    msg = str(e)
    for piece in ("2 missing", "k_proj.bias", "1 unexpected", "inv_freq", "wrong shape", "[1000, 256]"):
        assert piece in msg


def test_no_checkpoint_in_folder(tmp_path):
    with pytest.raises(WeightError, match="no model.safetensors"):
        CheckpointSource(str(tmp_path))


def test_sharded_checkpoint_through_index(tmp_path):
    d = str(tmp_path / "a")
    write_random_model(TINY_A, 0, d)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    names = f.names()
    half = len(names) // 2
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), [(n, f.read(n)) for n in names[:half]])
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), [(n, f.read(n)) for n in names[half:]])
    wm = {n: "model-00001-of-00002.safetensors" for n in names[:half]}
    wm.update({n: "model-00002-of-00002.safetensors" for n in names[half:]})
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    f.close()
    os.remove(os.path.join(d, "model.safetensors"))
    _, model = build_model(TINY_A)
    load_model(model, CheckpointSource(d), torch.float32, "cpu")


def test_stored_dtypes_and_roles(tmp_path):
    assert held_dtype("matrix", torch.bfloat16) == torch.bfloat16
    assert held_dtype("vector", torch.bfloat16) == torch.float32
    assert held_dtype("router", torch.bfloat16) == torch.float32
    assert held_dtype("table", torch.bfloat16) == torch.int32
    # a model stored in float32 loads into either engine dtype
    d = str(tmp_path / "f32")
    write_random_model(TINY_A, 0, d, store_dtype="float32")
    _, model = build_model(TINY_A)
    load_model(model, CheckpointSource(d), torch.bfloat16, "cpu")
    assert model.blocks[0].mixer.w_o.dtype == torch.bfloat16


def test_random_source_matches_written_folder(tmp_path):
    d = str(tmp_path / "a")
    write_random_model(TINY_A, 5, d)
    _, m1 = build_model(TINY_A)
    load_model(m1, CheckpointSource(d), torch.float32, "cpu")
    _, m2 = build_model(TINY_A)
    load_model(m2, RandomSource(m2.tensor_specs(), 5), torch.float32, "cpu")
    assert torch.equal(m1.blocks[1].feed_forward.w2, m2.blocks[1].feed_forward.w2)
    assert torch.equal(m1.final_norm.weight, m2.final_norm.weight)
