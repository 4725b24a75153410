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


def test_a_tensor_nobody_asked_for_is_a_warning_unless_strict(tmp_path, capsys):
    """Older exports carry `rotary_emb.inv_freq` buffers: everything needed is there, so the
    model loads and the extra names are listed on stderr; `strict` makes them an error."""
    d = str(tmp_path / "a")
    write_random_model(TINY_A, 0, d)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.read(n).clone() for n in f.names()}
    f.close()
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(32)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    _, model = build_model(TINY_A)
    load_model(model, CheckpointSource(d), torch.float32, "cpu")
    err = capsys.readouterr().err
    assert "rotary_emb.inv_freq" in err and "no part of the model asked for" in err
    _, ref = build_model(TINY_A)
    load_model(ref, RandomSource(ref.tensor_specs(), 0), torch.float32, "cpu")
    assert torch.equal(model.blocks[0].mixer.w_qkv, ref.blocks[0].mixer.w_qkv)
    _, model = build_model(TINY_A)
    with pytest.raises(WeightError, match="1 unexpected") as ei:
        load_model(model, CheckpointSource(d), torch.float32, "cpu", strict=True)
    assert ei.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"] and not ei.value.missing


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


def _draw_with_python_integers(seed, name, i, init):
    """A third statement of the random-weights function, in plain Python integers, for a few
    single elements."""
    import hashlib
    import numpy as np
    d = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    k1, k2 = int.from_bytes(d[:4], "little"), int.from_bytes(d[4:8], "little")
    M = 0xFFFFFFFF

    def mix(x):
        x ^= x >> 16
        x = (x * 0x7FEB352D) & M
        x ^= x >> 15
        x = (x * 0x846CA68B) & M
        return x ^ (x >> 16)

    s = mix(mix((i & M) ^ k1) ^ (i >> 32) ^ k2)
    n = -6138
    for c in (0x9E3779B9, 0x85EBCA6B, 0xC2B2AE35, 0x27D4EB2F):
        w = mix(s ^ c)
        n += (w & 1023) + ((w >> 10) & 1023) + ((w >> 20) & 1023)
    z = np.float32(n) * np.float32(1.0 / np.sqrt(np.float64(1048575.0)))
    v = np.float32(1.0) + np.float32(0.05) * z if init == "norm" else np.float32(0.02) * z
    return float(torch.tensor(float(v), dtype=torch.float32).to(torch.bfloat16))


def test_counter_based_weights_three_statements_agree():
    """The engine's generator (torch twin of the CUDA kernel), the plain model's restatement and
    plain Python integers give the same bfloat16 values for (seed, name, index), also beyond
    2^32 elements and whatever the chunking."""
    import plain_model
    from ninfer_amd_mi50_b200.weights import counter_rng
    for seed, name, init in ((0, "model.embed_tokens.weight", "linear"), (7, "model.norm.weight", "norm")):
        keys = counter_rng.tensor_keys(seed, name)
        ours = counter_rng.draw(0, 5000, keys, init)
        plain = plain_model.plain_random_tensor(seed, name, (50, 100), init).reshape(-1)
        assert torch.equal(ours, plain)
        for i in (0, 1, 77, 4999):
            assert ours[i].item() == _draw_with_python_integers(seed, name, i, init)
        far = (1 << 33) + 12345
        assert counter_rng.draw(far, 3, keys, init)[2].item() == _draw_with_python_integers(seed, name, far + 2, init)
        # the value of an element does not depend on where a chunk begins
        assert torch.equal(counter_rng.draw(1000, 50, keys, init), ours[1000:1050])
        out = torch.empty(5000, dtype=torch.bfloat16)
        assert torch.equal(counter_rng.fill(out, keys, init).float(), ours)
    z = counter_rng.draw(0, 1 << 18, counter_rng.tensor_keys(3, "x"), "linear") / 0.02
    assert abs(z.mean().item()) < 0.01 and abs(z.std().item() - 1) < 0.01 and z.abs().max().item() < 6


def test_plain_random_weights_name_the_tensors_of_a_written_folder(tmp_path):
    """The plain model can rebuild, from configuration and seed alone, exactly the tensors that
    `write_random_model` puts into a folder: same names, same shapes, same bits."""
    import plain_model
    for cfg, seed in ((TINY_A, 0), (TINY_B, 1)):
        d = str(tmp_path / f"m{seed}")
        write_random_model(cfg, seed, d)
        pcfg, stored = plain_model.read_model_folder(d)
        drawn = plain_model.RandomWeights(pcfg, seed)
        assert sorted(drawn.keys()) == sorted(stored)
        for name in list(stored)[::7] + ["model.norm.weight"]:
            assert torch.equal(drawn[name], stored[name]), name
