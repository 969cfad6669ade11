"""Safetensors I/O, loading by name with one listing error, random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

import helpers
from helpers import TINY_A, TINY_B
from pulsar_b200.config import config_from_dict
from pulsar_b200.models import build_model
from pulsar_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights, random_tensors,
                                 write_model_folder, write_safetensors)


def test_writer_is_read_by_the_safetensors_package_and_back(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(0)
    tensors = {"a.weight": torch.randn(3, 5, generator=g), "b": torch.randn(7, generator=g).bfloat16(),
               "c": torch.arange(6, dtype=torch.int32).view(2, 3), "empty": torch.zeros(0, 4)}
    mine = str(tmp_path / "mine.safetensors")
    write_safetensors(mine, tensors.items(), metadata={"k": "v"})
    with safe_open(mine, "pt") as f:
        assert sorted(f.keys()) == sorted(tensors)
        for n, t in tensors.items():
            assert torch.equal(f.get_tensor(n), t)
    theirs = str(tmp_path / "theirs.safetensors")
    save_file(tensors, theirs)
    sf = SafetensorsFile(theirs)
    for n, t in tensors.items():
        got = sf.tensor(n)
        assert got.dtype == t.dtype and torch.equal(got, t)
    sf.close()


def test_broken_files_are_refused(tmp_path):
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"\x05\x00")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFile(str(p))
    head = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(head).to_bytes(8, "little") + head + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="do not match"):
        SafetensorsFile(str(p))


def _folder(tmp_path, raw, seed=0, **kw):
    return helpers.make_folder(tmp_path, raw, seed, **kw)


def test_loads_every_tensor_by_name_and_fuses(tmp_path):
    d = _folder(tmp_path, TINY_B, 1)
    cfg, w = helpers.read_folder(d)
    model = build_model(config_from_dict(cfg), torch.float32)
    load_weights(model, d, "cpu")
    blk = model.blocks[2]
    p = "model.layers.2.self_attn."
    assert torch.equal(blk.mixer.w_qkv, torch.cat([w[p + "q_proj.weight"], w[p + "k_proj.weight"], w[p + "v_proj.weight"]]))
    assert torch.equal(blk.feed_forward.w_gate_up[:320], w["model.layers.2.mlp.gate_proj.weight"])
    assert torch.equal(blk.feed_forward.w_gate_up[320:], w["model.layers.2.mlp.up_proj.weight"])
    assert not model.tied and torch.equal(model.head, w["lm_head.weight"])
    assert torch.equal(model.final_norm.weight, w["model.norm.weight"])


def test_dtypes_held(tmp_path):
    d = _folder(tmp_path, TINY_A, 0, store_dtype=torch.bfloat16)
    cfg, w = helpers.read_folder(d)
    assert w["model.norm.weight"].dtype == torch.bfloat16
    model = build_model(config_from_dict(cfg), torch.bfloat16)
    load_weights(model, d, "cpu")
    assert model.embed.dtype == torch.bfloat16 and model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    # norm weights are held in float32: exact for values stored in bfloat16
    assert model.final_norm.weight.dtype == torch.float32
    assert torch.equal(model.final_norm.weight, w["model.norm.weight"].float())
    assert model.tied and model.head is model.embed
    # a folder stored in 32-bit: vectors stay 32-bit, matrices are held in the compute dtype
    d32 = _folder(tmp_path / "f32", TINY_A, 0)
    m16 = build_model(config_from_dict(cfg), torch.bfloat16)
    load_weights(m16, d32, "cpu")
    _, w32 = helpers.read_folder(d32)
    assert torch.equal(m16.final_norm.weight, w32["model.norm.weight"])
    assert torch.equal(m16.embed, w32["model.embed_tokens.weight"].bfloat16())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = _folder(tmp_path, TINY_B, 1)
    cfg, w = helpers.read_folder(d)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.layers.0.self_attn.k_norm.weight"]
    w["model.layers.7.extra.weight"] = torch.zeros(2)
    w["model.layers.2.self_attn.q_proj.weight"] = torch.zeros(96, 256)       # transposed
    w["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), w.items())
    model = build_model(config_from_dict(cfg), torch.float32)
    with pytest.raises(WeightError) as e:
        load_weights(model, d, "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.layers.0.self_attn.k_norm.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert len(err.wrong) == 2
    msg = str(err)
    for piece in ("missing (2)", "unexpected (1)", "model.layers.7.extra.weight", "expected shape [256, 96], found [96, 256]",
                  "model.norm.weight: expected a floating-point tensor"):
        assert piece in msg, msg


def test_tied_and_untied_head_rules(tmp_path):
    # tie_word_embeddings true: a head tensor is unexpected
    d = _folder(tmp_path / "a", TINY_A, 0)
    cfg, w = helpers.read_folder(d)
    w["lm_head.weight"] = torch.zeros(256, 64)
    write_safetensors(os.path.join(d, "model.safetensors"), w.items())
    with pytest.raises(WeightError, match="unexpected"):
        load_weights(build_model(config_from_dict(cfg), torch.float32), d, "cpu")
    # tie_word_embeddings false: the head tensor is required
    d = _folder(tmp_path / "b", TINY_B, 1)
    cfg, w = helpers.read_folder(d)
    del w["lm_head.weight"]
    write_safetensors(os.path.join(d, "model.safetensors"), w.items())
    with pytest.raises(WeightError, match="missing"):
        load_weights(build_model(config_from_dict(cfg), torch.float32), d, "cpu")
    # key absent: presence of the tensor decides (pulsar-core/src/model/qwen3.cpp:51-53)
    raw = dict(TINY_B)
    del raw["tie_word_embeddings"]
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(raw, f)
    m = build_model(config_from_dict(raw), torch.float32)
    load_weights(m, d, "cpu")
    assert m.tied and m.head is m.embed


def test_sharded_folder_and_duplicates(tmp_path):
    d = _folder(tmp_path, TINY_A, 0)
    cfg, w = helpers.read_folder(d)
    names = sorted(w)
    half = len(names) // 2
    os.remove(os.path.join(d, "model.safetensors"))
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), [(n, w[n]) for n in names[:half]])
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), [(n, w[n]) for n in names[half:]])
    weight_map = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                  for i, n in enumerate(names)}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": weight_map}, f)
    m = build_model(config_from_dict(cfg), torch.float32)
    load_weights(m, d, "cpu")
    assert torch.equal(m.embed, w["model.embed_tokens.weight"])
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), [(n, w[n]) for n in names[half - 1:]])
    with pytest.raises(SafetensorsError, match="appears in"):
        load_weights(build_model(config_from_dict(cfg), torch.float32), d, "cpu")


def test_random_weights_are_a_function_of_config_and_seed(tmp_path):
    a = dict(random_tensors(build_model(config_from_dict(TINY_A), torch.float32), 0, 0.02))
    b = dict(random_tensors(build_model(config_from_dict(TINY_A), torch.float32), 0, 0.02))
    c = dict(random_tensors(build_model(config_from_dict(TINY_A), torch.float32), 1, 0.02))
    assert list(a)[0] == "model.embed_tokens.weight" and list(a)[-1] == "model.norm.weight"
    assert all(torch.equal(a[n], b[n]) for n in a) and not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    emb, norm = a["model.embed_tokens.weight"], a["model.layers.1.input_layernorm.weight"]
    assert abs(float(emb.std()) - 0.02) < 0.002 and abs(float(norm.mean()) - 1.0) < 0.05 and 0.05 < float(norm.std()) < 0.15
    d = write_model_folder(config_from_dict(TINY_B), str(tmp_path / "m"), 1)
    cfg, w = helpers.read_folder(d)
    assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["hidden_size"] == 96 and "lm_head.weight" in w
    assert abs(float(w["model.layers.0.mlp.down_proj.weight"].std()) - 0.05) < 0.005
