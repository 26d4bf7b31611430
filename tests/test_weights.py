"""Weights by name: the container, the single error that lists every fault, random weights."""

import json
import struct

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import save_file

from conftest import TINY, tiny_raw
from emulated_ops import EmulatedOps
from starter_b200.config import config_from_dict
from starter_b200.engine.context import Runtime
from starter_b200.engine.model import DecoderModel
from starter_b200.weights import (RandomSource, SafetensorsError, SafetensorsFile, WeightsError, write_model_folder,
                                  write_safetensors)


def runtime(dtype=torch.bfloat16):
    return Runtime(dtype=dtype, device=torch.device("cpu"), ops=EmulatedOps())


def read_all(path):
    with safe_open(str(path), framework="pt") as f:
        return {k: f.get_tensor(k) for k in f.keys()}


def test_container_round_trip_agrees_with_the_safetensors_library(tmp_path):
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
               "c": torch.randn(4), "empty": torch.zeros(0, 3)}
    write_safetensors(tmp_path / "mine.safetensors", [(k, (v.dtype, tuple(v.shape))) for k, v in tensors.items()],
                      tensors.__getitem__)
    theirs = read_all(tmp_path / "mine.safetensors")
    save_file(tensors, str(tmp_path / "theirs.safetensors"))
    mine = SafetensorsFile(tmp_path / "theirs.safetensors")
    for k, v in tensors.items():
        assert torch.equal(theirs[k], v) and torch.equal(mine.get(k), v) and mine.entries[k] == (v.dtype, tuple(v.shape))
    mine.close()


def test_malformed_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    header = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    with pytest.raises(FileNotFoundError):
        SafetensorsFile(tmp_path / "absent.safetensors")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tiny_folders, tmp_path):
    tensors = read_all(tiny_folders["B"] / "model.safetensors")
    del tensors["model.layers.1.self_attn.q_norm.weight"], tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192, dtype=torch.bfloat16)
    tensors["model.layers.2.mlp.down_proj.weight"] = torch.zeros(96, 200, dtype=torch.bfloat16)
    (tmp_path / "config.json").write_text((tiny_folders["B"] / "config.json").read_text())
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightsError) as err:
        DecoderModel.from_folder(tmp_path, runtime())
    text = str(err.value)
    assert "missing (2)" in text and "model.layers.1.self_attn.q_norm.weight" in text and "lm_head.weight" in text
    assert "unexpected (1)" in text and "q_proj.bias" in text
    assert "wrong shape (1)" in text and "[96, 200]" in text and "[96, 224]" in text


def test_tied_and_untied_heads(tiny_folders, tmp_path):
    a = DecoderModel.from_folder(tiny_folders["A"], runtime())
    assert a.lm_head is a.embedding                      # engine/model.py:103-107
    tensors = read_all(tiny_folders["A"] / "model.safetensors")
    tensors["lm_head.weight"] = torch.ones(256, 64, dtype=torch.bfloat16)
    (tmp_path / "config.json").write_text((tiny_folders["A"] / "config.json").read_text())
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with_head = DecoderModel.from_folder(tmp_path, runtime())
    assert with_head.lm_head is not with_head.embedding and float(with_head.lm_head[0, 0]) == 1.0


def test_dtypes_kept(tiny_folders, tmp_path):
    tensors = read_all(tiny_folders["A"] / "model.safetensors")
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() + 1e-4   # stored in 32-bit
    (tmp_path / "config.json").write_text((tiny_folders["A"] / "config.json").read_text())
    save_file(tensors, str(tmp_path / "model.safetensors"))
    bf = DecoderModel.from_folder(tmp_path, runtime(torch.bfloat16))
    assert bf.final_norm.weight.dtype == torch.float32 and bf.embedding.dtype == torch.bfloat16
    assert torch.equal(bf.final_norm.weight, tensors["model.norm.weight"])
    f32 = DecoderModel.from_folder(tmp_path, runtime(torch.float32))
    assert f32.embedding.dtype == torch.float32 and f32.blocks[0].mixer.w_qkv.dtype == torch.float32
    assert torch.equal(f32.embedding, tensors["model.embed_tokens.weight"].float())


def test_fused_layouts(tiny_folders):
    """q, k, v rows one after another; gate rows before up rows (engine/model.py:112-116)."""
    t = read_all(tiny_folders["B"] / "model.safetensors")
    m = DecoderModel.from_folder(tiny_folders["B"], runtime())
    p = "model.layers.1."
    assert torch.equal(m.blocks[1].mixer.w_qkv, torch.cat([t[p + "self_attn.q_proj.weight"], t[p + "self_attn.k_proj.weight"],
                                                           t[p + "self_attn.v_proj.weight"]]))
    assert torch.equal(m.blocks[1].ff.w_gate_up, torch.cat([t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"]]))


def test_random_weights_are_a_function_of_seed_and_name(tmp_path):
    cfg = config_from_dict(tiny_raw("A"))
    write_model_folder(cfg, 7, tmp_path / "a")
    write_model_folder(cfg, 7, tmp_path / "b")
    write_model_folder(cfg, 8, tmp_path / "c")
    a, b, c = (read_all(tmp_path / n / "model.safetensors") for n in "abc")
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert "lm_head.weight" not in a                      # tied: the head is the embedding
    w = a["model.layers.0.mlp.up_proj.weight"].float()
    n = a["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(n.mean()) - 1.0) < 0.05
    bigger = config_from_dict(dict(tiny_raw("A"), num_hidden_layers=3))
    src = RandomSource(bigger, 7)
    assert torch.equal(src.get("model.layers.0.mlp.up_proj.weight"), a["model.layers.0.mlp.up_proj.weight"])
