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


# ---- checkpoints in several files (engine/model.py:67-75 reads every *.safetensors of the folder, sorted) ----

def _split_into_shards(src_folder, dst_folder, groups):
    """Write the tensors of ``src_folder`` into len(groups) + 1 shard files: ``groups`` are lists of
    predicates' names; what no group takes goes to the last file."""
    tensors = read_all(src_folder / "model.safetensors")
    (dst_folder / "config.json").write_text((src_folder / "config.json").read_text())
    taken = set()
    n = len(groups) + 1
    for i, names in enumerate(groups):
        save_file({k: tensors[k] for k in names}, str(dst_folder / f"model-{i + 1:05d}-of-{n:05d}.safetensors"))
        taken |= set(names)
    save_file({k: v for k, v in tensors.items() if k not in taken}, str(dst_folder / f"model-{n:05d}-of-{n:05d}.safetensors"))
    return tensors


def _odd_split(tensors):
    """The embedding alone in one file; layer 1 cut across two files."""
    layer1 = sorted(k for k in tensors if k.startswith("model.layers.1."))
    second = [k for k in tensors if k.startswith("model.layers.0.")] + layer1[:len(layer1) // 2]
    return [["model.embed_tokens.weight"], second]


def test_sharded_folder_gives_the_same_logits(tiny_folders, tmp_path):
    from conftest import random_tokens
    from helpers import make_session, run_whole
    tensors = read_all(tiny_folders["B"] / "model.safetensors")
    _split_into_shards(tiny_folders["B"], tmp_path, _odd_split(tensors))
    assert len(list(tmp_path.glob("*.safetensors"))) == 3
    seqs = random_tokens(TINY["B"]["vocab_size"], (5, 70, 33), seed=3)
    outs = []
    for folder in (tiny_folders["B"], tmp_path):
        sess = make_session(folder, "float32", ops=EmulatedOps(), max_tokens=64 * 6, max_seqs=3)
        outs.append(run_whole(sess, seqs, together=True))
    assert all(torch.equal(a, b) for a, b in zip(*outs))


def test_sharded_folder_faults_are_listed_together(tiny_folders, tmp_path):
    tensors = _split_into_shards(tiny_folders["B"], tmp_path, _odd_split(read_all(tiny_folders["B"] / "model.safetensors")))
    # a fourth file: one tensor a second time, one that nobody wants; and one tensor goes missing from shard 2
    save_file({"model.embed_tokens.weight": tensors["model.embed_tokens.weight"],
               "model.layers.0.mlp.gate_proj.bias": torch.zeros(224, dtype=torch.bfloat16)},
              str(tmp_path / "model-extra.safetensors"))
    second = read_all(tmp_path / "model-00002-of-00003.safetensors")
    del second["model.layers.0.self_attn.k_norm.weight"]
    save_file(second, str(tmp_path / "model-00002-of-00003.safetensors"))
    with pytest.raises(WeightsError) as err:
        DecoderModel.from_folder(tmp_path, runtime())
    text = str(err.value)
    assert "4 safetensors files" in text
    assert "missing (1)" in text and "model.layers.0.self_attn.k_norm.weight" in text
    assert "unexpected (1)" in text and "gate_proj.bias" in text
    assert "stored more than once (1)" in text
    assert "model.embed_tokens.weight in model-00001-of-00003.safetensors and model-extra.safetensors" in text


def test_folder_without_shards(tmp_path, tiny_folders):
    (tmp_path / "config.json").write_text((tiny_folders["A"] / "config.json").read_text())
    with pytest.raises(FileNotFoundError, match=r"no \*\.safetensors file"):
        DecoderModel.from_folder(tmp_path, runtime())


def test_random_weights_in_shards_equal_the_single_file(tmp_path):
    cfg = config_from_dict(tiny_raw("B"))
    write_model_folder(cfg, 5, tmp_path / "one")
    write_model_folder(cfg, 5, tmp_path / "three", shards=3)
    files = sorted((tmp_path / "three").glob("*.safetensors"))
    assert [f.name for f in files] == [f"model-0000{i}-of-00003.safetensors" for i in (1, 2, 3)]
    one = read_all(tmp_path / "one" / "model.safetensors")
    three = {}
    for f in files:
        part = read_all(f)
        assert part and not (part.keys() & three.keys())
        three.update(part)
    assert one.keys() == three.keys() and all(torch.equal(one[k], three[k]) for k in one)
    a = DecoderModel.from_folder(tmp_path / "one", runtime())
    b = DecoderModel.from_folder(tmp_path / "three", runtime())
    assert torch.equal(a.blocks[2].ff.w_gate_up, b.blocks[2].ff.w_gate_up) and torch.equal(a.lm_head, b.lm_head)
