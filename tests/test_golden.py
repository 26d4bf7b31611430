"""The plain implementation against outputs of the reference's own code (the pieces that run on a CPU).

tests/golden/make_golden.py made tests/golden/reference_cpu.json from the reference's rope tables,
its weight fusion and its attention oracle; this test never imports the reference."""

import json
import tempfile
from pathlib import Path

import torch

from plain import qwen3_plain as plain
from starter_b200.config import config_from_dict
from starter_b200.weights import write_model_folder

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "reference_cpu.json").read_text())


def test_rope_tables_match_the_reference_bit_for_bit():
    g = GOLDEN["rope"]
    cos, sin = plain.rope_tables(g["theta"], g["head_dim"], 40, plain._rounder("bfloat16"))
    assert torch.equal(cos[g["positions"]], torch.tensor(g["cos"]))
    assert torch.equal(sin[g["positions"]], torch.tensor(g["sin"]))


def test_fused_weight_layout_matches_the_reference():
    with tempfile.TemporaryDirectory() as folder:
        write_model_folder(config_from_dict(GOLDEN["config"]), 0, folder)
        cfg, t = plain.read_folder(folder)
    p = "model.layers.1."
    wqkv = torch.cat([t[p + "self_attn.q_proj.weight"], t[p + "self_attn.k_proj.weight"], t[p + "self_attn.v_proj.weight"]])
    wgu = torch.cat([t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"]])
    f = GOLDEN["fused"]
    assert list(wqkv.shape) == f["wqkv_shape"] and list(wgu.shape) == f["wgu_shape"]
    assert torch.allclose(wqkv.sum(1)[[0, 63, 64, 95, 96, 127]], torch.tensor(f["wqkv_row_sums"]), atol=1e-6)
    assert torch.allclose(wgu.sum(1)[[0, 159, 160, 319]], torch.tensor(f["wgu_row_sums"]), atol=1e-6)
    assert f["tied"] and plain.lm_head_weight(cfg, t) is t["model.embed_tokens.weight"]
    assert abs(f["scale"] - 1.0 / plain.head_dim_of(cfg) ** 0.5) < 1e-12


def test_attention_mask_and_grouping_match_the_reference_oracle():
    """R new rows on a cache that already holds pos tokens: the plain attention over the whole
    sequence must give the reference's rows for the last R positions."""
    a = GOLDEN["attention"]
    g = torch.Generator().manual_seed(a["seed"])
    B, HQ, HKV, D, R, cap = a["B"], a["HQ"], a["HKV"], a["D"], a["R"], a["cap"]
    q = torch.randn(B, HQ, R, D, generator=g)
    k = torch.randn(B, HKV, cap, D, generator=g)
    v = torch.randn(B, HKV, cap, D, generator=g)
    want = torch.tensor(a["out"])
    for b, pos in enumerate(a["pos"]):
        T = pos + R
        q_full = torch.zeros(T, HQ, D)
        q_full[pos:] = q[b].permute(1, 0, 2)
        got = plain.attention(q_full, k[b, :, :T].permute(1, 0, 2), v[b, :, :T].permute(1, 0, 2), a["scale"], None,
                              plain._rounder("float32"))
        assert torch.allclose(got[pos:].view(R, HQ, D), want[b], atol=2e-6)
