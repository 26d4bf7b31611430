"""Makes tests/golden/reference_cpu.json from the reference's own code, where that code runs on a CPU.

The reference's forward pass needs a CUDA device (its kernels are Triton), so it cannot be the
oracle here.  Three pieces of it do run on a CPU and anchor the plain implementation:

* ``model.rope_tables`` (engine/model.py:78-93): the bfloat16 cos/sin tables;
* ``model.Model`` (engine/model.py:96-130): the fused q/k/v and gate/up layouts and the tied head,
  loaded from a tiny random checkpoint written by this library;
* ``kernels.attention.reference_attention`` (engine/kernels/attention.py:221-242): causal attention
  with a start offset over a cache, the mask of the decode kernel.

Run once, by hand, where the reference is mounted:

    python tests/golden/make_golden.py /path/to/reference

The outputs are small (a few KB) and committed; tests/test_golden.py compares the plain
implementation with them and never imports the reference.
"""

import json
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

CONFIG = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=160, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256, rms_norm_eps=1e-6,
              rope_theta=10000.0, tie_word_embeddings=True)


def main(reference: str) -> None:
    sys.path.insert(0, str(Path(reference) / "engine"))
    import model as ref_model
    from kernels.attention import reference_attention
    from starter_b200.config import config_from_dict
    from starter_b200.weights import write_model_folder

    out = {"config": CONFIG}
    with tempfile.TemporaryDirectory() as folder:
        write_model_folder(config_from_dict(CONFIG), 0, folder)
        m = ref_model.Model(folder, device="cpu", max_pos=40)
    cos, sin = m.cos, m.sin  # [40, 16] bfloat16
    out["rope"] = {"theta": CONFIG["rope_theta"], "head_dim": 16, "positions": [0, 1, 7, 39],
                   "cos": cos[[0, 1, 7, 39]].float().tolist(), "sin": sin[[0, 1, 7, 39]].float().tolist()}
    layer = m.layers[1]
    out["fused"] = {
        "wqkv_shape": list(layer.wqkv.shape), "wgu_shape": list(layer.wgu.shape),
        "wqkv_row_sums": layer.wqkv.float().sum(1)[[0, 63, 64, 95, 96, 127]].tolist(),
        "wgu_row_sums": layer.wgu.float().sum(1)[[0, 159, 160, 319]].tolist(),
        "tied": bool(m.lm_head is m.embed), "scale": m.scale,
    }
    g = torch.Generator().manual_seed(5)
    B, HQ, HKV, D, R, cap = 2, 4, 2, 16, 3, 24
    q = torch.randn(B, HQ, R, D, generator=g)
    k = torch.randn(B, HKV, cap, D, generator=g)
    v = torch.randn(B, HKV, cap, D, generator=g)
    pos = torch.tensor([5, 0])
    att = reference_attention(q, k, v, pos, R, 0.25)  # [B, R, HQ, D]
    out["attention"] = {"seed": 5, "B": B, "HQ": HQ, "HKV": HKV, "D": D, "R": R, "cap": cap, "pos": pos.tolist(),
                        "scale": 0.25, "out": att.tolist()}
    path = Path(__file__).resolve().parent / "reference_cpu.json"
    path.write_text(json.dumps(out))
    print(f"wrote {path} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/reference   (the folder that holds engine/)")
    main(sys.argv[1])
