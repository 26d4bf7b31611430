"""Makes tests/golden/reference_gpu.safetensors from the reference's own kernels and forward pass.

The reference's kernels are Triton and its forward pass (``Plan.prefill`` / ``Plan.decode``,
engine/model.py:280-331) needs a CUDA device.  This script runs them there once, on small seeded
inputs, and stores their outputs (a few tens of KB); tests/test_golden_gpu_outputs.py rebuilds the
same inputs from the same seeds and holds the plain implementation (tests/plain/qwen3_plain.py,
bfloat16 mode) against the stored outputs: bit for bit where the reference's own tests are bit-exact
(RMSNorm, residual add + norm, SwiGLU, q/k norm + rotary + cache write: tests/test_kernels.py:22-57,
90-99 there), within the reference's own bound for logits (0.03 x the largest logit,
tests/test_engine.py:50-53 there) and for attention over a cache.  The test never imports the reference.

Run by hand on a machine with a CUDA device, with the path of the reference's checkout:

    python tests/golden/make_golden_gpu.py /path/to/reference

What is covered: ``kernels.rms_norm``, ``kernels.add_rms_norm``, ``kernels.swiglu``,
``kernels.qk_norm_rope_cache``, ``kernels.DecodeAttention``, ``model.Plan.prefill`` and
``model.Plan.decode`` on the reference's own tiny shape (tests/tiny.py:11-20 there: 2 layers,
hidden 256, 8 query and 2 key/value heads of 128, intermediate 512, vocabulary 1,024).
"""

import os
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

TINY = dict(architectures=["Qwen3ForCausalLM"], hidden_size=256, intermediate_size=512, num_hidden_layers=2,
            num_attention_heads=8, num_key_value_heads=2, head_dim=128, vocab_size=1024, rms_norm_eps=1e-6,
            rope_theta=5000000.0, tie_word_embeddings=True)
TINY_SEED = 0
EPS = 1e-6
PROMPT_LEN, DECODE_STEPS = 37, 3


def golden_inputs():
    """Every input of the stored cases, from fixed seeds (CPU generator), as bfloat16 / int tensors."""
    g = torch.Generator().manual_seed(123)
    bf = torch.bfloat16

    def rn(*shape, scale=1.0, shift=0.0):
        return (torch.randn(*shape, generator=g) * scale + shift).to(bf)

    ins = {
        "norm.x": rn(5, 256, scale=2.0), "norm.w": rn(256, scale=0.1, shift=1.0),
        "addnorm.x": rn(5, 256, scale=2.0), "addnorm.y": rn(5, 256), "addnorm.w": rn(256, scale=0.1, shift=1.0),
        "swiglu.gu": rn(5, 2 * 384, scale=3.0),
        # q/k norm + rotary + cache write: B=2 sequences of T=3 new rows at positions 5.. and 0..
        "rope.qkv": rn(6, (4 + 2 * 2) * 128, scale=1.5), "rope.q_norm": rn(128, scale=0.1, shift=1.0),
        "rope.k_norm": rn(128, scale=0.1, shift=1.0), "rope.pos": torch.tensor([5, 0], dtype=torch.int32),
        # decode attention: one query row per sequence over 201 and 38 keys of a cache of 256
        "attn.q": rn(2, 8, 1, 128), "attn.k": rn(2, 2, 256, 128), "attn.v": rn(2, 2, 256, 128),
        "attn.pos": torch.tensor([200, 37], dtype=torch.int32),
        "model.ids": torch.randint(0, TINY["vocab_size"], (2, PROMPT_LEN), generator=g),
    }
    return ins


def main(reference: str) -> None:
    os.environ.setdefault("ENGINE_SELF_CHECK", "0")
    sys.path.insert(0, str(Path(reference) / "engine"))
    import model as ref_model
    from engine import GraphPlan
    from kernels import DecodeAttention, add_rms_norm, qk_norm_rope_cache, rms_norm, swiglu
    from starter_b200.config import config_from_dict
    from starter_b200.weights import write_model_folder
    from starter_b200.weights.safetensors_io import write_safetensors

    dev = "cuda:0"
    ins = {k: v.to(dev) for k, v in golden_inputs().items()}
    out = {}
    out["norm.out"] = rms_norm(ins["norm.x"], ins["norm.w"], EPS)
    x = ins["addnorm.x"].clone()
    out["addnorm.out"] = add_rms_norm(x, ins["addnorm.y"], ins["addnorm.w"], EPS)
    out["addnorm.x_after"] = x
    out["swiglu.out"] = swiglu(ins["swiglu.gu"])

    with tempfile.TemporaryDirectory() as folder:
        write_model_folder(config_from_dict(TINY), TINY_SEED, folder)
        m = ref_model.Model(folder)
        B, T, HQ, HKV, D, cap = 2, 3, 4, 2, 128, 64
        q_out = torch.zeros((B, HQ, T, D), dtype=torch.bfloat16, device=dev)
        k_cache = torch.zeros((B, HKV, cap, D), dtype=torch.bfloat16, device=dev)
        v_cache = torch.zeros_like(k_cache)
        qk_norm_rope_cache(ins["rope.qkv"], ins["rope.q_norm"], ins["rope.k_norm"], m.cos, m.sin, ins["rope.pos"], q_out,
                           k_cache, v_cache, T, EPS)
        out["rope.q"] = q_out
        out["rope.k_rows"] = torch.stack([k_cache[b, :, int(ins["rope.pos"][b]):int(ins["rope.pos"][b]) + T] for b in range(B)])
        out["rope.v_rows"] = torch.stack([v_cache[b, :, int(ins["rope.pos"][b]):int(ins["rope.pos"][b]) + T] for b in range(B)])
        untouched = k_cache.clone()
        for b in range(B):
            p = int(ins["rope.pos"][b])
            untouched[b, :, p:p + T] = 0
        assert not untouched.any(), "the reference wrote cache rows outside pos..pos+T"

        attn = DecodeAttention(2, 8, 2, 128, 256, dev)
        a_out = torch.zeros((2, 1, 8, 128), dtype=torch.bfloat16, device=dev)
        attn(ins["attn.q"], ins["attn.k"], ins["attn.v"], ins["attn.pos"], a_out)
        out["attn.out"] = a_out

        plan = GraphPlan(m, 2, PROMPT_LEN, DECODE_STEPS + 1).plan
        plan.ids.copy_(ins["model.ids"])
        logits = [plan.prefill().clone()]
        forced = []
        for _ in range(DECODE_STEPS):
            forced.append(logits[-1].float().argmax(-1))
            plan.tok.copy_(forced[-1])
            logits.append(plan.decode().clone())
        out["model.logits"] = torch.stack(logits, dim=1)          # [B, 1 + steps, V], bfloat16 as the reference returns them
        out["model.forced"] = torch.stack(forced, dim=1).to(torch.int32)
    torch.cuda.synchronize()
    out = {k: v.detach().cpu().contiguous() for k, v in out.items()}
    path = Path(__file__).resolve().parent / "reference_gpu.safetensors"
    write_safetensors(path, [(k, (v.dtype, tuple(v.shape))) for k, v in out.items()], out.__getitem__)
    print(f"wrote {path} ({path.stat().st_size} bytes): " + ", ".join(f"{k}{list(v.shape)}" for k, v in out.items()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden_gpu.py /path/to/reference   (the folder that holds engine/)")
    main(sys.argv[1])
