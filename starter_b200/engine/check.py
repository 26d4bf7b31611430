"""The 32-bit check path: the same weights through the bfloat16 engine and through the float32 engine.

The reference checks itself against another implementation once at start-up:
teacher-forced tokens through prefill and decode, largest logit difference
and the gap at the chosen token (engine/engine.py:474-516).  Here the other
implementation is this library's own true 32-bit path (CUDA-core products, no
reduced-precision matrix mode, 32-bit cache and tables): the same prompts and
the same forced tokens go through both, cut the same way, and the report says
how far the bfloat16 logits are from the 32-bit ones and how often the two
choose the same token.  Kernels are picked by the shape rules as in any run,
so a wrong rule at a model's real sizes shows here.
"""

from __future__ import annotations

from typing import Dict, Sequence

import torch

from ..weights.random_weights import RandomSource
from .session import Session
from .step import StepEntry

# Largest |difference| of a bfloat16 logit from its 32-bit value, as a fraction of the largest |logit|.
# bfloat16 carries 8 bits: every rounded intermediate moves by up to 2^-9 relative, and a logit is a
# sum of many such values.
BF16_TOLERANCE = 3e-2


def _forced_run(session: Session, prompts, forced: torch.Tensor, decode_steps: int, choose: bool = False):
    """Prefill every prompt alone and whole (logits at its last token), then run all of them as one
    batch that decodes the tokens ``forced`` [n_prompts, decode_steps]; with ``choose`` the run fills
    ``forced`` with its own greedy choices as it goes.  Returns logits [n_prompts, 1 + decode_steps,
    vocab] on the host."""
    cache, stepper = session.cache, session.stepper
    slots = [cache.alloc() for _ in prompts]
    try:
        first = [stepper.step([StepEntry(s, p, [len(p) - 1])]) for s, p in zip(slots, prompts)]
        rows = [torch.cat(first).float().cpu()]
        for t in range(decode_steps):
            if choose:
                forced[:, t] = rows[-1].argmax(-1)
            out = stepper.step([StepEntry(s, [int(forced[b, t])], [0]) for b, s in enumerate(slots)])
            rows.append(out.float().cpu())
        stepper.raise_on_status()
        return torch.stack(rows, dim=1)
    finally:
        for s in slots:
            cache.free(s)


def compare_dtypes(config, seed: int = 0, prompt_lengths: Sequence[int] = (300, 2048),
                   decode_batches: Sequence[int] = (1, 8, 64), decode_steps: int = 6, device="cuda:0",
                   ops=None, verbose: bool = False) -> Dict[str, object]:
    """Run ``config`` with seeded random weights in bfloat16 and in float32 and compare the logits.

    For each batch size of ``decode_batches``: that many prompts (lengths cycling through
    ``prompt_lengths``, the first ending one token before a page boundary so that decoding crosses
    it) are prefilled, then ``decode_steps`` tokens chosen by the 32-bit run are fed to both.
    """
    vocab = config.model_spec().vocab_size
    gen = torch.Generator().manual_seed(seed + 1)
    longest = max(prompt_lengths) + decode_steps + 64
    sessions = {}
    for dtype in ("float32", "bfloat16"):
        source = RandomSource(config, seed, dtype=torch.bfloat16, device=device)   # bfloat16 values, widened for the 32-bit run
        sessions[dtype] = Session((config, source), dtype=dtype, max_tokens=max(decode_batches) * longest,
                                  max_seqs=max(decode_batches), max_seq_tokens=longest, device=device, ops=ops,
                                  verbose=verbose)
    worst, scale, same, total, cases = 0.0, 0.0, 0, 0, []
    for batch in decode_batches:
        lengths = [prompt_lengths[b % len(prompt_lengths)] for b in range(batch)]
        lengths[0] = max(1, ((lengths[0] + 63) // 64) * 64 - 1)
        prompts = [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in lengths]
        # the tokens to feed are the 32-bit run's own choices: decide them step by step in that run
        forced = torch.zeros((batch, decode_steps), dtype=torch.long)
        ref = _forced_run(sessions["float32"], prompts, forced, decode_steps, choose=True)
        got = _forced_run(sessions["bfloat16"], prompts, forced, decode_steps)
        diff = float((got - ref).abs().max())
        top = float(ref.abs().max())
        agree = int((got.argmax(-1) == ref.argmax(-1)).sum())
        cases.append({"batch": batch, "max_abs_diff": round(diff, 5), "scale": round(top, 4),
                      "rel": round(diff / top, 5), "argmax_same": agree, "of": got.shape[0] * got.shape[1]})
        worst, scale = max(worst, diff), max(scale, top)
        same += agree
        total += got.shape[0] * got.shape[1]
    rel = worst / scale if scale else 0.0
    return {"max_abs_diff": round(worst, 5), "scale": round(scale, 4), "max_rel_diff": round(rel, 5),
            "argmax_agreement": round(same / max(total, 1), 4), "positions": total, "tolerance": BF16_TOLERANCE,
            "within_tolerance": bool(rel <= BF16_TOLERANCE), "cases": cases}
