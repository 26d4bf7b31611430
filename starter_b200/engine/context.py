"""What a forward pass hands to every part: the run's kernels and the step's batch.

The reference passes ``pos[B]`` and fixed shapes (B, T) to its kernels
(engine/kernels/rope.py:43, engine/kernels/attention.py:41); here a step is a
ragged batch, described once on the device and read by every kernel:

* ``seq_slot[B]``: the cache slot of each sequence of the step;
* ``cu_q[B+1]``: first row of each sequence among the step's rows;
* ``row_seq[M]``: the sequence of each row;
* ``lengths[slot]``: tokens the sequence held before this step, so that row r of
  sequence b stands at position ``lengths[seq_slot[b]] + r - cu_q[b]``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Sequence

import torch


@dataclass
class Runtime:
    """Dtype, device and kernels of a run.  ``ops`` is the loaded CUDA extension's call table."""

    dtype: torch.dtype
    device: torch.device
    ops: Any

    @property
    def is_bf16(self) -> bool:
        return self.dtype == torch.bfloat16


@dataclass
class StepContext:
    runtime: Runtime
    cache: Any
    n_seqs: int
    n_rows: int
    max_q_len: int          # host-side bound on a sequence's rows in this step
    kv_bound: int           # host-side bound on any sequence's length after this step
    seq_slot: torch.Tensor  # int32 [n_seqs]
    cu_q: torch.Tensor      # int32 [n_seqs + 1]
    row_seq: torch.Tensor   # int32 [n_rows]
    lengths: torch.Tensor   # int32 [n_slots + 1], the cache's
    status: torch.Tensor    # int32 [1], kernels raise bits here instead of faulting
    scratch: Dict[str, Any] = field(default_factory=dict)
    uneven: bool = False    # host-side hint: the longest sequence is several times the mean (see lengths_uneven)

    @property
    def ops(self):
        return self.runtime.ops

    @property
    def is_decode(self) -> bool:
        return self.max_q_len == 1


def lengths_uneven(lengths: Sequence[int], page: int = 64) -> bool:
    """Whether a batch's sequences are of very unequal length: the longest holds more than three times the mean
    number of cache pages.  Kernels that hand each sequence's keys to a block of its own then wait for the longest
    one, and one that shares all pages out evenly is the better choice (the call table decides)."""
    if len(lengths) < 2:
        return False
    pages = [int(n) // page + 1 for n in lengths]
    return max(pages) * len(pages) > 3 * sum(pages)


class ResidualStream:
    """The residual x [rows, hidden] and a branch output not yet added to it.

    The sum x + pending is taken in 32-bit inside the kernel that also norms it
    (the reference's add_rms_norm, engine/kernels/add_rmsnorm.py:16-29), so a
    branch's output meets the residual in the same pass that feeds the next branch.
    A branch whose last product can add to x itself is given the stream as the
    place to add to (``ops.linear(..., add_to=stream)``) and pushes nothing.
    """

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending = None
        self.stats = None   # left by a product that added its result to x itself: what a norm folded into the next product reads

    def normed(self, norm) -> torch.Tensor:
        if self.pending is None:
            return norm.forward(self.x)
        delta, self.pending = self.pending, None
        self.stats = None   # x changes here
        return norm.add_forward(self.x, delta)

    def push(self, branch_output: torch.Tensor) -> None:
        if self.pending is not None:
            raise RuntimeError("a branch output is already waiting to be added to the residual")
        self.pending = branch_output
