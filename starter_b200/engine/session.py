"""A loaded model with its cache and step function: what replay, generation and benchmarks share."""

from __future__ import annotations

import os
from typing import Optional

import torch

from ..cache.cache import PAGE, Cache
from ..config.registry import ModelConfig
from .context import Runtime
from .model import DecoderModel
from .step import Stepper

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "fp32": torch.float32, "bf16": torch.bfloat16}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the run's dtype is float32 or bfloat16, not {name}")
        return name
    try:
        return DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"the run's dtype is float32 or bfloat16, not {name!r}") from None


class Session:
    """Model, cache and stepper on one device.

    ``model``: a folder with config.json and model.safetensors, or a pair
    (config, weight source).  ``max_tokens``: the tokens all live sequences may
    hold together, each rounded up to the page size; ``max_seqs``: how many
    sequences may be live at once; ``max_seq_tokens``: the longest sequence.
    ``ops``: the kernel call table; by default the CUDA extension, which must load.
    ``dependent_launch``: let each kernel start its preamble while its predecessor finishes
    (programmatic dependent launch).  On by default: measured on the 4B shapes it shortens the decode
    step by 4%; STARTER_B200_PDL=0 in the environment turns it off.
    """

    def __init__(self, model, dtype="bfloat16", max_tokens: int = 8192, max_seqs: Optional[int] = None,
                 max_seq_tokens: Optional[int] = None, max_step_tokens: int = 1024, max_rows: int = 8192,
                 device="cuda:0", ops=None, verbose: bool = True, dependent_launch=None):
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        if ops is None:
            from ..csrc.ops import get_ops
            if self.device.type != "cuda":
                raise ValueError("the kernels of this library run on a CUDA device only")
            ops = get_ops(verbose=verbose)   # first: without a CUDA device this raises the library's own error
            torch.cuda.set_device(self.device)
        if dependent_launch is None:
            dependent_launch = os.environ.get("STARTER_B200_PDL", "1") != "0"
        if hasattr(ops, "set_dependent_launch"):
            ops.set_dependent_launch(dependent_launch)
        self.runtime = Runtime(dtype=self.dtype, device=self.device, ops=ops)
        if isinstance(model, tuple):
            config, source = model
            if not isinstance(config, ModelConfig):
                raise TypeError("a model is a folder or a pair (configuration, weight source)")
            self.model = DecoderModel.from_source(config, source, self.runtime)
        else:
            self.model = DecoderModel.from_folder(model, self.runtime)
        self.config = self.model.config
        pages = (int(max_tokens) + PAGE - 1) // PAGE
        n_slots = int(max_seqs) if max_seqs else pages
        self.cache = Cache(self.model.cache_requests(), n_slots=n_slots, max_tokens=pages * PAGE, dtype=self.dtype,
                           device=self.device, max_seq_tokens=max_seq_tokens, max_step_tokens=max_step_tokens)
        self.stepper = Stepper(self.model, self.cache, max_rows=max_rows)

    @property
    def vocab_size(self) -> int:
        return self.model.spec.vocab_size
