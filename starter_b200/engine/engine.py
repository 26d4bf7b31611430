"""The Python entry point, in the reference's manner.

The reference's interface (README.md:54-66, engine/engine.py:430,582):

    engine = Engine(model_path)
    for step in engine.generate(input_ids, max_new_tokens): ...   # one token id per sequence per step

Kept here with the same names and meanings; additions are keyword arguments
with defaults that reproduce the reference's behaviour (greedy, no stop
tokens, exactly ``max_new_tokens`` steps).  Prompts of unequal length are
accepted (the reference raises ValueError for them, engine/engine.py:584-585).
``ENGINE_NO_GRAPHS`` in the environment turns CUDA graphs off, as it does
there (engine/engine.py:436).
"""

from __future__ import annotations

import os
from typing import Iterable, Iterator, List, Optional, Sequence

from ..sampling.sampler import SamplingParams
from .generate import Generator
from .session import Session


class Engine:
    def __init__(self, model_path, dtype: str = "bfloat16", max_batch: int = 64, max_context: int = 4096,
                 max_tokens: Optional[int] = None, device: str = "cuda:0", use_graphs: Optional[bool] = None,
                 ops=None, verbose: bool = False):
        """Load the model folder (config.json, model.safetensors) and set up the cache.

        ``max_batch`` sequences of up to ``max_context`` tokens each may be live at once;
        ``max_tokens`` bounds the tokens they hold together (default: all of them at full length).
        """
        if use_graphs is None:
            use_graphs = os.environ.get("ENGINE_NO_GRAPHS") is None
        self.model_path = model_path
        self.session = Session(model_path, dtype=dtype, max_tokens=max_tokens or max_batch * max_context,
                               max_seqs=max_batch, max_seq_tokens=max_context, device=device, ops=ops, verbose=verbose)
        self.generator = Generator(self.session, use_graphs=use_graphs)

    @classmethod
    def from_session(cls, session: Session, use_graphs: Optional[bool] = None) -> "Engine":
        """The entry point around a model that is loaded already (a Session made from a folder or from
        a configuration and a weight source)."""
        if use_graphs is None:
            use_graphs = os.environ.get("ENGINE_NO_GRAPHS") is None
        engine = cls.__new__(cls)
        engine.model_path = None
        engine.session = session
        engine.generator = Generator(session, use_graphs=use_graphs)
        return engine

    @property
    def config(self):
        return self.session.config

    def generate(self, input_ids: Sequence[Sequence[int]], max_new_tokens: int, temperature: float = 0.0,
                 top_k: int = 0, seed: int = 0, stop_token_ids: Iterable[int] = ()) -> Iterator[List[Optional[int]]]:
        """Continue every sequence, one step at a time: yields a list with one token id per sequence
        for each output step.  Without stop tokens that is exactly ``max_new_tokens`` lists of ints;
        with them, a sequence that has ended shows None, and the loop ends when all have ended."""
        sampling = SamplingParams(temperature=float(temperature), top_k=int(top_k), seed=int(seed))
        yield from self.generator.generate_batch(input_ids, max_new_tokens, sampling, stop_token_ids)

    def generate_all(self, input_ids: Sequence[Sequence[int]], max_new_tokens: int, temperature: float = 0.0,
                     top_k: int = 0, seed: int = 0, stop_token_ids: Iterable[int] = ()) -> List[List[int]]:
        """The new tokens of every request; more requests than fit at once run as batches one after another."""
        sampling = SamplingParams(temperature=float(temperature), top_k=int(top_k), seed=int(seed))
        return self.generator.run(input_ids, max_new_tokens, sampling, stop_token_ids)
