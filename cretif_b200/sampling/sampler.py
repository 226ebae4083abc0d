"""Choosing the next token from a row of logits, on the device.

Options follow the reference's ``generate(prompt, max_tokens, temperature, top_k)``
(include/cuinfer/model.h:116-119):

* ``temperature <= 0``: greedy arg-max, ties to the lowest id (src/embedding.cu:155-204);
* ``temperature > 0`` and ``top_k > 0``: the ``top_k`` largest logits divided by the
  temperature, softmax, one draw (src/embedding.cu:343-406; ``top_k`` above the
  vocabulary size means the whole vocabulary, :345);
* ``temperature > 0`` and ``top_k == 0``: temperature sampling over the whole
  vocabulary.  (The reference falls back to greedy whenever ``top_k <= 0``,
  src/model.cu:1071; here a temperature alone is honoured.)

``seed`` keys a counter-based generator: draw number ``n`` of request ``r`` uses
``uniform01(seed, r, n)``, whatever else is in the batch.  The reference's default
seed is 42 (include/cuinfer/embedding.h:108-110).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..csrc import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    seed: int = 42

    def validate(self, vocab_size: int) -> None:
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not (self.temperature == self.temperature):
            raise ValueError("temperature is NaN")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


def uniform01(seed: int, request: int, draw: int) -> float:
    """The uniform number in (0, 1) used for draw ``draw`` of request ``request``."""
    return ops.uniform01(seed, request, draw)


class Sampler:
    """Runs the sampling kernel: one token id per row of float32 logits.

    The seed lives in device memory and the kernel reads it from there, so a captured
    launch serves any seed: :meth:`set_seed` takes effect at the next launch or replay."""

    def __init__(self, params: SamplingParams, vocab_size: int):
        params.validate(vocab_size)
        self.params = params
        self._seed = int(params.seed)
        self._seed_dev: Optional[torch.Tensor] = None

    def set_seed(self, seed: int) -> None:
        self._seed = int(seed)
        if self._seed_dev is not None:
            self._seed_dev.fill_(_as_int64(self._seed))

    def __call__(self, logits: torch.Tensor, out: torch.Tensor,
                 request: Optional[torch.Tensor] = None,
                 draw: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``request`` [rows] int64 and ``draw`` [rows] int32 (incremented by the kernel)
        key the random numbers; both may be None for greedy sampling."""
        p = self.params
        if self._seed_dev is None or self._seed_dev.device != logits.device:
            self._seed_dev = torch.full((1,), _as_int64(self._seed), dtype=torch.int64,
                                        device=logits.device)
        ops.sample(logits, out, p.temperature, p.top_k, self._seed, request, draw,
                   seed_dev=self._seed_dev)
        return out


def _as_int64(seed: int) -> int:
    """The 64 bits of ``seed`` as a signed value (what an int64 tensor holds)."""
    seed &= 0xFFFFFFFFFFFFFFFF
    return seed - (1 << 64) if seed >= (1 << 63) else seed
