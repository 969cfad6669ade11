"""Token selection for the rows of one step.

Same knobs and meanings as the reference's ``GenerationParams`` and ``StochasticSampler``
(pulsar-core/inc/pulsar/runtime/sampler.hpp:21-40; pulsar-core/src/runtime/sampler.cpp:12-57):
temperature <= 0 is exact greedy on the raw logits and leaves the generator untouched;
otherwise softmax(logits / temperature), top_k > 0 keeps the k most probable, top_p in
(0, 1) keeps a token while the mass before it is <= top_p, both give the intersection;
seed >= 0 makes a request reproducible, seed < 0 draws a fresh seed.

The reference samples one row at a time with a device-to-host read each.  Here a few
kernels handle all rows of the step (many blocks per row) and the chosen ids stay on the
device for the next step or come back in one copy; the uniform number of each stochastic
row comes from that request's own host generator, so a request's tokens do not depend on
what else is in the batch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops


@dataclass
class GenerationParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int = -1

    def validate(self) -> None:
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must lie in (0, 1], found {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, found {self.top_k}")

    @property
    def greedy(self) -> bool:
        return not (self.temperature > 0.0)


def make_generator(seed: int) -> torch.Generator:
    """Per-request generator: seed >= 0 reproducible, seed < 0 nondeterministic
    (pulsar-core/src/runtime/sampler.cpp:48-57)."""
    g = torch.Generator(device="cpu")
    if seed >= 0:
        g.manual_seed(int(seed))
    else:
        g.seed()
    return g


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._ids: Optional[torch.Tensor] = None
        self.last_ids: Optional[torch.Tensor] = None      # what the last call returned

    def sample_on_device(self, logits: torch.Tensor, params: Sequence[GenerationParams],
                         generators: Sequence[Optional[torch.Generator]]) -> torch.Tensor:
        """One token id per row of ``logits`` (float32 [R, V] on the device), left on the device:
        an int32 tensor that stays valid until the next call."""
        rows = logits.shape[0]
        assert len(params) == rows and len(generators) == rows
        if self._ids is None or self._ids.numel() < rows:
            self._ids = torch.empty(max(rows, 64), dtype=torch.int32, device=self.device)
        out = self._ids[:rows]
        self.last_ids = out
        if rows == 0:
            return out
        if all(p.greedy for p in params):
            ops.sample(logits, out)
        else:
            uniform = [0.0 if p.greedy else float(torch.rand(1, generator=g).item()) for p, g in zip(params, generators)]
            packed = torch.tensor([[p.temperature for p in params], [p.top_p for p in params], uniform],
                                  dtype=torch.float32).to(self.device, non_blocking=True)
            top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32).to(self.device, non_blocking=True)
            ops.sample(logits, out, packed[0], top_k, packed[1], packed[2], any_greedy=any(p.greedy for p in params))
        return out

    def sample(self, logits: torch.Tensor, params: Sequence[GenerationParams],
               generators: Sequence[Optional[torch.Generator]]) -> List[int]:
        """One token id per row of ``logits``, read back to the host."""
        if logits.shape[0] == 0:
            return []
        return self.sample_on_device(logits, params, generators).tolist()
