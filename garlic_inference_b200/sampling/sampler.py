"""Choosing the next token: greedy, or a draw at a temperature.

Upstream takes the argmax of the logits and nothing else
(inference.cpp:145, src/src-cuda/reductions/argmax.cu:72-101).  Here
temperature 0 is that argmax with ties to the lowest id, and a positive
temperature draws from softmax(logits / temperature).  The draw for a given
(seed, request, token index) is the same whatever else is in the batch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from ..ops import kernels


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0      # 0 = greedy
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must not be negative, found {self.temperature}")


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: SamplingParams, request_ids: Sequence[int],
               token_indices: Sequence[int]) -> torch.Tensor:
        """int32 tokens [rows] on the device for float32 logits [rows, vocab].  `request_ids[r]` and
        `token_indices[r]` key row r's random stream: the request's number and how many tokens it
        has generated so far."""
        n = logits.shape[0]
        if params.temperature <= 0:
            return kernels.sample(logits, None, None, None, 0)
        pin = self.device.type == "cuda"               # pinned, so that the copies do not wait for the GPU
        streams = torch.tensor(list(request_ids), dtype=torch.int64, pin_memory=pin).to(self.device, non_blocking=True)
        counters = torch.tensor(list(token_indices), dtype=torch.int32, pin_memory=pin).to(self.device, non_blocking=True)
        temps = torch.full((n,), float(params.temperature), dtype=torch.float32, device=self.device)
        return kernels.sample(logits, temps, streams, counters, params.seed)
