"""Token sampling: greedy on the device (``argmax_f32``), everything else on the host from the step's f32 logits, like the reference's
``LogitsProcessor`` (src/openai/sampling_params.rs, src/openai/logits_processor.rs: temperature, top-k, top-p, seeded)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from .backend import argmax


@dataclass
class SamplingParams:
    temperature: float = 0.0            # 0 = greedy
    top_k: int = 0                      # 0 = off
    top_p: float = 1.0
    max_tokens: int = 16
    seed: Optional[int] = None
    stop_token_ids: Sequence[int] = field(default_factory=tuple)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1


def sample_host(logits: np.ndarray, p: SamplingParams, rng: np.random.Generator) -> int:
    """One row of f32 logits -> token id (temperature, then top-k, then top-p over the sorted tail)."""
    z = logits.astype(np.float64) / max(p.temperature, 1e-6)
    order = np.argsort(-z, kind="stable")
    if p.top_k and p.top_k < len(order):
        order = order[:p.top_k]
    zs = z[order] - z[order[0]]
    pr = np.exp(zs)
    pr /= pr.sum()
    if p.top_p < 1.0:
        keep = int(np.searchsorted(np.cumsum(pr), p.top_p, side="left")) + 1
        order, pr = order[:keep], pr[:keep] / pr[:keep].sum()
    return int(order[rng.choice(len(order), p=pr)])


class Sampler:
    def __init__(self):
        self._rngs = {}

    def rng(self, key, seed: Optional[int]) -> np.random.Generator:
        if key not in self._rngs:
            self._rngs[key] = np.random.default_rng(seed)
        return self._rngs[key]

    def forget(self, key) -> None:
        self._rngs.pop(key, None)

    def sample(self, logits: torch.Tensor, params: List[SamplingParams], keys: List) -> List[int]:
        """logits f32 [R, vocab] on the device, one SamplingParams per row"""
        out = [0] * len(params)
        if all(p.greedy for p in params):
            return [int(t) for t in argmax(logits).cpu().tolist()]
        host = logits.float().cpu().numpy()
        greedy = argmax(logits).cpu().tolist() if any(p.greedy for p in params) else None
        for i, (p, k) in enumerate(zip(params, keys)):
            out[i] = int(greedy[i]) if p.greedy else sample_host(host[i], p, self.rng(k, p.seed))
        return out
