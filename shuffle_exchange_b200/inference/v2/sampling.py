"""Next-token selection from logits: greedy, temperature, top-k and nucleus (top-p) sampling."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class SamplingParams:
    temperature: float = 0.0          # 0: greedy
    top_k: int = 0                    # 0: no limit
    top_p: float = 1.0
    seed: Optional[int] = None


def sample(logits: torch.Tensor, params: SamplingParams = None, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """``logits`` ``[n, vocab]`` -> int64 ``[n]``.  Greedy ties go to the lowest token id."""
    params = params or SamplingParams()
    logits = logits.float()
    if params.temperature <= 0.0:
        return logits.argmax(dim=-1)
    logits = logits / params.temperature
    if params.top_k > 0:
        kth = logits.topk(min(params.top_k, logits.shape[-1]), dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    probs = torch.softmax(logits, dim=-1)
    if params.top_p < 1.0:
        sp, si = probs.sort(dim=-1, descending=True)
        drop = sp.cumsum(-1) - sp > params.top_p          # keep the smallest prefix whose mass reaches top_p
        sp = sp.masked_fill(drop, 0.0)
        probs = torch.zeros_like(probs).scatter(-1, si, sp)
        probs = probs / probs.sum(-1, keepdim=True)
    return torch.multinomial(probs, 1, generator=generator).squeeze(-1)
