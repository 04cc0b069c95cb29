"""Token sampling as the reference's demo asks Hugging Face's generate() for it (notebooks/demo.ipynb, the chat cell:
do_sample=True, temperature=0.9, top_p=0.9): temperature scaling, then nucleus (top-p) filtering, then one draw
from the softmax of what is left.  Restated from transformers' TemperatureLogitsWarper and TopPLogitsWarper
(generation/logits_process.py); tests/test_sampling.py checks the filter against those classes."""
from __future__ import annotations

import torch


def top_p_filter(logits: torch.Tensor, top_p: float, min_tokens_to_keep: int = 1) -> torch.Tensor:
    """logits (..., vocab) float.  Tokens outside the smallest set whose probabilities sum to at least top_p get
    -inf (the least probable tokens whose cumulative probability stays <= 1 - top_p are removed; the
    min_tokens_to_keep most probable ones always stay)."""
    if not 0.0 < top_p <= 1.0:
        raise ValueError(f"top_p has to be in (0, 1], not {top_p}")
    if top_p == 1.0:
        return logits
    sorted_logits, sorted_idx = torch.sort(logits, descending=False, dim=-1)
    cumulative = sorted_logits.softmax(dim=-1).cumsum(dim=-1)
    remove = cumulative <= (1.0 - top_p)
    remove[..., -min_tokens_to_keep:] = False
    remove = remove.scatter(-1, sorted_idx, remove)
    return logits.masked_fill(remove, float("-inf"))


def sample_token(logits: torch.Tensor, temperature: float = 1.0, top_p: float = 1.0, generator=None) -> torch.Tensor:
    """One token id per row of logits (rows, vocab): int64 (rows,)."""
    if temperature <= 0.0:
        raise ValueError(f"temperature has to be positive, not {temperature}")
    scores = logits.float() / temperature
    scores = top_p_filter(scores, top_p)
    return torch.multinomial(scores.softmax(dim=-1), 1, generator=generator).squeeze(-1)
