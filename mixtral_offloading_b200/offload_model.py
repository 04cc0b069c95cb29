"""Decoder with offloaded experts: what the reference's build_model returns (src/build_model.py:166-241), for decoding.

Each layer is this package's attention step (AttentionDecode) followed by the reference's MoE block
(SparseMoeWrapper, custom_layers.py:259-314) over one ExpertCache shared by all layers, every layer its own
eviction group (build_model.py:219-235).  The host is in the loop once per layer, as in the reference: it has to
read which experts the router picked before it can ask the cache for them.

speculate=True turns on speculative expert loading, which the reference's README.md:24-27 lists as upcoming: each
block guesses the next layer's experts by running the next layer's router on its own input, and the cache starts
loading the guessed ones that are offloaded while this layer's experts and the next layer's attention run.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
from torch import nn

from .custom_layers import SparseMoeWrapper
from .decoder import AttentionDecode, add_rmsnorm


class MixtralOffloadModel(nn.Module):
    """embed (vocab, hidden) bf16; attentions[l]: AttentionDecode; blocks[l]: SparseMoeWrapper of layer l (all over
    one ExpertCache); final_norm (hidden) bf16; lm_head (vocab, hidden) bf16."""

    def __init__(self, embed: torch.Tensor, attentions: Sequence[AttentionDecode], blocks: Sequence[SparseMoeWrapper],
                 final_norm: torch.Tensor, lm_head: torch.Tensor, rms_eps: float = 1e-5, speculate: bool = False):
        super().__init__()
        assert len(attentions) == len(blocks)
        self.embed, self.final_norm, self.lm_head, self.rms_eps = embed, final_norm, lm_head, rms_eps
        self.attentions, self.blocks = nn.ModuleList(attentions), nn.ModuleList(blocks)
        dev = embed.device
        self.token = torch.zeros((1,), dtype=torch.int64, device=dev)
        self.position = torch.zeros((1,), dtype=torch.int32, device=dev)
        self.router_logits: List[torch.Tensor] = []
        self.set_speculation(speculate)

    def set_speculation(self, on: bool, width: int = 2) -> None:
        """width: how many of the next layer's guessed experts per token are loaded ahead (2, or 1 = the likelier)."""
        assert width in (1, 2)
        for l, blk in enumerate(self.blocks):
            blk.speculate_next = self.blocks[l + 1] if on and l + 1 < len(self.blocks) else None
            blk.speculate_width = width

    @property
    def expert_cache(self):
        return self.blocks[0].experts

    @torch.inference_mode()
    def step(self) -> torch.Tensor:
        """Feeds self.token at self.position; afterwards self.token is the greedy next token and self.position has
        advanced.  Returns the logits (1, vocab)."""
        h = self.embed[self.token]                       # (1, hidden), a fresh tensor; the residual stream
        delta, logits_per_layer = None, []
        for attn, blk in zip(self.attentions, self.blocks):
            x = attn(h, self.position, delta)            # h += previous block's output; attention; x = norm(h) * ln_post
            y, router_logits = blk(x.view(1, 1, -1))
            delta = y.view(1, -1)
            logits_per_layer.append(router_logits)
        x = add_rmsnorm(h, delta, self.final_norm, self.rms_eps)
        logits = torch.matmul(x, self.lm_head.t())
        self.router_logits = logits_per_layer
        self.token.copy_(logits.argmax(-1))
        self.position.add_(1)
        return logits

    @torch.inference_mode()
    def generate(self, prompt_ids: Sequence[int], new_tokens: int, force=None) -> List[int]:
        """Greedy decoding: the prompt is fed one token at a time, then new_tokens tokens are produced.
        force: optional list of token ids fed instead of the model's own choices (teacher forcing)."""
        self.position.zero_()
        out: List[int] = []
        for t in prompt_ids[:-1]:
            self.token.fill_(int(t))
            self.step()
        self.token.fill_(int(prompt_ids[-1]))
        for i in range(new_tokens):
            self.step()
            out.append(int(self.token.item()))
            if force is not None:
                self.token.fill_(int(force[i]))
        return out
