"""Greedy single-sequence decoding on top of DecoderLayerDecode: embedding lookup, the decoder layers (one
library call each), lm_head and argmax, with the step optionally replayed from a CUDA graph.

The reference generates through Hugging Face's `generate` on the model that src/build_model.py:166-241
assembles (notebooks/demo.ipynb).  Here a token is one fixed sequence of launches: the position lives in
device memory, the experts are picked on the device, nothing returns to the host inside a step.  The prompt is
either fed through the same single-token step or processed in one pass (prefill(): the quantized linears on
their many-row path, torch's attention over the prompt).
"""
from __future__ import annotations

from typing import List, Sequence

import torch
from torch import nn

from .decoder import DecoderLayerDecode, add_rmsnorm, rms_norm_rows, rope_append_rows
from .sampling import sample_token


class MixtralDecodeModel(nn.Module):
    """embed: (vocab, hidden) bf16; layers: DecoderLayerDecode, each built with next_ln = the following layer's
    input norm weight (the last one with the final norm weight); first_ln: layer 0's input norm weight;
    lm_head: (vocab, hidden) bf16."""

    def __init__(self, embed: torch.Tensor, layers: Sequence[DecoderLayerDecode], first_ln: torch.Tensor,
                 lm_head: torch.Tensor, rms_eps: float = 1e-5):
        super().__init__()
        self.embed, self.first_ln, self.lm_head, self.rms_eps = embed, first_ln, lm_head, rms_eps
        self.layers = nn.ModuleList(layers)
        dev = embed.device
        self.token = torch.zeros((1,), dtype=torch.int64, device=dev)     # the token being fed
        self.position = torch.zeros((1,), dtype=torch.int32, device=dev)   # its position
        self.router_logits: List[torch.Tensor] = []
        self._graph = None
        self._logits = None

    @property
    def max_len(self) -> int:
        return min(l.attention.max_len for l in self.layers)

    @torch.inference_mode()
    def step(self) -> torch.Tensor:
        """Feeds self.token at self.position through the model; afterwards self.token is the greedy next token
        and self.position has advanced.  Returns the logits (1, vocab)."""
        h = self.embed[self.token]                                         # (1, hidden), a fresh tensor
        x = add_rmsnorm(h, None, self.first_ln, self.rms_eps)
        self.router_logits = [layer(h, x, self.position) for layer in self.layers]
        logits = torch.matmul(x, self.lm_head.t())     # x is the final norm of h after the last layer
        self.token.copy_(logits.argmax(-1))
        self.position.add_(1)
        return logits

    @torch.inference_mode()
    def capture(self, warmup: int = 2) -> None:
        """Records step() into a CUDA graph; replay() then runs a whole token with one launch from the host."""
        tok, pos = self.token.clone(), self.position.clone()
        side = torch.cuda.Stream(self.embed.device)
        side.wait_stream(torch.cuda.current_stream(self.embed.device))
        with torch.cuda.stream(side):
            for _ in range(warmup):                                        # settle allocations and scratch sizes
                self.step()
        torch.cuda.current_stream(self.embed.device).wait_stream(side)
        self.token.copy_(tok)
        self.position.copy_(pos)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._logits = self.step()
        self.token.copy_(tok)                                              # capture does not execute, but keep it explicit
        self.position.copy_(pos)

    def replay(self) -> torch.Tensor:
        if self._graph is None:
            raise RuntimeError("capture() has not been called")
        self._graph.replay()
        return self._logits

    # ---- several tokens at once ---------------------------------------------------------------------------
    @torch.inference_mode()
    def extend(self, token_ids: Sequence[int]) -> torch.Tensor:
        """Feeds T tokens in one pass behind whatever the caches already hold (positions self.position ..
        self.position + T - 1): the quantized linears take the many-row tensor-core path, attention over the cache is
        torch's scaled_dot_product_attention, the MoE block groups the tokens per expert
        (DecoderLayerDecode.forward_tokens).  Leaves self.position advanced by T and self.token = the greedy next
        token.  Returns the logits of the last fed position (1, vocab)."""
        T = len(token_ids)
        pos0 = int(self.position.item())
        if T == 0 or pos0 + T >= self.max_len:
            raise ValueError(f"{T} tokens at position {pos0} do not fit a cache of {self.max_len}")
        ids = torch.tensor(list(token_ids), dtype=torch.int64, device=self.embed.device)
        h = self.embed[ids]                                                # (T, hidden)
        self.router_logits = []
        ln_in = self.first_ln                       # the norm weights step() applies: first_ln, then each layer's next_ln
        shared = self.layers[0].tokens_shared(T, pos0, h.device)
        for layer in self.layers:
            h, logits = layer.forward_tokens(h, pos0, ln_in, shared)
            self.router_logits.append(logits)
            ln_in = layer.next_ln
        x = rms_norm_rows(h[-1:], self.layers[-1].next_ln, self.rms_eps)
        logits = torch.matmul(x, self.lm_head.t())
        self.token.copy_(logits.argmax(-1))
        self.position.fill_(pos0 + T)
        return logits

    @torch.inference_mode()
    def prefill(self, prompt_ids: Sequence[int]) -> torch.Tensor:
        """The whole prompt in one pass on empty caches: extend() from position 0."""
        self.position.zero_()
        return self.extend(prompt_ids)

    @torch.inference_mode()
    def generate(self, prompt_ids: Sequence[int], new_tokens: int, use_graph: bool = True, prefill: bool = False,
                 do_sample: bool = False, temperature: float = 1.0, top_p: float = 1.0, generator=None,
                 eos_token_id=None, continue_cache: bool = False) -> List[int]:
        """Continuation of prompt_ids: greedy, or (do_sample) drawn with the demo's settings (notebooks/demo.ipynb:
        temperature and nucleus sampling, sampling.sample_token).  The prompt is fed token by token through the decode
        step, or, with prefill=True, in one pass through extend().  continue_cache=True keeps what the caches hold
        and appends behind it (the demo's multi-turn loop passes past_key_values back in); otherwise the caches
        start empty.  Stops early after eos_token_id.  Returns the new tokens."""
        start = int(self.position.item()) if continue_cache else 0
        if len(prompt_ids) == 0 or start + len(prompt_ids) + new_tokens > self.max_len:
            raise ValueError(f"{start} cached + {len(prompt_ids)} prompt + {new_tokens} new tokens do not fit a cache of "
                             f"{self.max_len}")
        if use_graph and self._graph is None:
            self.capture()
        run = self.replay if use_graph else self.step

        def choose(logits):              # step() leaves the greedy token in self.token; sampling overwrites it
            if do_sample:
                self.token.copy_(sample_token(logits, temperature, top_p, generator))
            return int(self.token.item())
        self.position.fill_(start)
        if prefill:
            logits = self.extend(prompt_ids)
        else:
            for t in prompt_ids:
                self.token.fill_(int(t))
                logits = run()
        out: List[int] = [choose(logits)]
        while len(out) < new_tokens and out[-1] != eos_token_id:
            out.append(choose(run()))
        return out


class BatchDecode:
    """B independent sequences advanced one token per step through the layers of a MixtralDecodeModel (the same
    weights), each sequence with its own key/value cache; all of them at the same position.

    The quantized projections and the experts run once per step on all B rows (the few-row streaming kernels read
    the weights once for the batch); norms, RoPE and attention over the caches are torch ops; the MoE block groups the
    rows per expert as SparseMoeWrapper.forward does (custom_layers.py:272-314), which needs the row counts on the
    host once per layer.  A step is therefore a chain of segments, one per layer: [add the previous block's output,
    attention half, post-attention norm, router] - read the counts back - [the active experts].  capture() records
    every segment in a CUDA graph (the position is device data: hqm_rope_append_rows reads it, and attention runs
    over the whole cache under a mask), so that the host issues one replay and the experts per layer."""

    def __init__(self, model: MixtralDecodeModel, batch: int, max_len: int):
        self.model, self.batch, self.max_len = model, batch, max_len
        a0 = model.layers[0].attention
        dev = model.embed.device
        hidden = model.embed.shape[1]
        shape = (batch, a0.n_kv_heads, max_len, a0.head_dim)
        self.k_caches = [torch.zeros(shape, dtype=torch.bfloat16, device=dev) for _ in model.layers]
        self.v_caches = [torch.zeros(shape, dtype=torch.bfloat16, device=dev) for _ in model.layers]
        self.tokens = torch.zeros((batch,), dtype=torch.int64, device=dev)
        self.position = torch.zeros((1,), dtype=torch.int64, device=dev)
        self.h = torch.zeros((batch, hidden), dtype=torch.bfloat16, device=dev)     # residual streams
        self.y = torch.zeros((batch, hidden), dtype=torch.bfloat16, device=dev)     # the last MoE block's output
        self._slots = torch.arange(max_len, device=dev)
        E = model.layers[0].moe.num_experts
        self._host_counts = torch.empty((2 * E + 1,), dtype=torch.int32).pin_memory()
        self.router_logits: List[torch.Tensor] = []
        self._graphs = None
        self._routes = [None] * len(model.layers)
        self._x_moe = [None] * len(model.layers)
        self._mask = None
        self._logits = None

    # ---- segments ---------------------------------------------------------------------------------------------
    def _prologue(self):
        """The streams of the fed tokens and the mask of filled cache rows."""
        self._mask = (self._slots <= self.position)[None, None, None, :]
        self.h.copy_(self.model.embed[self.tokens])
        self.y.zero_()

    def _attention_segment(self, l: int):
        layer = self.model.layers[l]
        a, B, h = layer.attention, self.batch, self.h
        hidden = h.shape[-1]
        mask = self._mask
        h.add_(self.y)
        self.y.zero_()
        ln_in = self.model.first_ln if l == 0 else self.model.layers[l - 1].next_ln     # the weights step() applies
        x = rms_norm_rows(h, ln_in, a.rms_eps)
        q = a.q_proj(x)
        rope_append_rows(q, a.k_proj(x), a.v_proj(x), self.k_caches[l], self.v_caches[l], a.n_heads, a.n_kv_heads,
                         a.head_dim, a.rope_theta, self.position, 0)
        q = q.view(B, a.n_heads, a.head_dim)
        ctx = torch.nn.functional.scaled_dot_product_attention(q.unsqueeze(2), self.k_caches[l], self.v_caches[l],
                                                               attn_mask=mask, enable_gqa=True)   # (B, heads, 1, head_dim)
        h.add_(a.o_proj(ctx.reshape(B, hidden)))
        self._x_moe[l] = rms_norm_rows(h, a.ln_post, a.rms_eps)
        self._routes[l] = layer.moe._router.route(self._x_moe[l])

    def _head_segment(self):
        self.h.add_(self.y)
        x = rms_norm_rows(self.h, self.model.layers[-1].next_ln, self.model.rms_eps)
        self._logits = torch.matmul(x, self.model.lm_head.t())

    def _experts(self, l: int):
        """The per-expert loop of SparseMoeWrapper.forward (custom_layers.py:295-312) into self.y."""
        moe = self.model.layers[l].moe
        E = moe.num_experts
        logits, _, _, meta, token_idx, token_w = self._routes[l]
        self._host_counts.copy_(meta, non_blocking=True)
        torch.cuda.current_stream(self.h.device).synchronize()
        host = self._host_counts.tolist()
        counts, offsets = host[:E], host[E:]
        for e in range(E):
            if counts[e] > 0:
                lo, hi = offsets[e], offsets[e + 1]
                moe._experts[e].forward_routed(self._x_moe[l], token_idx[lo:hi], token_w[lo:hi], self.y, accumulate=True)
        return logits

    # ---- a step -----------------------------------------------------------------------------------------------
    @torch.inference_mode()
    def capture(self) -> None:
        """Records the segments (call after at least one plain step at this batch size, so that the library's
        workspace has its size)."""
        dev = self.h.device
        tokens, pos = self.tokens.clone(), self.position.clone()
        caches = [(k[:, :, int(pos)].clone(), v[:, :, int(pos)].clone()) for k, v in zip(self.k_caches, self.v_caches)]
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self._run_eager()                                              # settles allocations on the capture stream
        torch.cuda.current_stream(dev).wait_stream(side)
        graphs, pool = [], None
        segments = [self._prologue] + [lambda l=l: self._attention_segment(l) for l in range(len(self.model.layers))] \
            + [self._head_segment]
        for seg in segments:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool):
                seg()
            pool = g.pool()
            graphs.append(g)
        self._graphs = graphs
        self.tokens.copy_(tokens)
        self.position.copy_(pos)
        for (k0, v0), k, v in zip(caches, self.k_caches, self.v_caches):   # the settling step wrote this row
            k[:, :, int(pos)], v[:, :, int(pos)] = k0, v0

    def _run_eager(self):
        self._prologue()
        self.router_logits = []
        for l in range(len(self.model.layers)):
            self._attention_segment(l)
            self.router_logits.append(self._experts(l))
        self._head_segment()

    def _run_graphs(self):
        g = self._graphs
        g[0].replay()
        self.router_logits = []
        for l in range(len(self.model.layers)):
            g[1 + l].replay()
            self.router_logits.append(self._experts(l))
        g[-1].replay()

    @torch.inference_mode()
    def step(self, tokens: torch.Tensor, pos: int) -> torch.Tensor:
        """tokens: (B,) int64 on the device, the token each sequence is fed at position pos.  Returns the logits
        (B, vocab) (a buffer that the next step overwrites); appends the tokens' keys and values to the caches."""
        if tokens.shape != (self.batch,) or not 0 <= pos < self.max_len:
            raise ValueError(f"step wants {self.batch} tokens and a position below {self.max_len}")
        self.tokens.copy_(tokens)
        self.position.fill_(pos)
        if self._graphs is not None:
            self._run_graphs()
        else:
            self._run_eager()
        return self._logits
