"""Expert-parallel MoE block: the experts of a layer sharded over the ranks of one node.

The reference has no distributed code; this is the multi-GPU form of its
SparseMoeWrapper.forward (src/custom_layers.py:272-314).  Attention and the router are
replicated, so every rank holds the same hidden states and computes the same routing:
dispatch needs no data movement (a rank simply runs the experts it owns on the rows
routed to them).  Only the combine is an exchange.  Two forms:

  "all_to_all"  token t is owned by rank t % R.  Each rank writes its experts' weighted
                outputs into a send buffer ordered by owner (the down-projection's
                epilogue writes those rows directly, there is no pack kernel), one
                all-to-all brings every owner the R partial rows of its tokens, the
                owner adds them, an all-gather restores the replica.
  "all_reduce"  one sum of the (tokens, hidden) partials; fewer launches, the better
                choice when there are fewer tokens than ranks (decode).

Both give the same numbers as the single-GPU block: a token has two non-zero
contributions, and a two-term bf16 sum does not depend on the order.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.distributed as dist
from torch import nn

from .custom_layers import SparseMoeWrapper, _as_bf16_2d


def expert_owner(expert: int, num_experts: int, world: int) -> int:
    """Rank holding an expert: contiguous blocks of num_experts / world experts per rank."""
    assert num_experts % world == 0, "the number of experts must be a multiple of the number of ranks"
    return expert // (num_experts // world)


def owner_layout(tokens: int, world: int):
    """Row permutation that groups tokens by owner (t % world): returns (rows per owner, perm) with
    perm[t] = row of token t in the (world, rows_per_owner) buffer."""
    per = (tokens + world - 1) // world
    t = torch.arange(tokens)
    return per, (t % world) * per + t // world


class ExpertParallelMoe(nn.Module):
    def __init__(self, config, layer_id, gate, local_experts: Dict[int, nn.Module], group=None,
                 combine: str = "all_to_all"):
        """local_experts maps expert index -> a module with forward_routed() (MixtralExpertWrapper or
        MixtralBLockSparseTop2MLP_HQQ) for the experts this rank owns."""
        super().__init__()
        assert combine in ("all_to_all", "all_reduce")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.combine = combine
        self.num_experts = config.num_local_experts
        self.hidden_dim = config.hidden_size
        self.layer_id = layer_id
        for e in local_experts:
            assert expert_owner(e, self.num_experts, self.world) == self.rank, f"expert {e} is not this rank's"
        self.local_experts = dict(local_experts)
        self.router = SparseMoeWrapper(config, layer_id, gate, expert_cache=None)
        self._host_counts = None
        self._perm_cache = {}

    # -- pieces the CPU tests override -------------------------------------------------------
    def route(self, x2d):
        """(logits, counts, offsets, token_idx, token_w) with counts/offsets as host lists."""
        E = self.num_experts
        logits, _, _, meta, token_idx, token_w = self.router.route(x2d)
        if self._host_counts is None:
            with torch.inference_mode(False):     # a normal tensor: it is written from any mode later
                self._host_counts = torch.empty((2 * E + 1,), dtype=torch.int32).pin_memory()
        self._host_counts.copy_(meta, non_blocking=True)
        torch.cuda.current_stream(x2d.device).synchronize()
        host = self._host_counts.tolist()
        return logits, host[:E], host[E:], token_idx, token_w

    def run_expert(self, e, x_rows, row_idx, row_w, out):
        """Rows row_idx of x_rows through local expert e, scaled by row_w, accumulated into the same rows of out."""
        self.local_experts[e].forward_routed(x_rows, row_idx, row_w, out, accumulate=True)

    # -- forward -----------------------------------------------------------------------------
    def _perm(self, tokens, device):
        key = (tokens, str(device))
        if key not in self._perm_cache:
            per, perm = owner_layout(tokens, self.world)
            self._perm_cache[key] = (per, perm.to(device), perm.to(device=device, dtype=torch.int32))
        return self._perm_cache[key]

    @torch.inference_mode()
    def forward(self, hidden_states: torch.Tensor):
        batch, seq, hidden = hidden_states.shape
        x2 = _as_bf16_2d(hidden_states, hidden) if hidden_states.is_cuda else hidden_states.reshape(-1, hidden)
        T, R = x2.shape[0], self.world
        logits, counts, offsets, token_idx, token_w = self.route(x2)
        mine = [e for e in sorted(self.local_experts) if counts[e] > 0]

        if self.combine == "all_reduce" or R == 1:
            partial = torch.zeros((T, hidden), dtype=x2.dtype, device=x2.device)
            for e in mine:
                lo, hi = offsets[e], offsets[e + 1]
                self.run_expert(e, x2, token_idx[lo:hi], token_w[lo:hi], partial)
            if R > 1:
                dist.all_reduce(partial, group=self.group)
            out = partial
        else:
            per, perm, perm32 = self._perm(T, x2.device)
            # rows ordered by owner: the send buffer of the all-to-all; x is laid out the same way so that
            # one index addresses both the gathered input row and the output row
            x_by_owner = torch.zeros((R * per, hidden), dtype=x2.dtype, device=x2.device)
            x_by_owner[perm] = x2
            send = torch.zeros((R * per, hidden), dtype=x2.dtype, device=x2.device)
            rows = perm32[token_idx.long()]
            for e in mine:
                lo, hi = offsets[e], offsets[e + 1]
                self.run_expert(e, x_by_owner, rows[lo:hi].contiguous(), token_w[lo:hi], send)
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=self.group)          # recv[q] = rank q's rows for my tokens
            owned = recv.view(R, per, hidden).sum(dim=0, dtype=torch.float32).to(x2.dtype)
            gathered = torch.empty((R * per, hidden), dtype=x2.dtype, device=x2.device)
            dist.all_gather_into_tensor(gathered, owned.contiguous(), group=self.group)
            out = gathered[perm]
        out = out.reshape(batch, seq, hidden)
        if hidden_states.dtype != out.dtype:
            out, logits = out.to(hidden_states.dtype), logits.to(hidden_states.dtype)
        return out, logits
