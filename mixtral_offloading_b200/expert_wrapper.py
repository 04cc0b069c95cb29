"""MixtralExpertWrapper: one contiguous slab per expert (src/expert_wrapper.py:9-85).

All tensors of the three quantized linears are moved into ONE UntypedStorage, in the
reference's order (nested_flatten: dictionary keys sorted at every level, i.e. per
layer W_q, meta.meta_scale.scale, meta.meta_scale.zero, meta.meta_zero.scale,
meta.meta_zero.zero, meta.scale_q, meta.zero_q; w1, w2, w3), and the layers are
re-pointed at views of it.  The slab is the unit of every host<->device copy.  Unlike
the reference, each tensor starts on a 256-byte boundary so that the kernels' 128-bit
loads are aligned for any shape.
"""
from __future__ import annotations

import typing as tp

import torch
from torch import nn

from .utils import nested_flatten

SLAB_ALIGN = 256


def slab_layout(state: dict):
    """[(tensor, offset)] in slab order and the slab size for a nested state dictionary."""
    offset, placed = 0, []
    for t in nested_flatten(state):
        if not isinstance(t, torch.Tensor):
            continue
        offset = (offset + SLAB_ALIGN - 1) // SLAB_ALIGN * SLAB_ALIGN
        placed.append((t, offset))
        offset += t.nbytes
    return placed, (offset + SLAB_ALIGN - 1) // SLAB_ALIGN * SLAB_ALIGN


class MixtralExpertWrapper(nn.Module):
    def __init__(self, expert_module: tp.Any, device: torch.device):
        super().__init__()
        expert_module, self.storage = self.replace_layer_storage(expert_module, device)
        # kept out of nn.Module's registry, as the reference does with a lambda
        # (expert_wrapper.py:18): the only state of a wrapper is its slab
        object.__setattr__(self, "_expert", expert_module)
        self.expert_module = lambda *args, **kwargs: expert_module(*args, **kwargs)
        self._register_state_dict_hook(self._add_storage_to_state_dict_hook)
        self._register_load_state_dict_pre_hook(self._load_storage_from_state_dict_hook)

    @staticmethod
    def _add_storage_to_state_dict_hook(self, state_dict, prefix, local_metadata):
        state_dict[prefix + "storage"] = torch.as_tensor(self.storage, dtype=torch.uint8)
        return state_dict

    def _load_storage_from_state_dict_hook(self, state_dict, prefix, local_metadata, strict, missing_keys,
                                           unexpected_keys, error_msgs):
        self.storage.copy_(state_dict[prefix + "storage"].untyped_storage())
        del state_dict[prefix + "storage"]

    def forward(self, *args, **kwargs):
        return self.expert_module(*args, **kwargs)

    def forward_routed(self, *args, **kwargs):
        return self._expert.forward_routed(*args, **kwargs)

    @staticmethod
    def replace_layer_storage(layer: tp.Any, device: torch.device):
        """expert_wrapper.py:41-85 with aligned sub-tensors."""
        state = {f"w{i}": {"W_q": getattr(layer, f"w{i}").W_q, "meta": getattr(layer, f"w{i}").meta,
                           "bias": getattr(layer, f"w{i}").bias} for i in range(1, 4)}
        placed, size = slab_layout(state)
        storage = torch.UntypedStorage(size, device=device)
        whole = torch.as_tensor(storage, dtype=torch.uint8, device=device)
        whole.zero_()
        views = {}
        for t, off in placed:
            view = whole[off:off + t.nbytes].view(t.dtype).view(t.shape)
            view.copy_(t)
            assert view.data_ptr() == storage.data_ptr() + off
            views[id(t)] = view

        def repoint(node):
            if isinstance(node, dict):
                return {k: repoint(v) for k, v in node.items()}
            if isinstance(node, torch.Tensor):
                return views[id(node)]
            return node

        for name, states in state.items():
            patched = getattr(layer, name)
            patched.W_q = views[id(states["W_q"])]
            patched.meta = repoint(states["meta"])
            patched.bias = None if states["bias"] is None else views[id(states["bias"])]
            patched._desc = None
        return layer, storage
