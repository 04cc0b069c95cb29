"""Helpers that define orderings the rest of the package relies on."""
from __future__ import annotations


import torch


def nested_flatten(t):
    """Depth-first leaves of nested lists / tuples / dicts, dict entries by sorted key.

    This is the order in which the reference lays an expert's tensors into its slab
    (src/utils.py:34-45 as used by src/expert_wrapper.py:52-66)."""
    if isinstance(t, (list, tuple)):
        for item in t:
            yield from nested_flatten(item)
    elif isinstance(t, dict):
        for key in sorted(t):
            yield from nested_flatten(t[key])
    else:
        yield t
